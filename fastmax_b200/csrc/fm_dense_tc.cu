// Fastmax attention in tiled score form on the tcgen05 tensor cores (bf16 inputs,
// fp32 accumulation in tensor memory), head dimension 64 or 128.
//
// Two kernel modes cover the forward pass and the three gradients:
//
//   OP_A   out_r = sum_c f(x_r . y_c) z_c                       (forward, grad_v)
//   OP_B   out_r = sum_c f'(x_r . y_c) (u_r . z_c - dvec) y_c   (grad_q, grad_k)
//
// r runs over the rows a CTA owns, c over column tiles; "forward direction"
// keeps c <= r + off (causal), "reverse direction" keeps c >= r - off.  With
//   forward: x=q  y=k  z=v                    grad_q: x=q u=gs y=k z=v  dvec per row
//   grad_v : x=k  y=q  z=gs  (reverse)        grad_k: x=k u=v  y=q z=gs dvec per column
// where gs_i = grad_out_i / den_i and dvec_i = (grad_out_i . out_i) / den_i, these are
// the sums the reference evaluates through running moments (see fm_dense_ffma.cu).
//
// These kernels serve the forward pass at head dimension 128 and, with
// FASTMAX_B200_NO_WIDE=1, everything else; the default d = 64 kernels and the d = 128
// backward are in fm_dense_tc_wide.cu and fm_dense_tc_dkdv128.cu.
//
// One CTA owns two 128-row tiles (two "groups" of four warps each, one row per
// thread) and streams column tiles through a shared-memory ring filled by TMA.
// One issuer warp per group issues the group's tcgen05.mma (the whole warp runs the
// loop, an elected lane issues); per column tile and group:
//   S = X Y^T (and W = U Z^T)            smem x smem  -> TMEM
//   the group's warps read S (W) from TMEM, apply the polynomial and the mask and
//   write the bf16 result P back to TMEM
//   O += P Z   (or P Y)                  TMEM x smem  -> TMEM accumulator
// A group copies its whole S (W) row block to registers and hands the TMEM region
// back at once, so its issuer can start the next tile's S while the group is still
// computing; the tensor pipe therefore runs ahead of the CUDA cores of both groups.
// The polynomial is evaluated on packed fp32 pairs.  All waits are bounded; a wait
// that gives up records an error status and the kernel winds down without hanging.
#include <climits>

#include "fm_common.cuh"
#include "fm_sm100.cuh"

namespace fm {

__device__ int g_tc_status = 0;  // first protocol error seen by any tensor-core kernel

namespace {
using namespace sm100;

enum { OP_A = 0, OP_B = 1 };

struct TcArgs {
  void* o;              // (heads, nrows, d) bf16 result rows
  float* den_out;       // OP_A with fwd_div: (heads, nrows) row sums
  const float* dvec;    // OP_B: (heads, nq) grad_out.out / den
  const void* x;        // row operand in global memory (for the normalisation dots)
  float* dots;          // OP_B: per head sum of o . x  (null when not normalised)
  const stat_t* stat_q;
  const stat_t* stat_k;
  int nrows, ncols, off, mask, rev, fwd_div, npairs;
  float a0, a1, a2, lim;
  int ratio;             // query heads per key/value head (forward-direction modes only)
  int chunk;             // > 0: only the columns of the row pair's own chunk
  const float* o_add;    // fp32 (heads, nrows, d) added to the accumulator row
  const float* den_add;  // OP_A with fwd_div: added to the row sum
  int o_heads;           // OP_A with fwd_div: > 0 writes out as (batch, nrows, o_heads, d)
};

constexpr int BM = 128;
constexpr int kThreads = 352;  // warps 0-3: group 0, 4-7: group 1, 8: TMA producer, 9/10: MMA issuers

// Tiling per mode and head dimension DD (64 or 128).  Tiles of 128-byte-swizzled rows hold
// 64 bf16 per row, so a DD = 128 tile is two sub-tiles side by side.  TMEM columns per
// group (stride 256): S | W | P | O.  DD = 128 needs 128 columns for O, so OP_A shrinks
// the column tile to 64 and OP_B runs a single group per CTA.
template <int MODE, int DD>
struct Cfg {
  static constexpr int D = DD;
  static constexpr int NSUB = DD / 64;
  static constexpr int BN = (MODE == OP_A && DD == 64) ? 128 : 64;
  static constexpr int NG = (MODE == OP_B && DD == 128) ? 1 : 2;
  static constexpr int NS = (DD == 128) ? 3 : ((MODE == OP_A) ? 4 : 6);
  static constexpr int ROW_SUB = BM * 128;          // one 64-wide sub-tile of a row tile
  static constexpr int COL_SUB = BN * 128;
  static constexpr int ROW_TILE = NSUB * ROW_SUB;
  static constexpr int COL_TILE = NSUB * COL_SUB;
  static constexpr int NROWOPS = (MODE == OP_A) ? 1 : 2;
  static constexpr int STAGE = 2 * COL_TILE;
  static constexpr int OFF_X = 0;
  static constexpr int OFF_U = NG * ROW_TILE;
  static constexpr int OFF_ST = NROWOPS * NG * ROW_TILE;
  static constexpr int OFF_VEC = OFF_ST + NS * STAGE;
  static constexpr int OFF_BAR = OFF_VEC + NS * BN * 4;
  static constexpr int NBAR = 1 + 2 * NS + 8;
  static constexpr int OFF_TMEM = OFF_BAR + NBAR * 8;
  static constexpr int SMEM = OFF_TMEM + 16 + 1024;  // + slack for the 1024-byte alignment
  static constexpr int T_S = 0, T_W = 64;
  static constexpr int T_P = (DD == 64) ? 128 : ((MODE == OP_A) ? 64 : 128);
  static constexpr int T_O = (DD == 64) ? 192 : ((MODE == OP_A) ? 96 : 192);
};

__device__ __forceinline__ void report(int code) { atomicCAS(&g_tc_status, 0, code); }

template <int MODE, int DD>
__global__ void __launch_bounds__(kThreads, 1)
dense_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmU,
                const __grid_constant__ CUtensorMap tmY, const __grid_constant__ CUtensorMap tmZ,
                const TcArgs a) {
  using C = Cfg<MODE, DD>;
  constexpr int BN = C::BN, NS = C::NS, D = DD;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::OFF_BAR;
  // barrier map: x | kv_full[NS] | kv_empty[NS] | s_full[2] | s_free[2] | p_full[2] | pv_done[2]
  auto BAR_X = [&]() { return bar0; };
  auto BAR_FULL = [&](int s) { return bar0 + 8u * (1 + s); };
  auto BAR_EMPTY = [&](int s) { return bar0 + 8u * (1 + NS + s); };
  auto BAR_S = [&](int g) { return bar0 + 8u * (1 + 2 * NS + g); };
  auto BAR_SFREE = [&](int g) { return bar0 + 8u * (3 + 2 * NS + g); };
  auto BAR_P = [&](int g) { return bar0 + 8u * (5 + 2 * NS + g); };
  auto BAR_PV = [&](int g) { return bar0 + 8u * (7 + 2 * NS + g); };
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem + C::OFF_TMEM);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // consecutive CTAs work on the same head, so its K/V (or Q/G) tiles stay in L2 while the
  // row tiles that share them are in flight; causal row pairs are issued longest first
  const int head = blockIdx.x / a.npairs;
  const int pidx = blockIdx.x % a.npairs;
  const int pair = a.rev ? pidx : a.npairs - 1 - pidx;
  const int r0 = pair * C::NG * BM;
  const bool colvec = (MODE == OP_B) && a.rev;

  // ---- tile ranges: group g walks column tiles [tb_g, te_g) -------------------------
  const int ntile = (a.ncols + BN - 1) / BN;
  int tb0 = 0, te0 = ntile, tb1 = 0, te1 = ntile;
  if (a.mask) {
    if (a.rev) {
      tb0 = max(0, r0 - a.off) / BN;
      tb1 = max(0, r0 + BM - a.off) / BN;
    } else {
      te0 = min(ntile, (min(r0 + BM - 1, a.nrows - 1) + a.off) / BN + 1);
      te1 = min(ntile, (min(r0 + 2 * BM - 1, a.nrows - 1) + a.off) / BN + 1);
    }
  }
  if (a.chunk > 0) {  // both row tiles lie in one chunk (chunk % 256 == 0)
    const int cb = (r0 / a.chunk) * (a.chunk / BN), ce = cb + a.chunk / BN;
    if (a.rev) { te0 = min(te0, ce); te1 = min(te1, ce); }
    else { tb0 = cb; tb1 = cb; }
  }
  const bool act1 = C::NG == 2 && r0 + BM < a.nrows;  // group 0 always has rows
  if (!act1) { tb1 = INT_MAX; te1 = 0; }
  const int tb = min(tb0, tb1);
  const int te = max(te0, te1);

  // ---- set-up -----------------------------------------------------------------------
  if (tid == 0) {
    mbar_init(BAR_X(), 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(BAR_FULL(s), colvec ? 33 : 1);
      mbar_init(BAR_EMPTY(s), 2);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(BAR_S(g), 1);
      mbar_init(BAR_SFREE(g), 4);
      mbar_init(BAR_P(g), 4);
      mbar_init(BAR_PV(g), 1);
    }
    mbar_fence_init();
  }
  if (warp == 9) tmem_alloc(smem_u32((const void*)tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 8) {
    // ================= TMA producer =================
    if (lane == 0) {
      tma_prefetch_desc(&tmX);
      tma_prefetch_desc(&tmY);
      tma_prefetch_desc(&tmZ);
      if (MODE == OP_B) tma_prefetch_desc(&tmU);
      mbar_expect_tx(BAR_X(), (act1 ? 2 : 1) * C::NROWOPS * C::ROW_TILE);
      for (int g = 0; g < (act1 ? 2 : 1); ++g)
        for (int sub = 0; sub < C::NSUB; ++sub) {
          tma_load_3d(sbase + C::OFF_X + g * C::ROW_TILE + sub * C::ROW_SUB, &tmX, BAR_X(), sub * 64,
                      r0 + g * BM, head);
          if (MODE == OP_B)
            tma_load_3d(sbase + C::OFF_U + g * C::ROW_TILE + sub * C::ROW_SUB, &tmU, BAR_X(), sub * 64,
                        r0 + g * BM, head);
        }
    }
    for (int t = tb; t < te; ++t) {
      const int k = t - tb, s = k % NS;
      if (!mbar_wait(BAR_EMPTY(s), (((k / NS) & 1) ^ 1))) { report(1); break; }
      if (lane == 0) {
        mbar_expect_tx(BAR_FULL(s), C::STAGE);
        const uint32_t dst = sbase + C::OFF_ST + s * C::STAGE;
        for (int sub = 0; sub < C::NSUB; ++sub) {
          tma_load_3d(dst + sub * C::COL_SUB, &tmY, BAR_FULL(s), sub * 64, t * BN, head / a.ratio);
          tma_load_3d(dst + C::COL_TILE + sub * C::COL_SUB, &tmZ, BAR_FULL(s), sub * 64, t * BN, head / a.ratio);
        }
      }
      if (colvec) {
        float* vec = (float*)(smem + C::OFF_VEC) + s * BN;
        for (int e = lane; e < BN; e += 32) {
          const int col = t * BN + e;
          vec[e] = (col < a.ncols) ? -__ldg(a.dvec + (size_t)head * a.ncols + col) : 0.f;  // negated
        }
        mbar_arrive(BAR_FULL(s));
      }
    }
  } else if (warp >= 9) {
    // ================= MMA issuers: warp 9 serves group 0, warp 10 group 1 =================
    const int g = warp - 9;
    const int tbg = g ? tb1 : tb0, teg = g ? te1 : te0;
    const int J = (g == 0 || act1) ? teg - tbg : 0;
    // the whole warp runs the loop (uniform control flow and operands); one elected lane
    // executes the tcgen05 instructions
    if (J > 0) {
      constexpr uint32_t idescS = idesc_bf16(BM, BN, 0, 0);
      constexpr uint32_t idescO = idesc_bf16(BM, D, 0, 1);
      static_assert(C::T_O + D <= 256 || C::NG == 1, "accumulator does not fit the group's TMEM columns");
      const uint32_t tg = tmem + g * 256;
      const uint32_t x_lo = desc_lo(sbase + C::OFF_X + g * C::ROW_TILE, 16);
      const uint32_t u_lo = desc_lo(sbase + C::OFF_U + g * C::ROW_TILE, 16);
      const uint32_t st_k = desc_lo(sbase + C::OFF_ST, 16);               // stage 0, K-major view
      const uint32_t st_mn = desc_lo(sbase + C::OFF_ST, C::COL_SUB);      // stage 0, MN-major view
      // the other group also reads tile t unless t is outside its range
      const int otb = g ? tb0 : tb1, ote = g ? te0 : te1;
      bool ok = mbar_wait_warp(BAR_X(), 0);
      if (!ok) report(2);
      tc_fence_after();
      auto issue_S = [&](int t) -> bool {
        const int k = t - tb, s = k % NS;
        if (!mbar_wait_warp(BAR_FULL(s), (uint32_t)((k / NS) & 1))) { report(3); return false; }
        tc_fence_after();
        const uint32_t y_lo = st_k + (uint32_t)s * (C::STAGE >> 4);
        if (elect_one()) {
#pragma unroll
          for (int sub = 0; sub < C::NSUB; ++sub)
            umma_ss_k64(tg + C::T_S, x_lo + sub * (C::ROW_SUB >> 4), y_lo + sub * (C::COL_SUB >> 4), idescS, sub > 0);
          if (MODE == OP_B) {
#pragma unroll
            for (int sub = 0; sub < C::NSUB; ++sub)
              umma_ss_k64(tg + C::T_W, u_lo + sub * (C::ROW_SUB >> 4),
                          y_lo + (C::COL_TILE >> 4) + sub * (C::COL_SUB >> 4), idescS, sub > 0);
          }
          umma_commit(BAR_S(g));
        }
        __syncwarp();
        return true;
      };
      if (ok) ok = issue_S(tbg);
      for (int j = 0; ok && j < J; ++j) {
        const int t = tbg + j;
        if (j + 1 < J) {
          if (!mbar_wait_warp(BAR_SFREE(g), (uint32_t)(j & 1))) { report(4); ok = false; break; }
          if (!issue_S(t + 1)) { ok = false; break; }
        }
        if (!mbar_wait_warp(BAR_P(g), (uint32_t)(j & 1))) { report(5); ok = false; break; }
        tc_fence_after();
        const int s = (t - tb) % NS;
        // OP_A multiplies by the Z tile (second half of the stage), OP_B by the Y tile
        const uint32_t b_lo = st_mn + (uint32_t)s * (C::STAGE >> 4) + ((MODE == OP_A) ? (C::COL_TILE >> 4) : 0);
        if (elect_one()) {
          umma_ts_steps<BN / 16>(tg + C::T_O, tg + C::T_P, b_lo, idescO, j > 0 ? 1u : 0u);
          umma_commit(BAR_PV(g));
          // the ring stage is free once both groups' MMAs on it are done (2 arrivals)
          umma_commit(BAR_EMPTY(s));
          if (t < otb || t >= ote) umma_commit(BAR_EMPTY(s));
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else {
    // ================= compute groups =================
    const int g = warp >> 2, qd = warp & 3;
    const int tbg = g ? tb1 : tb0, teg = g ? te1 : te0;
    if (g == 0 || act1) {
      const int row = r0 + g * BM + qd * 32 + lane;
      const bool row_ok = row < a.nrows;
      const float c = stat_scale(a.stat_q, head, a.lim) * stat_scale(a.stat_k, head / a.ratio, a.lim);
      const float A0 = a.a0, A1 = a.a1 * c, A2 = a.a2 * c * c;
      const uint64_t A0v = pack2(A0, A0), A1v = pack2(A1, A1);
      const uint64_t A2v = (MODE == OP_A) ? pack2(A2, A2) : pack2(2.f * A2, 2.f * A2);
      // columns kept for this row: lowcol <= col <= limcol
      int limcol = a.ncols - 1, lowcol = 0;
      if (a.mask) {
        if (a.rev) lowcol = row - a.off;
        else limcol = min(limcol, row + a.off);
      }
      const int wrow_lo = r0 + g * BM + qd * 32, wrow_hi = wrow_lo + 31;
      float dl_row = 0.f;
      if (MODE == OP_B && !a.rev && row_ok) dl_row = __ldg(a.dvec + (size_t)head * a.nrows + row);
      const uint64_t ndl_row = pack2(-dl_row, -dl_row);
      const uint32_t tg = tmem + g * 256 + ((uint32_t)(qd * 32) << 16);
      uint64_t rs2[4] = {pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f)};
      bool ok = true;
      for (int t = tbg; t < teg; ++t) {
        const int j = t - tbg;
        if (!mbar_wait(BAR_S(g), (uint32_t)(j & 1))) { report(7); ok = false; break; }
        tc_fence_after();
        // the whole tile row goes to registers, then the TMEM region is handed back
        uint32_t sv[BN];
        uint32_t wv[(MODE == OP_B) ? BN : 1];
        tmem_ld64(tg + C::T_S, sv);
        if constexpr (MODE == OP_A) tmem_ld64(tg + C::T_S + 64, sv + 64);
        else tmem_ld64(tg + C::T_W, wv);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR_SFREE(g));
        const float* vec = nullptr;
        if (colvec) {
          const int k = t - tb, s = k % NS;
          if (!mbar_wait(BAR_FULL(s), (uint32_t)((k / NS) & 1))) { report(8); ok = false; break; }
          vec = (const float*)(smem + C::OFF_VEC) + s * BN;
        }
        const int c0 = t * BN;
        bool need_mask = (c0 + BN > a.ncols);
        if (a.mask) need_mask = need_mask || (a.rev ? (c0 < wrow_hi - a.off) : (c0 + BN - 1 > wrow_lo + a.off));
        uint32_t pk[BN / 2];
        if (!need_mask) {
#pragma unroll
          for (int e = 0; e < BN / 2; ++e) {
            const uint64_t s2 = pack2u(sv[2 * e], sv[2 * e + 1]);
            uint64_t p2;
            if (MODE == OP_A) {
              p2 = fma2(fma2(A2v, s2, A1v), s2, A0v);
              rs2[e & 3] = add2(rs2[e & 3], p2);
            } else {
              const uint64_t ndl = a.rev ? ((const uint64_t*)vec)[e] : ndl_row;
              p2 = mul2(fma2(A2v, s2, A1v), add2(pack2u(wv[2 * e], wv[2 * e + 1]), ndl));
            }
            pk[e] = pack_bf16_2(p2);
          }
        } else {
#pragma unroll
          for (int e = 0; e < BN / 2; ++e) {
            float pv[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int col = c0 + 2 * e + h;
              const float s = __uint_as_float(sv[2 * e + h]);
              float v;
              if (MODE == OP_A) {
                v = fmaf(fmaf(A2, s, A1), s, A0);
              } else {
                const float dl = a.rev ? -vec[2 * e + h] : dl_row;
                v = fmaf(2.f * A2, s, A1) * (__uint_as_float(wv[2 * e + h]) - dl);
              }
              pv[h] = (col > limcol || col < lowcol) ? 0.f : v;
            }
            pk[e] = pack_bf16(pv[0], pv[1]);
            // Tiles on the causal diagonal (and ragged last tiles) hold most of what an early row sees, so
            // their share of the row sum is taken from the ROUNDED values the product will use: numerator
            // and denominator then carry the same rounding, and a row with one key returns its value exactly.
            if (MODE == OP_A)
              rs2[e & 3] = add2(rs2[e & 3], pack2(__uint_as_float(pk[e] << 16), __uint_as_float(pk[e] & 0xFFFF0000u)));
          }
        }
        // P(t-1) must have been consumed by its MMA before it is overwritten
        if (j > 0 && !mbar_wait(BAR_PV(g), (uint32_t)((j - 1) & 1))) { report(9); ok = false; break; }
        tc_fence_after();
        tmem_st32(tg + C::T_P, pk);
        if constexpr (BN == 128) tmem_st32(tg + C::T_P + 32, pk + 32);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR_P(g));
      }
      // ---- epilogue: this thread's row of the accumulator -> global ----
      const int Jg = teg - tbg;
      if (ok && Jg > 0) {
        if (!mbar_wait(BAR_PV(g), (uint32_t)((Jg - 1) & 1))) { report(10); ok = false; }
      }
      tc_fence_after();
      if (ok && Jg > 0) {
        float rlo, rhi;
        unpack2(add2(add2(rs2[0], rs2[1]), add2(rs2[2], rs2[3])), rlo, rhi);
        float rowsum = rlo + rhi;
        if (MODE == OP_A && a.fwd_div && a.den_add && row_ok) rowsum += a.den_add[(size_t)head * a.nrows + row];
        float scale = 1.f;
        if (MODE == OP_A && a.fwd_div) scale = 1.0f / rowsum;
        float part = 0.f;
        const size_t grow = (size_t)head * a.nrows + (row_ok ? row : 0);
        const bool want_dots = (MODE == OP_B) && a.dots != nullptr;
#pragma unroll 1
        for (int hc = 0; hc < D / 64; ++hc) {      // 64 accumulator columns at a time
          uint32_t ov[64];
          tmem_ld64(tg + C::T_O + hc * 64, ov);
          tmem_wait_ld();
          if (row_ok) {
            const size_t orow = (MODE == OP_A && a.fwd_div) ? out_row(head, row, a.nrows, a.o_heads) : grow;
            uint4* dst = (uint4*)((__nv_bfloat16*)a.o + orow * D + hc * 64);
            const uint4* xr = (const uint4*)((const __nv_bfloat16*)a.x + grow * D + hc * 64);
            const float4* addr = a.o_add ? (const float4*)(a.o_add + grow * D + hc * 64) : nullptr;
#pragma unroll
            for (int v8 = 0; v8 < 8; ++v8) {
              float f[8];
              float4 ad0 = make_float4(0.f, 0.f, 0.f, 0.f), ad1 = ad0;
              if (addr) { ad0 = __ldg(addr + 2 * v8); ad1 = __ldg(addr + 2 * v8 + 1); }
              const float ad[8] = {ad0.x, ad0.y, ad0.z, ad0.w, ad1.x, ad1.y, ad1.z, ad1.w};
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = (__uint_as_float(ov[v8 * 8 + e]) + ad[e]) * scale;
              uint4 w;
              w.x = pack_bf16(f[0], f[1]); w.y = pack_bf16(f[2], f[3]);
              w.z = pack_bf16(f[4], f[5]); w.w = pack_bf16(f[6], f[7]);
              dst[v8] = w;
              if (want_dots) {
                const uint4 xv = __ldg(xr + v8);
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  part = fmaf(f[2 * e], __uint_as_float(xw[e] << 16), part);
                  part = fmaf(f[2 * e + 1], __uint_as_float(xw[e] & 0xFFFF0000u), part);
                }
              }
            }
          }
        }
        if (MODE == OP_A && a.fwd_div && row_ok) a.den_out[grow] = rowsum;
        if (MODE == OP_B && a.dots != nullptr) {
#pragma unroll
          for (int m = 16; m >= 1; m >>= 1) part += __shfl_xor_sync(0xffffffffu, part, m);
          if (lane == 0) atomicAdd(a.dots + head, part);
        }
      }
    }
  }

  // ---- teardown ------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ---- host side ---------------------------------------------------------------------------
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                             CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                             CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (EncodeFn)p;
  }();
  return fn;
}

// (heads, n, d) bf16 tensor as a rank-3 map with boxes of box_rows x 64, 128-byte swizzle;
// rows past n read as zero.
int make_map(CUtensorMap* m, const void* base, int heads, int n, int box_rows, int d) {
  EncodeFn enc = encode_fn();
  if (!enc) return fail(FASTMAX_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[3] = {(cuuint64_t)d, (cuuint64_t)n, (cuuint64_t)heads};
  cuuint64_t gstr[2] = {(cuuint64_t)d * 2, (cuuint64_t)n * d * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};   // 64 elements = one 128-byte swizzle row
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FASTMAX_E_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return FASTMAX_OK;
}

}  // namespace

int tma_map_bf16(CUtensorMap* m, const void* base, size_t mats, size_t rows, int d, int box_rows) {
  EncodeFn enc = encode_fn();
  if (!enc) return fail(FASTMAX_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[3] = {(cuuint64_t)d, (cuuint64_t)rows, (cuuint64_t)mats};
  cuuint64_t gstr[2] = {(cuuint64_t)d * 2, (cuuint64_t)rows * d * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FASTMAX_E_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return FASTMAX_OK;
}

namespace {

template <int MODE, int DD>
int launch_tc_d(const Ctx& c, const char* name, const void* x, const void* u, const void* y,
                const void* z, int nrows, int ncols, TcArgs a) {
  using C = Cfg<MODE, DD>;
  const int heads = c.p.bh;
  if (heads == 0 || nrows == 0) return FASTMAX_OK;
  CUtensorMap tx, tu, ty, tz;
  int rc;
  if ((rc = make_map(&tx, x, heads, nrows, BM, DD))) return rc;
  if ((rc = make_map(&tu, u ? u : x, heads, nrows, BM, DD))) return rc;
  // grouped k/v heads reach this launcher only in the forward direction (rows = query heads)
  const int col_heads = a.rev ? heads : c.p.bhkv;
  a.ratio = a.rev ? 1 : c.p.bh / c.p.bhkv;
  if ((rc = make_map(&ty, y, col_heads, ncols, C::BN, DD))) return rc;
  if ((rc = make_map(&tz, z, col_heads, ncols, C::BN, DD))) return rc;
  a.nrows = nrows;
  a.ncols = ncols;
  a.x = x;
  FM_CUDA_TRY(cudaFuncSetAttribute(dense_tc_kernel<MODE, DD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   C::SMEM));
  a.npairs = (nrows + C::NG * BM - 1) / (C::NG * BM);
  dim3 grid((unsigned)((size_t)heads * a.npairs));
  FM_LAUNCH(name, c.stream,
            (dense_tc_kernel<MODE, DD><<<grid, kThreads, C::SMEM, c.stream>>>(tx, tu, ty, tz, a)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

template <int MODE>
int launch_tc(const Ctx& c, const char* name, const void* x, const void* u, const void* y,
              const void* z, int nrows, int ncols, const TcArgs& a) {
  if (c.p.d == 128) return launch_tc_d<MODE, 128>(c, name, x, u, y, z, nrows, ncols, a);
  return launch_tc_d<MODE, 64>(c, name, x, u, y, z, nrows, ncols, a);
}

TcArgs base_args(const Ctx& c, const stat_t* stats) {
  const fastmax_problem& p = c.p;
  TcArgs a = {};
  a.stat_q = p.normalize ? stats : nullptr;
  a.stat_k = p.normalize ? stats + p.bh : nullptr;
  a.off = p.nk - p.nq;
  a.mask = p.mask;
  a.a0 = p.a0;
  a.a1 = p.a1;
  a.a2 = (p.p == 2) ? p.a2 : 0.f;
  a.lim = p.lim;
  return a;
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

bool dense_tc_supports(const fastmax_problem& p) {
  if (p.dtype != FASTMAX_BF16) return false;
  if ((p.d == 64 || p.d == 128) && p.bh == p.bhkv) return true;
  // grouped k/v heads: the kernels that walk a key/value head's tiles once per query head
  return dense_tc_wide_supports(p) || dense_tc_dkdv128_supports(p);
}

int dense_tc_forward(const Ctx& c, const void* q, const void* k, const void* v,
                     const stat_t* stats, void* out, float* den, const ChunkAdd* ca) {
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out))
    return fail(FASTMAX_E_ARG, "the tensor-core family needs 16-byte aligned tensors");
  if (dense_tc_wide_supports(c.p)) return dense_tc_wide_forward(c, q, k, v, stats, out, den, ca);
  TcArgs a = base_args(c, stats);
  a.o = out;
  a.den_out = den;
  a.fwd_div = 1;
  a.rev = 0;
  a.o_heads = c.out_heads;
  if (ca) { a.chunk = ca->chunk; a.o_add = ca->out_add; a.den_add = ca->den_add; }
  return launch_tc<OP_A>(c, "fm_dense_tc_fwd", q, nullptr, k, v, c.p.nq, c.p.nk, a);
}

int dense_tc_backward(const Ctx& c, const void* q, const void* k, const void* v, const void* gs,
                      const float* dvec, const stat_t* stats, float* dots, void* grad_q,
                      void* grad_k, void* grad_v, const ChunkAdd* ca) {
  const fastmax_problem& p = c.p;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(gs) || !aligned16(grad_q) ||
      !aligned16(grad_k) || !aligned16(grad_v))
    return fail(FASTMAX_E_ARG, "the tensor-core family needs 16-byte aligned tensors");
  if (dense_tc_wide_supports(p))
    return dense_tc_wide_backward(c, q, k, v, gs, dvec, stats, dots, grad_q, grad_k, grad_v, ca);
  if (dense_tc_dkdv128_supports(p))
    return dense_tc_backward128(c, q, k, v, gs, dvec, stats, dots, grad_q, grad_k, grad_v, ca);
  int rc;
  TcArgs a = base_args(c, stats);
  a.dvec = dvec;
  // grad_q: rows = queries, columns = keys
  a.o = grad_q;
  a.rev = 0;
  a.dots = p.normalize ? dots : nullptr;
  if (ca) { a.chunk = ca->chunk; a.o_add = ca->gq_add; }
  if ((rc = launch_tc<OP_B>(c, "fm_dense_tc_dq", q, gs, k, v, p.nq, p.nk, a))) return rc;
  // grad_k: rows = keys, columns = queries
  a.o = grad_k;
  a.rev = 1;
  a.dots = p.normalize ? dots + p.bh : nullptr;
  if (ca) a.o_add = ca->gk_add;
  if ((rc = launch_tc<OP_B>(c, "fm_dense_tc_dk", k, v, q, gs, p.nk, p.nq, a))) return rc;
  // grad_v: rows = keys, columns = queries, plain sum
  a.o = grad_v;
  a.dots = nullptr;
  a.fwd_div = 0;
  if (ca) a.o_add = ca->gv_add;
  return launch_tc<OP_A>(c, "fm_dense_tc_dv", k, nullptr, q, gs, p.nk, p.nq, a);
}

// One warp waits on a barrier that nobody ever arrives at, with the same bounded wait the
// kernels above use but a caller-chosen limit; when the wait gives up it records code 99 and
// the kernel returns.  This is how the give-up path is exercised without breaking a real
// kernel's protocol.
__global__ void wait_selftest_kernel(long long limit_clocks) {
  __shared__ __align__(8) unsigned long long bar;
  const uint32_t b = sm100::smem_u32(&bar);
  if (threadIdx.x == 0) {
    sm100::mbar_init(b, 1);
    sm100::mbar_fence_init();
  }
  __syncwarp();
  if (!sm100::mbar_wait_limit(b, 0, limit_clocks)) {
    if (threadIdx.x == 0) atomicCAS(&g_tc_status, 0, 99);
  }
}

int tc_wait_selftest(long long limit_clocks, cudaStream_t stream) {
  if (limit_clocks < 0 || limit_clocks > sm100::kWaitLimitClocks)
    return fail(FASTMAX_E_ARG, "limit_clocks must lie in [0, %lld]", sm100::kWaitLimitClocks);
  FM_LAUNCH("fm_wait_selftest", stream, (wait_selftest_kernel<<<1, 32, 0, stream>>>(limit_clocks)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

int tc_status(int* out, cudaStream_t stream) {
  FM_CUDA_TRY(cudaMemcpyFromSymbolAsync(out, g_tc_status, sizeof(int), 0, cudaMemcpyDeviceToHost, stream));
  FM_CUDA_TRY(cudaStreamSynchronize(stream));
  return FASTMAX_OK;
}
int tc_status_reset(cudaStream_t stream) {
  const int zero = 0;
  FM_CUDA_TRY(cudaMemcpyToSymbolAsync(g_tc_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream));
  FM_CUDA_TRY(cudaStreamSynchronize(stream));
  return FASTMAX_OK;
}

}  // namespace fm
