// Backward of the score form for head dimension 128 (bf16, tcgen05).
//   FUSED = 1  grad_k and grad_v in one pass: rows = keys (x = k, u = v), columns = queries
//              (y = q, z = gs), reverse direction (column >= row - off):
//                S = X Y^T, W = U Z^T,  E = f'(S) (W - dvec_col),  P = f(S),
//                grad_k += E Y,  grad_v += P Z.
//              Sharing S between the two gradients makes a 128 x 64 tile cost 24 + 8 MMA
//              instructions instead of the 40 + 8 of separate grad_k and grad_v kernels.
//   FUSED = 0  grad_q: rows = queries (x = q, u = gs), columns = keys (y = k, z = v), forward
//              direction:  E = f'(S) (W - dvec_row),  grad_q += E Y.
//
// One CTA owns one 128-row tile.  Two 128-column fp32 accumulators take 256 of the 512 TMEM
// columns, so S, W (64 columns each) and E, P (32 each, bf16 pairs) are single-buffered:
//   S 0..63 | W 64..127 | E 128..159 | P 160..191 | grad_k 192..319 | grad_v 320..447
// (grad_q, 128-column tiles: S 0..127 | W 128..255 | E 256..319 | grad_q 320..447).
// Warps 0-7 compute (warp % 4 = TMEM lane quarter = 32 rows, warp / 4 = which 32 of the 64
// columns), warp 8 is the TMA producer, warp 9 allocates TMEM and issues the S / W products
// (as soon as the compute warps have copied the previous tile to registers), warp 10 issues
// the accumulating products.  All waits are bounded; a wait that gives up records a status
// and the CTA winds down.
#include <climits>
#include <cstdlib>

#include "fm_common.cuh"
#include "fm_sm100.cuh"

namespace fm {

__device__ int g_ktc_status = 0;

namespace {
using namespace sm100;

struct KArgs {
  void* gk;              // (heads, nrows, 128) bf16: grad_k, or grad_q when not FUSED
  void* gv;
  const float* gk_add;   // fp32 rows added before rounding (may be null)
  const float* gv_add;
  const void* x;         // row operand in global memory (normalisation dot)
  const float* dvec;     // (heads, ncols)
  float* dots;           // per head sum of gk . x, or null
  const stat_t* stat_q;
  const stat_t* stat_k;
  int nrows, ncols, off, mask, ntr, chunk;
  int ratio;             // query heads per key/value head (grouped k/v heads)
  float a0, a1, a2, lim;
};

constexpr int BM = 128, D = 128;
constexpr int kThreads = 352, kComputeWarps = 8, kProducerWarp = 8, kIssuerWarp = 9, kAccIssuerWarp = 10;
constexpr int ROW_SUB = BM * 128, ROW_TILE = 2 * ROW_SUB;   // a row tile is two 64-wide sub-tiles
constexpr int OFF_X = 0, OFF_U = ROW_TILE, OFF_ST = 2 * ROW_TILE;
// The fused kernel needs two 128-column accumulators and stays at 64-column tiles; grad_q has
// room for 128-column tiles, whose S / W products are not bound by the shared-memory port.
template <bool FUSED>
struct KCfg {
  static constexpr int BN = FUSED ? 64 : 128;
  static constexpr int NS = FUSED ? 4 : 2;
  static constexpr int COL_SUB = BN * 128, COL_TILE = 2 * COL_SUB, STAGE = 2 * COL_TILE;
  static constexpr int OFF_VEC = OFF_ST + NS * STAGE;       // per compute warp 2 x 32 floats
  static constexpr int OFF_BAR = OFF_VEC + kComputeWarps * 2 * 32 * 4;
  static constexpr int NBAR = 2 + 2 * NS + 4;
  static constexpr int OFF_TMEM = OFF_BAR + NBAR * 8;
  static constexpr int SMEM = OFF_TMEM + 16 + 1024;
  // TMEM columns: S | W | E (| P) | accumulator(s)
  static constexpr int T_S = 0, T_W = BN, T_E = 2 * BN, T_P = T_E + BN / 2;
  static constexpr int T_GK = FUSED ? 192 : 320, T_GV = 320;
};

__device__ __forceinline__ void report(int code) { atomicCAS(&g_ktc_status, 0, code); }

template <bool FUSED>
__global__ void __launch_bounds__(kThreads, 1)
dkdv128_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmU,
               const __grid_constant__ CUtensorMap tmY, const __grid_constant__ CUtensorMap tmZ,
               const KArgs a) {
  using C = KCfg<FUSED>;
  constexpr int BN = C::BN, NS = C::NS, COL_SUB = C::COL_SUB, COL_TILE = C::COL_TILE, STAGE = C::STAGE;
  constexpr int OFF_VEC = C::OFF_VEC, OFF_BAR = C::OFF_BAR, OFF_TMEM = C::OFF_TMEM;
  constexpr int T_S = C::T_S, T_W = C::T_W, T_E = C::T_E, T_P = C::T_P, T_GK = C::T_GK, T_GV = C::T_GV;
  constexpr int HB = BN / 2;          // columns of one compute warp = packed bf16 columns of a tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + OFF_BAR;
  // barrier map: x | done | full[NS] | empty[NS] | s_full | s_free | p_full | pv_done
  const uint32_t BAR_X = bar0, BAR_DONE = bar0 + 8;
  auto BAR_FULL = [&](int s) { return bar0 + 8u * (2 + s); };
  auto BAR_EMPTY = [&](int s) { return bar0 + 8u * (2 + NS + s); };
  const uint32_t BAR_S = bar0 + 8u * (2 + 2 * NS), BAR_SFREE = BAR_S + 8, BAR_P = BAR_S + 16, BAR_PV = BAR_S + 24;
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem + OFF_TMEM);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // consecutive CTAs work on one head (its column tiles stay in L2); longest rows first
  constexpr bool rev = FUSED;
  const int head = blockIdx.x / a.ntr;
  const int pidx = blockIdx.x % a.ntr;
  const int r0 = (rev ? pidx : a.ntr - 1 - pidx) * BM;

  const int ntile = (a.ncols + BN - 1) / BN;
  int tb = 0, te = ntile;
  if (a.mask) {
    if (rev) tb = max(0, r0 - a.off) / BN;
    else te = min(ntile, (min(r0 + BM - 1, a.nrows - 1) + a.off) / BN + 1);
  }
  if (a.chunk > 0) {  // the row tile lies in one chunk (chunk % 256 == 0)
    const int cb = (r0 / a.chunk) * (a.chunk / BN), ce = cb + a.chunk / BN;
    if (rev) te = min(te, ce);
    else tb = cb;
  }
  // Grouped k/v heads: a query head reads the tiles of key/value head `head / ratio`; a key/value
  // head (FUSED rows) walks the same tile range once for each of its `ratio` query heads.
  const int Jh = max(te - tb, 0);
  const int J = rev ? Jh * a.ratio : Jh;
  // Column head and tile of the running tile number, advanced without divisions: `t` is the tile
  // inside the head's range [tb, tb + Jh), `h` the column head.
  struct ColPos { int t, h; };
  const ColPos pos0 = {tb, rev ? head * a.ratio : head / a.ratio};
  auto advance = [&](ColPos& cp, int steps) {
    cp.t += steps;
    if (rev)
      while (cp.t >= tb + Jh && Jh > 0) { cp.t -= Jh; ++cp.h; }
  };

  if (tid == 0) {
    mbar_init(BAR_X, 1);
    mbar_init(BAR_DONE, 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(BAR_FULL(s), 1);
      mbar_init(BAR_EMPTY(s), 1);
    }
    mbar_init(BAR_S, 1);
    mbar_init(BAR_SFREE, kComputeWarps);
    mbar_init(BAR_P, kComputeWarps);
    mbar_init(BAR_PV, 1);
    mbar_fence_init();
  }
  if (warp == kIssuerWarp) tmem_alloc(smem_u32((const void*)tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == kProducerWarp) {
    // ================= TMA producer =================
    if (lane == 0 && J > 0) {
      tma_prefetch_desc(&tmX);
      tma_prefetch_desc(&tmU);
      tma_prefetch_desc(&tmY);
      tma_prefetch_desc(&tmZ);
      mbar_expect_tx(BAR_X, 2 * ROW_TILE);
      for (int sub = 0; sub < 2; ++sub) {
        tma_load_3d(sbase + OFF_X + sub * ROW_SUB, &tmX, BAR_X, sub * 64, r0, head);
        tma_load_3d(sbase + OFF_U + sub * ROW_SUB, &tmU, BAR_X, sub * 64, r0, head);
      }
    }
    ColPos pc = pos0;
    for (int j = 0; j < J; ++j, advance(pc, 1)) {
      const int s = j % NS;
      if (!mbar_wait(BAR_EMPTY(s), (((j / NS) & 1) ^ 1))) { report(1); break; }
      if (lane == 0) {
        mbar_expect_tx(BAR_FULL(s), STAGE);
        const uint32_t dst = sbase + OFF_ST + s * STAGE;
        for (int sub = 0; sub < 2; ++sub) {
          tma_load_3d(dst + sub * COL_SUB, &tmY, BAR_FULL(s), sub * 64, pc.t * BN, pc.h);
          tma_load_3d(dst + COL_TILE + sub * COL_SUB, &tmZ, BAR_FULL(s), sub * 64, pc.t * BN, pc.h);
        }
      }
    }
  } else if (warp == kIssuerWarp) {
    // ================= MMA issuer of the S / W products (whole warp, one elected lane issues) ============
    if (J > 0) {
      constexpr uint32_t idescS = idesc_bf16(BM, BN, 0, 0);
      const uint32_t x_lo = desc_lo(sbase + OFF_X, 16), u_lo = desc_lo(sbase + OFF_U, 16);
      const uint32_t st_k = desc_lo(sbase + OFF_ST, 16);   // stage 0, K-major view
      bool ok = mbar_wait_warp(BAR_X, 0);
      if (!ok) report(2);
      tc_fence_after();
      for (int j = 0; ok && j < J; ++j) {
        const int s = j % NS;
        if (!mbar_wait_warp(BAR_FULL(s), (uint32_t)((j / NS) & 1))) { report(3); break; }
        if (j >= 1 && !mbar_wait_warp(BAR_SFREE, (uint32_t)((j - 1) & 1))) { report(4); break; }
        tc_fence_after();
        const uint32_t y_lo = st_k + (uint32_t)s * (STAGE >> 4);
        if (elect_one()) {
#pragma unroll
          for (int sub = 0; sub < 2; ++sub)
            umma_ss_k64(tmem + T_S, x_lo + sub * (ROW_SUB >> 4), y_lo + sub * (COL_SUB >> 4), idescS, sub > 0);
#pragma unroll
          for (int sub = 0; sub < 2; ++sub)
            umma_ss_k64(tmem + T_W, u_lo + sub * (ROW_SUB >> 4), y_lo + (COL_TILE >> 4) + sub * (COL_SUB >> 4),
                        idescS, sub > 0);
          umma_commit(BAR_S);
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else if (warp == kAccIssuerWarp) {
    // ================= MMA issuer of the accumulating products =================
    if (J > 0) {
      constexpr uint32_t idescO = idesc_bf16(BM, D, 0, 1);
      const uint32_t st_mn = desc_lo(sbase + OFF_ST, COL_SUB);   // stage 0, MN-major view (two 64-wide blocks)
      for (int j = 0; j < J; ++j) {
        const int s = j % NS;
        if (!mbar_wait_warp(BAR_P, (uint32_t)(j & 1))) { report(5); break; }
        tc_fence_after();
        const uint32_t y_mn = st_mn + (uint32_t)s * (STAGE >> 4);
        if (elect_one()) {
          umma_ts_steps<BN / 16>(tmem + T_GK, tmem + T_E, y_mn, idescO, j > 0 ? 1u : 0u);
          if (FUSED)
            umma_ts_steps<BN / 16>(tmem + T_GV, tmem + T_P, y_mn + (COL_TILE >> 4), idescO, j > 0 ? 1u : 0u);
          umma_commit(BAR_PV);
          umma_commit(BAR_EMPTY(s));
          if (j + 1 == J) umma_commit(BAR_DONE);
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else {
    // ================= compute warps =================
    const int cpart = warp >> 2, qd = warp & 3;
    const int row = r0 + qd * 32 + lane;
    const bool row_ok = row < a.nrows;
    // scale of the scores: query-head statistic times key-head statistic (the query head of a
    // FUSED tile changes with the tile when k/v heads are grouped)
    const float ck = stat_scale(a.stat_k, rev ? head : head / a.ratio, a.lim);
    const uint64_t A0v = pack2(a.a0, a.a0);
    uint64_t A1v, A2v, A2d;
    auto set_coefficients = [&](int hq) {
      const float c = stat_scale(a.stat_q, hq, a.lim) * ck;
      const float A1 = a.a1 * c, A2 = a.a2 * c * c;
      A1v = pack2(A1, A1);
      A2v = pack2(A2, A2);
      A2d = pack2(2.f * A2, 2.f * A2);
    };
    set_coefficients(rev ? head * a.ratio : head);
    int limcol = a.ncols - 1, lowcol = 0;                   // columns kept: lowcol <= col <= limcol
    if (a.mask) {
      if (rev) lowcol = row - a.off;
      else limcol = min(limcol, row + a.off);
    }
    const int wrow_lo = r0 + qd * 32, wrow_hi = wrow_lo + 31;
    float dl_row = 0.f;
    if (!rev && row_ok) dl_row = __ldg(a.dvec + (size_t)head * a.nrows + row);
    const uint64_t ndl_row = pack2(-dl_row, -dl_row);
    const uint32_t tl = tmem + ((uint32_t)(qd * 32) << 16);
    float* myvec = (float*)(smem + OFF_VEC) + warp * 64;
    const uint32_t myvec_s = sbase + OFF_VEC + warp * 256;
    // negated dvec of this lane's column in the next tile, fetched one tile ahead
    auto fetch_vec = [&](int j, const ColPos& cp) -> float {
      if (j >= J) return 0.f;
      const int col = cp.t * BN + cpart * 32 + lane;
      return (col < a.ncols) ? -__ldg(a.dvec + (size_t)cp.h * a.ncols + col) : 0.f;
    };
    ColPos pc = pos0;                     // position of the current tile
    float nxt = rev ? fetch_vec(0, pc) : 0.f;
    int hq_now = -1;
    bool ok = true;
    for (int j = 0; j < J; ++j, advance(pc, 1)) {
      const float cur = nxt;
      if (rev) {
        ColPos pn = pc;                   // the next tile
        advance(pn, 1);
        nxt = fetch_vec(j + 1, pn);
      }
      if (rev && a.ratio > 1 && pc.h != hq_now) {
        hq_now = pc.h;
        set_coefficients(pc.h);
      }
      if (!mbar_wait(BAR_S, (uint32_t)(j & 1))) { report(7); ok = false; break; }
      tc_fence_after();
      const uint32_t vec_s = myvec_s + (j & 1) * 128;
      if (rev) {
        myvec[(j & 1) * 32 + lane] = cur;
        __syncwarp();
      }
      // the warp's HB columns in passes of 32
#pragma unroll
      for (int ps = 0; ps < HB / 32; ++ps) {
        uint32_t sv[32], wv[32];
        tmem_ld32(tl + T_S + cpart * HB + ps * 32, sv);
        tmem_ld32(tl + T_W + cpart * HB + ps * 32, wv);
        tmem_wait_ld();
        if (ps + 1 == HB / 32) {
          // S and W of this tile are in registers: the next tile's may be issued
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(BAR_SFREE);
        }
        const int c0 = pc.t * BN + cpart * HB + ps * 32;    // first of these 32 columns
        bool need_mask = (c0 + 32 > a.ncols);
        if (a.mask) need_mask = need_mask || (rev ? (c0 < wrow_hi - a.off) : (c0 + 31 > wrow_lo + a.off));
        // the mask test stays outside the element loops so that each loop is one basic block whose
        // sixteen independent pairs the compiler can interleave
        uint32_t pe[16], pp[FUSED ? 16 : 1];
        ulonglong2 nd2 = make_ulonglong2(0ull, 0ull);
        if (!need_mask) {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const uint64_t s2 = pack2u(sv[2 * e], sv[2 * e + 1]);
            if (rev && (e & 1) == 0) nd2 = lds_v2(vec_s + (e >> 1) * 16);   // four column values per load
            const uint64_t ndl = rev ? ((e & 1) ? nd2.y : nd2.x) : ndl_row;
            pe[e] = pack_bf16_2(mul2(fma2(A2d, s2, A1v), add2(pack2u(wv[2 * e], wv[2 * e + 1]), ndl)));
            if (FUSED) pp[e] = pack_bf16_2(fma2(fma2(A2v, s2, A1v), s2, A0v));
          }
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const uint64_t s2 = pack2u(sv[2 * e], sv[2 * e + 1]);
            if (rev && (e & 1) == 0) nd2 = lds_v2(vec_s + (e >> 1) * 16);
            const uint64_t ndl = rev ? ((e & 1) ? nd2.y : nd2.x) : ndl_row;
            const int col = c0 + 2 * e;
            const bool z0 = col > limcol || col < lowcol, z1 = col + 1 > limcol || col + 1 < lowcol;
            float v0, v1;
            unpack2(mul2(fma2(A2d, s2, A1v), add2(pack2u(wv[2 * e], wv[2 * e + 1]), ndl)), v0, v1);
            pe[e] = pack_bf16(z0 ? 0.f : v0, z1 ? 0.f : v1);
            if (FUSED) {
              unpack2(fma2(fma2(A2v, s2, A1v), s2, A0v), v0, v1);
              pp[e] = pack_bf16(z0 ? 0.f : v0, z1 ? 0.f : v1);
            }
          }
        }
        // the previous tile's products must have consumed E and P before they are overwritten
        if (ps == 0 && j > 0) {
          if (!mbar_wait(BAR_PV, (uint32_t)((j - 1) & 1))) { report(9); ok = false; break; }
          tc_fence_after();
        }
        tmem_st16(tl + T_E + cpart * (HB / 2) + ps * 16, pe);
        if constexpr (FUSED) tmem_st16(tl + T_P + cpart * (HB / 2) + ps * 16, pp);
      }
      if (!ok) break;
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR_P);
    }
    // ---- epilogue: fused: warps 0-3 write grad_k (and the normalisation dot), warps 4-7 grad_v;
    // otherwise each warp writes 64 of the 128 grad_q columns of its rows ----
    if (ok && J > 0) {
      if (!mbar_wait(BAR_DONE, 0)) { report(10); ok = false; }
    }
    tc_fence_after();
    if (ok && J > 0) {
      const size_t grow = (size_t)head * a.nrows + (row_ok ? row : 0);
      const bool second = FUSED && cpart == 1;
      const bool dots_here = !second && a.dots != nullptr;
      float part;
      if constexpr (FUSED) {
        const float* add = second ? a.gv_add : a.gk_add;
        part = store_row<D>(tl + (second ? T_GV : T_GK), row_ok, (__nv_bfloat16*)(second ? a.gv : a.gk) + grow * D,
                            add ? add + grow * D : nullptr,
                            dots_here ? (const __nv_bfloat16*)a.x + grow * D : nullptr, 1.f);
      } else {
        const int cc = cpart * 64;
        part = store_row<64>(tl + T_GK + cc, row_ok, (__nv_bfloat16*)a.gk + grow * D + cc,
                             a.gk_add ? a.gk_add + grow * D + cc : nullptr,
                             dots_here ? (const __nv_bfloat16*)a.x + grow * D + cc : nullptr, 1.f);
      }
      if (dots_here) {
        float sum = part;
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
        if (lane == 0) atomicAdd(a.dots + head, sum);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kIssuerWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace

// bf16, head dimension 128, bh a multiple of bhkv; FASTMAX_B200_NO_WIDE=1 keeps separate grad_k / grad_v kernels.
bool dense_tc_dkdv128_supports(const fastmax_problem& p) {
  static const bool off = [] {
    const char* e = getenv("FASTMAX_B200_NO_WIDE");
    return e && e[0] == '1';
  }();
  return !off && p.dtype == FASTMAX_BF16 && p.d == 128 && p.bhkv > 0 && p.bh % p.bhkv == 0;
}

namespace {
template <bool FUSED>
int launch128(const Ctx& c, const char* name, const void* x, const void* u, const void* y, const void* z,
              int nrows, int ncols, KArgs a) {
  // rows are key/value heads in the fused kernel and query heads in grad_q; the columns are the other kind
  const int heads = FUSED ? c.p.bhkv : c.p.bh, col_heads = FUSED ? c.p.bh : c.p.bhkv;
  a.ratio = c.p.bh / c.p.bhkv;
  if (heads == 0 || nrows == 0) return FASTMAX_OK;
  CUtensorMap tx, tu, ty, tz;
  int rc;
  if ((rc = tma_map_bf16(&tx, x, heads, nrows, D, BM))) return rc;
  if ((rc = tma_map_bf16(&tu, u, heads, nrows, D, BM))) return rc;
  if ((rc = tma_map_bf16(&ty, y, col_heads, ncols, D, KCfg<FUSED>::BN))) return rc;
  if ((rc = tma_map_bf16(&tz, z, col_heads, ncols, D, KCfg<FUSED>::BN))) return rc;
  const fastmax_problem& p = c.p;
  a.x = x;
  a.nrows = nrows;
  a.ncols = ncols;
  a.off = p.nk - p.nq;
  a.mask = p.mask;
  a.ntr = (nrows + BM - 1) / BM;
  a.a0 = p.a0;
  a.a1 = p.a1;
  a.a2 = (p.p == 2) ? p.a2 : 0.f;
  a.lim = p.lim;
  FM_CUDA_TRY(cudaFuncSetAttribute(dkdv128_kernel<FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   KCfg<FUSED>::SMEM));
  dim3 grid((unsigned)((size_t)heads * a.ntr));
  FM_LAUNCH(name, c.stream, (dkdv128_kernel<FUSED><<<grid, kThreads, KCfg<FUSED>::SMEM, c.stream>>>(tx, tu, ty, tz, a)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}
}  // namespace

// The whole backward for d == 128: grad_q, then grad_k and grad_v in one kernel.
int dense_tc_backward128(const Ctx& c, const void* q, const void* k, const void* v, const void* gs,
                         const float* dvec, const stat_t* stats, float* dots, void* grad_q, void* grad_k,
                         void* grad_v, const ChunkAdd* ca) {
  const fastmax_problem& p = c.p;
  KArgs a = {};
  a.dvec = dvec;
  a.stat_q = p.normalize ? stats : nullptr;
  a.stat_k = p.normalize ? stats + p.bh : nullptr;
  a.chunk = ca ? ca->chunk : 0;
  int rc;
  a.gk = grad_q;
  a.gk_add = ca ? ca->gq_add : nullptr;
  a.dots = p.normalize ? dots : nullptr;
  if ((rc = launch128<false>(c, "fm_dense_tc_dq", q, gs, k, v, p.nq, p.nk, a))) return rc;
  a.gk = grad_k;
  a.gv = grad_v;
  a.gk_add = ca ? ca->gk_add : nullptr;
  a.gv_add = ca ? ca->gv_add : nullptr;
  a.dots = p.normalize ? dots + p.bh : nullptr;
  return launch128<true>(c, "fm_dense_tc_dkdv", k, v, q, gs, p.nk, p.nq, a);
}

int tc_dkdv128_status(int* out, cudaStream_t stream) {
  FM_CUDA_TRY(cudaMemcpyFromSymbolAsync(out, g_ktc_status, sizeof(int), 0, cudaMemcpyDeviceToHost, stream));
  FM_CUDA_TRY(cudaStreamSynchronize(stream));
  return FASTMAX_OK;
}
int tc_dkdv128_status_reset(cudaStream_t stream) {
  const int zero = 0;
  FM_CUDA_TRY(cudaMemcpyToSymbolAsync(g_ktc_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream));
  FM_CUDA_TRY(cudaStreamSynchronize(stream));
  return FASTMAX_OK;
}

}  // namespace fm
