// Fastmax attention in tiled score form on the tcgen05 tensor cores (bf16 inputs,
// fp32 accumulation in tensor memory), head dimension 64.
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
// One CTA owns two 128-row tiles (two "groups" of four warps each, one row per
// thread) and streams column tiles through a shared-memory ring filled by TMA.
// A single thread issues every tcgen05.mma; per column tile and group:
//   S = X Y^T (and W = U Z^T)            smem x smem  -> TMEM
//   the group's warps read S (W) from TMEM, apply the polynomial and the mask and
//   write the bf16 result P back to TMEM
//   O += P Z   (or P Y)                  TMEM x smem  -> TMEM accumulator
// The issue order S0 S1 | O0 S0' | O1 S1' ... lets one group's CUDA-core work
// overlap the other group's tensor-core work.  All waits are bounded; a wait that
// gives up records an error status and the kernel winds down without hanging.
#include <climits>

#include "fm_common.cuh"
#include "fm_sm100.cuh"

namespace fm {

__device__ int g_tc_status = 0;  // first protocol error seen by any tensor-core kernel

namespace {
using namespace sm100;

enum { OP_A = 0, OP_B = 1 };

struct TcArgs {
  void* o;              // (heads, nrows, 64) bf16 result rows
  float* den_out;       // OP_A with fwd_div: (heads, nrows) row sums
  const float* dvec;    // OP_B: (heads, nq) grad_out.out / den
  const void* x;        // row operand in global memory (for the normalisation dots)
  float* dots;          // OP_B: per head sum of o . x  (null when not normalised)
  const stat_t* stat_q;
  const stat_t* stat_k;
  int nrows, ncols, off, mask, rev, fwd_div;
  float a0, a1, a2, lim;
};

constexpr int D = 64, BM = 128;
constexpr int kThreads = 320;  // warps 0-3: group 0, 4-7: group 1, 8: TMA producer, 9: MMA issuer

template <int MODE>
struct Cfg {
  static constexpr int BN = (MODE == OP_A) ? 128 : 64;
  static constexpr int NS = (MODE == OP_A) ? 3 : 4;
  static constexpr int ROW_TILE = BM * D * 2;
  static constexpr int COL_TILE = BN * D * 2;
  static constexpr int NROWOPS = (MODE == OP_A) ? 1 : 2;
  static constexpr int STAGE = 2 * COL_TILE;
  static constexpr int OFF_X = 0;
  static constexpr int OFF_U = 2 * ROW_TILE;
  static constexpr int OFF_ST = NROWOPS * 2 * ROW_TILE;
  static constexpr int OFF_VEC = OFF_ST + NS * STAGE;
  static constexpr int OFF_BAR = OFF_VEC + NS * BN * 4;
  static constexpr int NBAR = 1 + 2 * NS + 6;
  static constexpr int OFF_TMEM = OFF_BAR + NBAR * 8;
  static constexpr int SMEM = OFF_TMEM + 16 + 1024;  // + slack for the 1024-byte alignment
  // TMEM columns inside a group's 256-column half
  static constexpr int T_S = 0, T_W = 64, T_P = 128, T_O = 192;
};

__device__ __forceinline__ void report(int code) { atomicCAS(&g_tc_status, 0, code); }

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
dense_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmU,
                const __grid_constant__ CUtensorMap tmY, const __grid_constant__ CUtensorMap tmZ,
                const TcArgs a) {
  using C = Cfg<MODE>;
  constexpr int BN = C::BN, NS = C::NS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::OFF_BAR;
  auto BAR_X = [&]() { return bar0; };
  auto BAR_FULL = [&](int s) { return bar0 + 8u * (1 + s); };
  auto BAR_EMPTY = [&](int s) { return bar0 + 8u * (1 + NS + s); };
  auto BAR_S = [&](int g) { return bar0 + 8u * (1 + 2 * NS + g); };
  auto BAR_P = [&](int g) { return bar0 + 8u * (3 + 2 * NS + g); };
  auto BAR_O = [&](int g) { return bar0 + 8u * (5 + 2 * NS + g); };
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem + C::OFF_TMEM);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.x;
  const int pair = a.rev ? (int)blockIdx.y : (int)(gridDim.y - 1 - blockIdx.y);
  const int r0 = pair * 2 * BM;
  const bool colvec = (MODE == OP_B) && a.rev;

  // ---- tile ranges ----------------------------------------------------------------
  const int ntile = (a.ncols + BN - 1) / BN;
  int tbg[2], teg[2];
  bool act[2];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    const int R = r0 + g * BM;
    act[g] = R < a.nrows;
    tbg[g] = 0;
    teg[g] = ntile;
    if (a.mask) {
      if (a.rev) tbg[g] = max(0, R - a.off) / BN;
      else teg[g] = min(ntile, (min(R + BM - 1, a.nrows - 1) + a.off) / BN + 1);
    }
    if (!act[g]) { tbg[g] = INT_MAX; teg[g] = 0; }
  }
  const int tb = min(tbg[0], tbg[1]);
  const int te = max(teg[0], teg[1]);

  // ---- set-up -----------------------------------------------------------------------
  if (tid == 0) {
    mbar_init(BAR_X(), 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(BAR_FULL(s), colvec ? 33 : 1);
      mbar_init(BAR_EMPTY(s), 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(BAR_S(g), 1);
      mbar_init(BAR_P(g), 128);
      mbar_init(BAR_O(g), 1);
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
      const int nact = (act[0] ? 1 : 0) + (act[1] ? 1 : 0);
      mbar_expect_tx(BAR_X(), nact * C::NROWOPS * C::ROW_TILE);
      for (int g = 0; g < 2; ++g) {
        if (!act[g]) continue;
        tma_load_3d(sbase + C::OFF_X + g * C::ROW_TILE, &tmX, BAR_X(), 0, r0 + g * BM, head);
        if (MODE == OP_B)
          tma_load_3d(sbase + C::OFF_U + g * C::ROW_TILE, &tmU, BAR_X(), 0, r0 + g * BM, head);
      }
    }
    for (int t = tb; t < te; ++t) {
      const int k = t - tb, s = k % NS;
      if (!mbar_wait(BAR_EMPTY(s), (((k / NS) & 1) ^ 1))) { report(1); break; }
      if (lane == 0) {
        mbar_expect_tx(BAR_FULL(s), C::STAGE);
        const uint32_t dst = sbase + C::OFF_ST + s * C::STAGE;
        tma_load_3d(dst, &tmY, BAR_FULL(s), 0, t * BN, head);
        tma_load_3d(dst + C::COL_TILE, &tmZ, BAR_FULL(s), 0, t * BN, head);
      }
      if (colvec) {
        float* vec = (float*)(smem + C::OFF_VEC) + s * BN;
        for (int e = lane; e < BN; e += 32) {
          const int col = t * BN + e;
          vec[e] = (col < a.ncols) ? __ldg(a.dvec + (size_t)head * a.ncols + col) : 0.f;
        }
        mbar_arrive(BAR_FULL(s));
      }
    }
  } else if (warp == 9) {
    // ================= MMA issuer =================
    constexpr uint32_t idescS = idesc_bf16(BM, BN, 0, 0);
    constexpr uint32_t idescO = idesc_bf16(BM, D, 0, 1);
    bool ok = te > tb ? mbar_wait(BAR_X(), 0) : true;
    if (!ok) report(2);
    tc_fence_after();
    auto stage_of = [&](int t) { return (t - tb) % NS; };
    auto full_parity = [&](int t) { return (uint32_t)(((t - tb) / NS) & 1); };
    auto issue_S = [&](int g, int t) {
      const uint32_t st = sbase + C::OFF_ST + stage_of(t) * C::STAGE;
      const uint32_t xa = sbase + C::OFF_X + g * C::ROW_TILE;
      const uint32_t tg = tmem + g * 256;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        umma_ss(tg + C::T_S, smem_desc_sw128(xa + ks * 32, 16, 1024),
                smem_desc_sw128(st + ks * 32, 16, 1024), idescS, ks > 0);
      if (MODE == OP_B) {
        const uint32_t ua = sbase + C::OFF_U + g * C::ROW_TILE;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_ss(tg + C::T_W, smem_desc_sw128(ua + ks * 32, 16, 1024),
                  smem_desc_sw128(st + C::COL_TILE + ks * 32, 16, 1024), idescS, ks > 0);
      }
      umma_commit(BAR_S(g));
    };
    auto issue_O = [&](int g, int t, bool acc) {
      const uint32_t st = sbase + C::OFF_ST + stage_of(t) * C::STAGE;
      const uint32_t b = (MODE == OP_A) ? st + C::COL_TILE : st;  // OP_A: Z tile, OP_B: Y tile
      const uint32_t tg = tmem + g * 256;
#pragma unroll
      for (int ks = 0; ks < BN / 16; ++ks)
        umma_ts(tg + C::T_O, tg + C::T_P + ks * 8, smem_desc_sw128(b + ks * 2048, C::COL_TILE, 1024),
                idescO, (acc || ks > 0) ? 1u : 0u);
    };
    if (ok && te > tb) {
      if (!mbar_wait(BAR_FULL(stage_of(tb)), full_parity(tb))) { report(3); ok = false; }
      tc_fence_after();
      if (ok && lane == 0)
        for (int g = 0; g < 2; ++g)
          if (act[g] && tbg[g] == tb) issue_S(g, tb);
      __syncwarp();
    }
    for (int t = tb; ok && t < te; ++t) {
      for (int g = 0; ok && g < 2; ++g) {
        if (!act[g]) continue;
        if (t >= tbg[g] && t < teg[g]) {
          if (!mbar_wait(BAR_P(g), (uint32_t)((t - tbg[g]) & 1))) { report(4); ok = false; break; }
          tc_fence_after();
          if (lane == 0) issue_O(g, t, t > tbg[g]);
          if (t + 1 < teg[g]) {
            if (!mbar_wait(BAR_FULL(stage_of(t + 1)), full_parity(t + 1))) { report(5); ok = false; break; }
            tc_fence_after();
            if (lane == 0) issue_S(g, t + 1);
          } else if (lane == 0) {
            umma_commit(BAR_O(g));
          }
        } else if (t + 1 == tbg[g]) {
          if (!mbar_wait(BAR_FULL(stage_of(t + 1)), full_parity(t + 1))) { report(6); ok = false; break; }
          tc_fence_after();
          if (lane == 0) issue_S(g, t + 1);
        }
        __syncwarp();
      }
      if (ok && lane == 0) umma_commit(BAR_EMPTY(stage_of(t)));
      __syncwarp();
    }
  } else {
    // ================= compute groups =================
    const int g = warp >> 2, qd = warp & 3;
    if (act[g]) {
      const int row = r0 + g * BM + qd * 32 + lane;
      const bool row_ok = row < a.nrows;
      const float c = stat_scale(a.stat_q, head, a.lim) * stat_scale(a.stat_k, head, a.lim);
      const float A0 = a.a0, A1 = a.a1 * c, A2 = a.a2 * c * c;
      // columns kept for this row: lowcol <= col <= limcol
      int limcol = a.ncols - 1, lowcol = 0;
      if (a.mask) {
        if (a.rev) lowcol = row - a.off;
        else limcol = min(limcol, row + a.off);
      }
      const int wrow_lo = r0 + g * BM + qd * 32, wrow_hi = wrow_lo + 31;
      float dl_row = 0.f;
      if (MODE == OP_B && !a.rev && row_ok) dl_row = __ldg(a.dvec + (size_t)head * a.nrows + row);
      const uint32_t tg = tmem + g * 256 + ((uint32_t)(qd * 32) << 16);
      float rowsum = 0.f;
      bool ok = true;
      for (int t = tbg[g]; t < teg[g]; ++t) {
        if (!mbar_wait(BAR_S(g), (uint32_t)((t - tbg[g]) & 1))) { report(7); ok = false; break; }
        tc_fence_after();
        const float* vec = nullptr;
        if (colvec) {
          const int k = t - tb, s = k % NS;
          if (!mbar_wait(BAR_FULL(s), (uint32_t)((k / NS) & 1))) { report(8); ok = false; break; }
          vec = (const float*)(smem + C::OFF_VEC) + s * BN;
        }
        const int c0 = t * BN;
        // does any element of this warp's 32 x BN block need masking?
        bool need_mask = (c0 + BN > a.ncols);
        if (a.mask) need_mask = need_mask || (a.rev ? (c0 < wrow_hi - a.off) : (c0 + BN - 1 > wrow_lo + a.off));
#pragma unroll
        for (int cc = 0; cc < BN / 32; ++cc) {
          uint32_t sv[32], pk[16];
          float pv[32];
          tmem_ld32(tg + C::T_S + cc * 32, sv);
          if (MODE == OP_B) {
            uint32_t wv[32];
            tmem_ld32(tg + C::T_W + cc * 32, wv);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float s = __uint_as_float(sv[e]);
              const float dl = a.rev ? vec[cc * 32 + e] : dl_row;
              pv[e] = fmaf(2.f * A2, s, A1) * (__uint_as_float(wv[e]) - dl);
            }
          } else {
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float s = __uint_as_float(sv[e]);
              pv[e] = fmaf(fmaf(A2, s, A1), s, A0);
            }
          }
          if (need_mask) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int col = c0 + cc * 32 + e;
              if (col > limcol || col < lowcol) pv[e] = 0.f;
            }
          }
          if (MODE == OP_A) {
#pragma unroll
            for (int e = 0; e < 32; ++e) rowsum += pv[e];
          }
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = pack_bf16(pv[2 * e], pv[2 * e + 1]);
          tmem_st16(tg + C::T_P + cc * 16, pk);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(BAR_P(g));
      }
      // ---- epilogue: this thread's row of the accumulator -> global ----
      if (ok && teg[g] > tbg[g]) {
        if (!mbar_wait(BAR_O(g), 0)) { report(9); ok = false; }
      }
      tc_fence_after();
      if (ok && teg[g] > tbg[g]) {
        uint32_t o0[32], o1[32];
        tmem_ld32(tg + C::T_O, o0);
        tmem_ld32(tg + C::T_O + 32, o1);
        tmem_wait_ld();
        float scale = 1.f;
        if (MODE == OP_A && a.fwd_div) scale = 1.0f / rowsum;
        float part = 0.f;
        if (row_ok) {
          const size_t grow = (size_t)head * a.nrows + row;
          uint4* dst = (uint4*)((__nv_bfloat16*)a.o + grow * D);
          const uint4* xr = (const uint4*)((const __nv_bfloat16*)a.x + grow * D);
          const bool want_dots = (MODE == OP_B) && a.dots != nullptr;
#pragma unroll
          for (int v8 = 0; v8 < 8; ++v8) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int idx = v8 * 8 + e;
              f[e] = __uint_as_float(idx < 32 ? o0[idx] : o1[idx - 32]) * scale;
            }
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
          if (MODE == OP_A && a.fwd_div) a.den_out[grow] = rowsum;
        }
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

// (heads, n, 64) bf16 tensor as a rank-3 map with boxes of box_rows x 64, 128-byte swizzle;
// rows past n read as zero.
int make_map(CUtensorMap* m, const void* base, int heads, int n, int box_rows) {
  EncodeFn enc = encode_fn();
  if (!enc) return fail(FASTMAX_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[3] = {(cuuint64_t)D, (cuuint64_t)n, (cuuint64_t)heads};
  cuuint64_t gstr[2] = {(cuuint64_t)D * 2, (cuuint64_t)n * D * 2};
  cuuint32_t box[3] = {(cuuint32_t)D, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FASTMAX_E_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return FASTMAX_OK;
}

template <int MODE>
int launch_tc(const Ctx& c, const char* name, const void* x, const void* u, const void* y,
              const void* z, int nrows, int ncols, TcArgs a) {
  using C = Cfg<MODE>;
  const int heads = c.p.bh;
  if (heads == 0 || nrows == 0) return FASTMAX_OK;
  CUtensorMap tx, tu, ty, tz;
  int rc;
  if ((rc = make_map(&tx, x, heads, nrows, BM))) return rc;
  if ((rc = make_map(&tu, u ? u : x, heads, nrows, BM))) return rc;
  if ((rc = make_map(&ty, y, heads, ncols, C::BN))) return rc;
  if ((rc = make_map(&tz, z, heads, ncols, C::BN))) return rc;
  a.nrows = nrows;
  a.ncols = ncols;
  a.x = x;
  FM_CUDA_TRY(cudaFuncSetAttribute(dense_tc_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   C::SMEM));
  dim3 grid(heads, (nrows + 2 * BM - 1) / (2 * BM));
  FM_LAUNCH(name, c.stream,
            (dense_tc_kernel<MODE><<<grid, kThreads, C::SMEM, c.stream>>>(tx, tu, ty, tz, a)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
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
  return p.dtype == FASTMAX_BF16 && p.d == 64 && p.bh == p.bhkv;
}

int dense_tc_forward(const Ctx& c, const void* q, const void* k, const void* v,
                     const stat_t* stats, void* out, float* den) {
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out))
    return fail(FASTMAX_E_ARG, "the tensor-core family needs 16-byte aligned tensors");
  TcArgs a = base_args(c, stats);
  a.o = out;
  a.den_out = den;
  a.fwd_div = 1;
  a.rev = 0;
  return launch_tc<OP_A>(c, "fm_dense_tc_fwd", q, nullptr, k, v, c.p.nq, c.p.nk, a);
}

int dense_tc_backward(const Ctx& c, const void* q, const void* k, const void* v, const void* gs,
                      const float* dvec, const stat_t* stats, float* dots, void* grad_q,
                      void* grad_k, void* grad_v) {
  const fastmax_problem& p = c.p;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(gs) || !aligned16(grad_q) ||
      !aligned16(grad_k) || !aligned16(grad_v))
    return fail(FASTMAX_E_ARG, "the tensor-core family needs 16-byte aligned tensors");
  int rc;
  TcArgs a = base_args(c, stats);
  a.dvec = dvec;
  // grad_q: rows = queries, columns = keys
  a.o = grad_q;
  a.rev = 0;
  a.dots = p.normalize ? dots : nullptr;
  if ((rc = launch_tc<OP_B>(c, "fm_dense_tc_dq", q, gs, k, v, p.nq, p.nk, a))) return rc;
  // grad_k: rows = keys, columns = queries
  a.o = grad_k;
  a.rev = 1;
  a.dots = p.normalize ? dots + p.bh : nullptr;
  if ((rc = launch_tc<OP_B>(c, "fm_dense_tc_dk", k, v, q, gs, p.nk, p.nq, a))) return rc;
  // grad_v: rows = keys, columns = queries, plain sum
  a.o = grad_v;
  a.dots = nullptr;
  a.fwd_div = 0;
  return launch_tc<OP_A>(c, "fm_dense_tc_dv", k, nullptr, q, gs, p.nk, p.nq, a);
}

int tc_status(int* out, cudaStream_t stream) {
  FM_CUDA_TRY(cudaMemcpyFromSymbolAsync(out, g_tc_status, sizeof(int), 0, cudaMemcpyDeviceToHost, stream));
  FM_CUDA_TRY(cudaStreamSynchronize(stream));
  return FASTMAX_OK;
}

}  // namespace fm
