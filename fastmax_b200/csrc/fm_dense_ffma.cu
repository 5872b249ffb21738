// Fastmax attention in tiled score form on CUDA cores (fp32 math, fp32 or bf16
// storage).  This family covers every supported head dimension, both
// polynomial orders, causal and unmasked, grouped k/v heads and nq != nk; it is
// the fp32 product path at short sequences and the on-device cross-check for
// the tensor-core families.
//
// One kernel template serves all three passes.  A 64-row tile owns its outputs
// and walks 64-column tiles; for each tile pair it forms S = X Y^T (and, for the
// gradients, W = U Z^T), applies the polynomial, and multiplies the result into
// the row tile's accumulators:
//
//   FWD   rows i = queries, cols j = keys:   num_i += f(s_ij) v_j, den_i += f(s_ij)
//   DQ    rows i = queries, cols j = keys:   dq_i  += f'(s_ij) w_ij k_j
//   DKDV  rows j = keys,    cols i = queries: dk_j += f'(s_ij) w_ij q_i,
//                                             dv_j += f(s_ij) g_i / den_i
//   with w_ij = (g_i.v_j - g_i.out_i) / den_i.
//
// These are the sums the reference evaluates through running moments
// (fastmax_cuda_forward.cu:25-197, fastmax_cuda_backward.cu:26-871 and the
// second-order terms in `old stuff/*_quad.cu`); expanding the moments gives the
// same polynomial in s.  The per-head normalisation scale is folded into the
// polynomial coefficients, so q and k are read as stored.
#include "fm_common.cuh"

namespace fm {
namespace {

enum { MODE_FWD = 0, MODE_DQ = 1, MODE_DKDV = 2 };
constexpr int BM = 64, BN = 64, LP = BN + 4;   // LP: row stride of the P / E tiles (16-byte aligned rows)

struct DenseArgs {
  const void* x;  // row operand: q (FWD, DQ) or k (DKDV)          [row heads][nrows][D]
  const void* u;  // 2nd row operand: grad_out (DQ) or v (DKDV)
  const void* y;  // column operand: k (FWD, DQ) or q (DKDV)       [col heads][ncols][D]
  const void* z;  // 2nd column operand: v (FWD, DQ) or grad_out (DKDV)
  const float* delta;  // (bh, nq) grad_out.out
  const float* den;    // (bh, nq)
  void* o1;            // out (FWD), grad_q (DQ), grad_k (DKDV)
  void* o2;            // grad_v (DKDV)
  float* den_out;      // FWD
  float* dots;         // per row head: sum o1 . x   (null when not normalised)
  const stat_t* stat_q;
  const stat_t* stat_k;
  int nrows, ncols, ratio, off, mask;
  int o_stride, den_stride, out_f32;
  float a0, a1, a2, lim;
  int chunk;              // > 0: only the columns of the row tile's own chunk
  const float* o1_add;    // fp32 (row heads, nrows, D) added to o1 before it is divided / stored
  const float* o2_add;    // same for o2
  const float* den_add;   // FWD: added to the row sum
};

// 64 rows of D elements -> fp32 tile with row stride D + 4 (rows stay 16-byte aligned, and the odd
// number of 16-byte units per row keeps 128-bit reads of eight consecutive rows free of bank
// conflicts).  Four elements per access where the source is aligned for it, else element by element.
__device__ __forceinline__ float4 ld4(const float* p) { return __ldg((const float4*)p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
  const uint2 w = __ldg((const uint2*)p);
  return make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xFFFF0000u), __uint_as_float(w.y << 16),
                     __uint_as_float(w.y & 0xFFFF0000u));
}
template <int D, typename T>
__device__ __forceinline__ void load_tile(float* dst, const T* src, int r0, int n) {
  constexpr int LD = D + 4, Q = D / 4;
  if ((reinterpret_cast<uintptr_t>(src) & (4 * sizeof(T) - 1)) == 0) {
    for (int idx = threadIdx.x; idx < 64 * Q; idx += 256) {
      const int r = idx / Q, c = (idx % Q) * 4;
      const float4 v = (r0 + r < n) ? ld4(src + (size_t)(r0 + r) * D + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      *(float4*)(dst + r * LD + c) = v;
    }
  } else {
    for (int idx = threadIdx.x; idx < 64 * D; idx += 256) {
      const int r = idx / D, c = idx % D;
      dst[r * LD + c] = (r0 + r < n) ? ldf(src + (size_t)(r0 + r) * D + c) : 0.f;
    }
  }
}

// N consecutive floats of shared memory (N in {1, 2, 4, 8}; p is N-float aligned) with the widest reads
template <int N>
__device__ __forceinline__ void ld_vec(float (&r)[N], const float* p) {
  if constexpr (N == 1) {
    r[0] = p[0];
  } else if constexpr (N == 2) {
    const float2 v = *(const float2*)p;
    r[0] = v.x; r[1] = v.y;
  } else {
#pragma unroll
    for (int q = 0; q < N / 4; ++q) {
      const float4 v = *(const float4*)(p + 4 * q);
      r[4 * q] = v.x; r[4 * q + 1] = v.y; r[4 * q + 2] = v.z; r[4 * q + 3] = v.w;
    }
  }
}

template <typename T>
__device__ __forceinline__ void store_any(void* base, size_t idx, float v, int f32) {
  if (f32) ((float*)base)[idx] = v;
  else stf((T*)base + idx, v);
}

// Two CTAs per SM up to d = 64 (128 registers, at most 105 KB of shared memory each); d = 128 runs one.
template <int D, int MODE, typename T>
__global__ void __launch_bounds__(256, (D <= 64) ? 2 : 1) dense_ffma_kernel(const DenseArgs a) {
  constexpr int LD = D + 4;
  constexpr int NC = (D + 15) / 16;
  extern __shared__ __align__(16) float smem[];
  float* Xs = smem;          // [BM][LD]
  float* Ys = Xs + BM * LD;  // [BN][LD]
  float* Zs = Ys + BN * LD;  // [BN][LD]
  float* Ps = Zs + BN * LD;  // [BM][LP]
  float* Us = Ps + BM * LP;  // [BM][LD]   DQ, DKDV
  float* Es = Us + BM * LD;  // [BM][LP]   DKDV
  float* cdelta = Es + BM * LP;  // [BN]   DKDV
  float* cinvd = cdelta + BN;    // [BN]   DKDV

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  // one-dimensional grid (head-major), so neither heads nor row tiles meet the 65535 limit of
  // grid.y; causal FWD/DQ tiles are issued longest (latest rows) first
  const int ntr = (a.nrows + BM - 1) / BM;
  const int hr = blockIdx.x / ntr;
  const int tidx = blockIdx.x % ntr;
  const int tile = (MODE == MODE_DKDV) ? tidx : ntr - 1 - tidx;
  const int r0 = tile * BM;
  const int kvh = (MODE == MODE_DKDV) ? hr : hr / a.ratio;

  load_tile<D>(Xs, (const T*)a.x + (size_t)hr * a.nrows * D, r0, a.nrows);
  if (MODE != MODE_FWD) load_tile<D>(Us, (const T*)a.u + (size_t)hr * a.nrows * D, r0, a.nrows);

  float rdelta[4], rinvd[4];
  if (MODE == MODE_DQ) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int r = r0 + ty + 16 * i;
      bool ok = r < a.nrows;
      rdelta[i] = ok ? a.delta[(size_t)hr * a.nrows + r] : 0.f;
      rinvd[i] = ok ? 1.0f / a.den[(size_t)hr * a.nrows + r] : 0.f;
    }
  }

  // the epilogue reads Xs written by other threads even when the column loop below runs zero times
  __syncthreads();

  float o1[4][NC], o2[4][NC], rsum[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    rsum[i] = 0.f;
#pragma unroll
    for (int m = 0; m < NC; ++m) { o1[i][m] = 0.f; o2[i][m] = 0.f; }
  }

  const float ck = stat_scale(a.stat_k, kvh, a.lim);
  const int groups = (MODE == MODE_DKDV) ? a.ratio : 1;
  for (int g = 0; g < groups; ++g) {
    const int qh = (MODE == MODE_DKDV) ? hr * a.ratio + g : hr;
    const int ch = (MODE == MODE_DKDV) ? qh : kvh;
    const float c = stat_scale(a.stat_q, qh, a.lim) * ck;
    const float A0 = a.a0, A1 = a.a1 * c, A2 = a.a2 * c * c;
    const T* Y = (const T*)a.y + (size_t)ch * a.ncols * D;
    const T* Z = (const T*)a.z + (size_t)ch * a.ncols * D;
    int ct0 = 0, ct1 = (a.ncols + BN - 1) / BN;
    if (a.mask) {
      if (MODE == MODE_DKDV) ct0 = max(0, r0 - a.off) / BN;
      else ct1 = min(ct1, (min(r0 + BM - 1, a.nrows - 1) + a.off) / BN + 1);
    }
    if (a.chunk > 0) {
      if (MODE == MODE_DKDV) ct1 = min(ct1, (r0 / a.chunk + 1) * (a.chunk / BN));
      else ct0 = (r0 / a.chunk) * (a.chunk / BN);
    }
    for (int ct = ct0; ct < ct1; ++ct) {
      const int c0 = ct * BN;
      __syncthreads();
      load_tile<D>(Ys, Y, c0, a.ncols);
      load_tile<D>(Zs, Z, c0, a.ncols);
      if (MODE == MODE_DKDV && tid < BN) {
        int i = c0 + tid;
        bool ok = i < a.ncols;
        cdelta[tid] = ok ? a.delta[(size_t)qh * a.ncols + i] : 0.f;
        cinvd[tid] = ok ? 1.0f / a.den[(size_t)qh * a.ncols + i] : 0.f;
      }
      __syncthreads();

      float s[4][4], w[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { s[i][j] = 0.f; w[i][j] = 0.f; }
      // four features per step, one 128-bit shared-memory read per row and step: a thread's four rows
      // (ty + 16 i) are broadcast within a quarter warp, its four columns (tx + 16 j) lie in rows whose
      // stride (D + 4 floats) spreads eight neighbours over all banks
#pragma unroll 2
      for (int kk = 0; kk < D; kk += 4) {
        float4 xr[4], yc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          xr[i] = *(const float4*)(Xs + (ty + 16 * i) * LD + kk);
          yc[i] = *(const float4*)(Ys + (tx + 16 * i) * LD + kk);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            s[i][j] = fmaf(xr[i].x, yc[j].x, s[i][j]);
            s[i][j] = fmaf(xr[i].y, yc[j].y, s[i][j]);
            s[i][j] = fmaf(xr[i].z, yc[j].z, s[i][j]);
            s[i][j] = fmaf(xr[i].w, yc[j].w, s[i][j]);
          }
        if (MODE != MODE_FWD) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            xr[i] = *(const float4*)(Us + (ty + 16 * i) * LD + kk);
            yc[i] = *(const float4*)(Zs + (tx + 16 * i) * LD + kk);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              w[i][j] = fmaf(xr[i].x, yc[j].x, w[i][j]);
              w[i][j] = fmaf(xr[i].y, yc[j].y, w[i][j]);
              w[i][j] = fmaf(xr[i].z, yc[j].z, w[i][j]);
              w[i][j] = fmaf(xr[i].w, yc[j].w, w[i][j]);
            }
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int row = r0 + ty + 16 * i, col = c0 + tx + 16 * j;
          bool ok = col < a.ncols;
          if (a.mask) ok = ok && (MODE == MODE_DKDV ? (row <= col + a.off) : (col <= row + a.off));
          const float sv = s[i][j];
          const float pf = ok ? fmaf(fmaf(A2, sv, A1), sv, A0) : 0.f;
          if (MODE == MODE_FWD) {
            Ps[(ty + 16 * i) * LP + tx + 16 * j] = pf;
            rsum[i] += pf;
          } else {
            const float dl = (MODE == MODE_DQ) ? rdelta[i] : cdelta[tx + 16 * j];
            const float iv = (MODE == MODE_DQ) ? rinvd[i] : cinvd[tx + 16 * j];
            const float ef = ok ? fmaf(2.f * A2, sv, A1) * (w[i][j] - dl) * iv : 0.f;
            if (MODE == MODE_DQ) {
              Ps[(ty + 16 * i) * LP + tx + 16 * j] = ef;
            } else {
              Es[(ty + 16 * i) * LP + tx + 16 * j] = ef;
              Ps[(ty + 16 * i) * LP + tx + 16 * j] = pf * iv;
            }
          }
        }
      }
      __syncthreads();

      // four score columns per step: the P (and E) values of a thread's rows come as 128-bit reads
#pragma unroll 2
      for (int j4 = 0; j4 < BN; j4 += 4) {
        float4 pr4[4], er4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          pr4[i] = *(const float4*)(Ps + (ty + 16 * i) * LP + j4);
          if (MODE == MODE_DKDV) er4[i] = *(const float4*)(Es + (ty + 16 * i) * LP + j4);
        }
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int j = j4 + jj;
          float pr[4], er[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            pr[i] = jj == 0 ? pr4[i].x : jj == 1 ? pr4[i].y : jj == 2 ? pr4[i].z : pr4[i].w;
            if (MODE == MODE_DKDV) er[i] = jj == 0 ? er4[i].x : jj == 1 ? er4[i].y : jj == 2 ? er4[i].z : er4[i].w;
          }
          // the thread's NC features of row j of Y and / or Z: one vector read each
          float yv[NC], zv[NC];
          if (D % 16 == 0 || tx * NC < D) {
            if (MODE != MODE_FWD) ld_vec<NC>(yv, Ys + j * LD + tx * NC);
            if (MODE != MODE_DQ) ld_vec<NC>(zv, Zs + j * LD + tx * NC);
#pragma unroll
            for (int m = 0; m < NC; ++m) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                if (MODE == MODE_FWD) o1[i][m] = fmaf(pr[i], zv[m], o1[i][m]);
                else if (MODE == MODE_DQ) o1[i][m] = fmaf(pr[i], yv[m], o1[i][m]);
                else {
                  o1[i][m] = fmaf(er[i], yv[m], o1[i][m]);
                  o2[i][m] = fmaf(pr[i], zv[m], o2[i][m]);
                }
              }
            }
          }
        }
      }
    }
  }

  // ---- epilogue -------------------------------------------------------------
  if (MODE == MODE_FWD) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int m = 8; m >= 1; m >>= 1) rsum[i] += __shfl_xor_sync(0xffffffffu, rsum[i], m);
      const int r = r0 + ty + 16 * i;
      if (r < a.nrows) {
        const size_t grow = (size_t)hr * a.nrows + r;
        const float dsum = rsum[i] + (a.den_add ? a.den_add[grow] : 0.f);
        const float inv = 1.0f / dsum;
        if (tx == 0) a.den_out[grow * a.den_stride] = dsum;
#pragma unroll
        for (int m = 0; m < NC; ++m) {
          const int cidx = tx * NC + m;   // a thread's output features are contiguous
          if (D % 16 == 0 || cidx < D) {
            const float num = o1[i][m] + (a.o1_add ? a.o1_add[grow * D + cidx] : 0.f);
            store_any<T>(a.o1, grow * a.o_stride + cidx, num * inv, a.out_f32);
          }
        }
      }
    }
  } else {
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = r0 + ty + 16 * i;
      if (r < a.nrows) {
        const size_t grow = (size_t)hr * a.nrows + r;
#pragma unroll
        for (int m = 0; m < NC; ++m) {
          const int cidx = tx * NC + m;   // a thread's output features are contiguous
          if (D % 16 == 0 || cidx < D) {
            const float g1 = o1[i][m] + (a.o1_add ? a.o1_add[grow * D + cidx] : 0.f);
            stf((T*)a.o1 + grow * D + cidx, g1);
            if (MODE == MODE_DKDV)
              stf((T*)a.o2 + grow * D + cidx, o2[i][m] + (a.o2_add ? a.o2_add[grow * D + cidx] : 0.f));
            part = fmaf(g1, Xs[(ty + 16 * i) * LD + cidx], part);
          }
        }
      }
    }
    if (a.dots) {
#pragma unroll
      for (int m = 16; m >= 1; m >>= 1) part += __shfl_xor_sync(0xffffffffu, part, m);
      __syncthreads();          // every warp is past its last read of Ps
      if ((tid & 31) == 0) Ps[tid >> 5] = part;
      __syncthreads();
      if (tid == 0) {
        float t = 0.f;
        for (int wv = 0; wv < 8; ++wv) t += Ps[wv];
        atomicAdd(a.dots + hr, t);
      }
    }
  }
}

size_t smem_bytes(int d, int mode) {
  size_t ld = d + 4;
  size_t f = 3 * 64 * ld + 64 * LP;
  if (mode != MODE_FWD) f += 64 * ld;
  if (mode == MODE_DKDV) f += 64 * LP + 2 * BN;
  return f * sizeof(float);
}

template <int D, int MODE, typename T>
int launch_one(const Ctx& c, const DenseArgs& a, int row_heads) {
  if (row_heads == 0 || a.nrows == 0) return FASTMAX_OK;
  size_t sm = smem_bytes(D, MODE);
  FM_CUDA_TRY(cudaFuncSetAttribute(dense_ffma_kernel<D, MODE, T>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
  const long long blocks = (long long)row_heads * ((a.nrows + BM - 1) / BM);
  if (blocks > 0x7FFFFFFFLL) return fail(FASTMAX_E_ARG, "heads x row tiles = %lld exceeds the grid limit", blocks);
  dim3 grid((unsigned)blocks);
  static const char* const names[3] = {"fm_dense_ffma_fwd", "fm_dense_ffma_dq", "fm_dense_ffma_dkdv"};
  FM_LAUNCH(names[MODE], c.stream, (dense_ffma_kernel<D, MODE, T><<<grid, 256, sm, c.stream>>>(a)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

template <int MODE>
int launch_mode(const Ctx& c, const DenseArgs& a, int row_heads) {
  const bool f32 = c.p.dtype == FASTMAX_F32;
  switch (c.p.d) {
#define FM_CASE(DD)                                                          \
  case DD:                                                                   \
    return f32 ? launch_one<DD, MODE, float>(c, a, row_heads)                \
               : launch_one<DD, MODE, __nv_bfloat16>(c, a, row_heads);
    FM_CASE(8) FM_CASE(16) FM_CASE(32) FM_CASE(64) FM_CASE(128)
#undef FM_CASE
  }
  return fail(FASTMAX_E_ARG, "head dimension %d is not one of 8,16,32,64,128", c.p.d);
}

DenseArgs base_args(const Ctx& c, const stat_t* stats) {
  const fastmax_problem& p = c.p;
  DenseArgs a = {};
  a.stat_q = p.normalize ? stats : nullptr;
  a.stat_k = p.normalize ? stats + p.bh : nullptr;
  a.ratio = p.bh / p.bhkv;
  a.off = p.nk - p.nq;
  a.mask = p.mask;
  a.a0 = p.a0;
  a.a1 = p.a1;
  a.a2 = (p.p == 2) ? p.a2 : 0.f;
  a.lim = p.lim;
  return a;
}

}  // namespace

int dense_ffma_forward(const Ctx& c, const void* q, const void* k, const void* v,
                       const stat_t* stats, const FwdOut& o, const ChunkAdd& ca) {
  DenseArgs a = base_args(c, stats);
  a.chunk = ca.chunk; a.o1_add = ca.out_add; a.den_add = ca.den_add;
  a.x = q; a.y = k; a.z = v;
  a.nrows = c.p.nq; a.ncols = c.p.nk;
  a.o1 = o.out; a.den_out = o.den;
  a.o_stride = o.o_stride; a.den_stride = o.den_stride; a.out_f32 = o.out_f32;
  return launch_mode<MODE_FWD>(c, a, c.p.bh);
}

int dense_ffma_backward(const Ctx& c, const void* q, const void* k, const void* v,
                        const float* den, const stat_t* stats, const void* grad_out,
                        const float* delta, float* dots, void* grad_q, void* grad_k,
                        void* grad_v, const ChunkAdd& ca) {
  const fastmax_problem& p = c.p;
  DenseArgs a = base_args(c, stats);
  a.delta = delta; a.den = den;
  a.chunk = ca.chunk; a.o1_add = ca.gq_add;
  // grad_q: rows are queries
  a.x = q; a.u = grad_out; a.y = k; a.z = v;
  a.nrows = p.nq; a.ncols = p.nk;
  a.o1 = grad_q;
  a.dots = p.normalize ? dots : nullptr;
  int rc = launch_mode<MODE_DQ>(c, a, p.bh);
  if (rc) return rc;
  // grad_k, grad_v: rows are keys, columns the queries of every head in the group
  a.x = k; a.u = v; a.y = q; a.z = grad_out;
  a.nrows = p.nk; a.ncols = p.nq;
  a.o1 = grad_k; a.o2 = grad_v;
  a.o1_add = ca.gk_add; a.o2_add = ca.gv_add;
  a.dots = p.normalize ? dots + p.bh : nullptr;
  return launch_mode<MODE_DKDV>(c, a, p.bhkv);
}

}  // namespace fm
