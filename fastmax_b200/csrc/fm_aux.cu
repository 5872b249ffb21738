// HBM-bound helper kernels of the Fastmax passes: per-head max row norm (the
// normalisation statistic), the grad_out.out row dots of the backward pass and
// the single-row gradient of the max-norm scaling.
#include "fm_common.cuh"

namespace fm {

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(const uint32_t*)&v;
}

// ---------------------------------------------------------------------------
// Row statistics: for every head, max_n ||x_n||^2 and the row that attains it.
// Replaces calc_norms + find_max (reference fastmax_cuda_forward.cu:223-253);
// the scale lim/max is applied inside the attention kernels instead of
// rewriting q and k in place (reference apply_norm, :255-269).
// Each warp owns rows; a row of D elements is read by D/VEC lanes, so a warp
// covers 32*VEC/D rows per load and every load is a full 128-byte line.
template <typename T, int D, bool WIDE>
__global__ void __launch_bounds__(256) rowmax_kernel(const T* __restrict__ x, int n,
                                                     int rows_per_block, int row_offset,
                                                     stat_t* __restrict__ stats) {
  // elements per lane: 16 bytes for the wide bf16 rows, else 4 (or 1) elements
  // (WIDE needs 16-byte aligned rows; the launcher checks the base pointer)
  constexpr int VEC = WIDE ? 8 : ((D >= 32) ? 4 : 1);
  constexpr int LPR = D / VEC;                 // lanes per row
  constexpr int RPW = 32 / LPR;                // rows per warp per step
  static_assert(D % VEC == 0 && LPR <= 32 && 32 % LPR == 0, "bad head dimension");
  const int head = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / LPR, off = (lane % LPR) * VEC;
  const int row0 = blockIdx.y * rows_per_block;
  const int row1 = min(n, row0 + rows_per_block);
  const T* base = x + (size_t)head * n * D;
  float best = -1.0f;
  int best_row = 0;
  // the loop bound is warp-uniform: every lane takes part in every shuffle
  for (int rb = row0 + warp * RPW; rb < row1; rb += 8 * RPW) {
    const int r = rb + sub;
    float s = 0.f;
    if (r < row1) {
      const T* p = base + (size_t)r * D + off;
      if constexpr (VEC == 8) {
        const uint4 w = __ldg((const uint4*)p);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = __uint_as_float(ww[e] << 16), hi = __uint_as_float(ww[e] & 0xFFFF0000u);
          s = fmaf(lo, lo, fmaf(hi, hi, s));
        }
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          float t = ldf(p + e);
          s = fmaf(t, t, s);
        }
      }
    }
#pragma unroll
    for (int m = LPR / 2; m >= 1; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
    if (r < row1 && s > best) { best = s; best_row = r; }
  }
  // NaN norms never compare greater, so they are ignored as a maximum.
  if (best >= 0.f && (lane % LPR) == 0) {
    stat_t w = ((stat_t)__float_as_uint(best) << 32) | (stat_t)(0xFFFFFFFFu - (unsigned)(best_row + row_offset));
    atomicMax(&stats[head], w);
  }
}

template <typename T>
static int rowmax_one(const Ctx& c, const T* x, int heads, int n, stat_t* stats, int row_offset) {
  if (heads == 0 || n == 0) return FASTMAX_OK;
  // enough blocks per head to fill the GPU, at least 256 rows each
  int splits = max(1, min((n + 255) / 256, (148 * 8 + heads - 1) / heads));
  int rpb = (n + splits - 1) / splits;
  dim3 grid(heads, (n + rpb - 1) / rpb);
  switch (c.p.d) {
#define FM_CASE(DD) \
  case DD:                                                                              \
    if (sizeof(T) == 2 && DD >= 64 && ((uintptr_t)x & 15) == 0)                           \
      FM_LAUNCH("fm_rowmax", c.stream,                                                    \
                (rowmax_kernel<T, DD, (sizeof(T) == 2 && DD >= 64)><<<grid, 256, 0, c.stream>>>(x, n, rpb, row_offset, stats))); \
    else                                                                                  \
      FM_LAUNCH("fm_rowmax", c.stream,                                                    \
                (rowmax_kernel<T, DD, false><<<grid, 256, 0, c.stream>>>(x, n, rpb, row_offset, stats)));      \
    break;
    FM_CASE(8) FM_CASE(16) FM_CASE(32) FM_CASE(64) FM_CASE(128)
#undef FM_CASE
    default: return fail(FASTMAX_E_ARG, "head dimension %d is not one of 8,16,32,64,128", c.p.d);
  }
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

int launch_rowmax(const Ctx& c, const void* q, const void* k, stat_t* stats, int row_offset) {
  const fastmax_problem& p = c.p;
  FM_CUDA_TRY(cudaMemsetAsync(stats, 0, sizeof(stat_t) * (size_t)(p.bh + p.bhkv), c.stream));
  int rc;
  if (p.dtype == FASTMAX_F32) {
    if ((rc = rowmax_one<float>(c, (const float*)q, p.bh, p.nq, stats, row_offset))) return rc;
    return rowmax_one<float>(c, (const float*)k, p.bhkv, p.nk, stats + p.bh, row_offset);
  }
  if ((rc = rowmax_one<__nv_bfloat16>(c, (const __nv_bfloat16*)q, p.bh, p.nq, stats, row_offset))) return rc;
  return rowmax_one<__nv_bfloat16>(c, (const __nv_bfloat16*)k, p.bhkv, p.nk, stats + p.bh, row_offset);
}

// ---------------------------------------------------------------------------
// delta[row] = grad_out[row,:] . out[row,:]; one warp per row.  Together with
// 1/den this is the "-O . dDen" part of the reference's backward
// (fastmax_cuda_backward.cu:63-161 and div_grad_output :874-882), computed once
// instead of inside every gradient kernel, and without touching grad_out.
template <typename T>
__global__ void __launch_bounds__(256) delta_kernel(const T* __restrict__ go,
                                                    const T* __restrict__ out, size_t rows,
                                                    int d, float* __restrict__ delta) {
  size_t row = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float s = 0.f;
  for (int c = lane; c < d; c += 32) s = fmaf(ldf(go + row * d + c), ldf(out + row * d + c), s);
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
  if (lane == 0) delta[row] = s;
}

// The same for bf16 rows of 64 or 128 elements with 16-byte aligned tensors: 16 bytes per lane,
// several rows per warp, two independent steps per warp.
template <int D>
__global__ void __launch_bounds__(256) delta_wide_kernel(const __nv_bfloat16* __restrict__ go,
                                                         const __nv_bfloat16* __restrict__ out, size_t rows,
                                                         float* __restrict__ delta) {
  constexpr int LPR = D / 8, RPW = 32 / LPR, STEPS = 2;
  const int lane = threadIdx.x & 31, sub = lane / LPR, part = lane % LPR;
  const size_t row0 = ((size_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * (RPW * STEPS) + sub;
  uint4 g[STEPS], o[STEPS];
#pragma unroll
  for (int t = 0; t < STEPS; ++t) {
    const size_t row = row0 + (size_t)t * RPW;
    g[t] = (row < rows) ? __ldg((const uint4*)(go + row * D) + part) : make_uint4(0u, 0u, 0u, 0u);
    o[t] = (row < rows) ? __ldg((const uint4*)(out + row * D) + part) : make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int t = 0; t < STEPS; ++t) {
    const size_t row = row0 + (size_t)t * RPW;
    const uint32_t gw[4] = {g[t].x, g[t].y, g[t].z, g[t].w}, ow[4] = {o[t].x, o[t].y, o[t].z, o[t].w};
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      s = fmaf(__uint_as_float(gw[e] << 16), __uint_as_float(ow[e] << 16), s);
      s = fmaf(__uint_as_float(gw[e] & 0xFFFF0000u), __uint_as_float(ow[e] & 0xFFFF0000u), s);
    }
#pragma unroll
    for (int m = LPR / 2; m >= 1; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
    if (row < rows && part == 0) delta[row] = s;
  }
}

int launch_delta(const Ctx& c, const void* go, const void* out, float* delta) {
  size_t rows = (size_t)c.p.bh * c.p.nq;
  if (rows == 0) return FASTMAX_OK;
  if (c.p.dtype == FASTMAX_BF16 && (c.p.d == 64 || c.p.d == 128) && (((uintptr_t)go | (uintptr_t)out) & 15) == 0) {
    const size_t rows_per_block = 8 * (32 / (c.p.d / 8)) * 2;
    const unsigned nb = (unsigned)((rows + rows_per_block - 1) / rows_per_block);
    if (c.p.d == 64)
      FM_LAUNCH("fm_delta", c.stream,
                (delta_wide_kernel<64><<<nb, 256, 0, c.stream>>>((const __nv_bfloat16*)go, (const __nv_bfloat16*)out,
                                                                 rows, delta)));
    else
      FM_LAUNCH("fm_delta", c.stream,
                (delta_wide_kernel<128><<<nb, 256, 0, c.stream>>>((const __nv_bfloat16*)go, (const __nv_bfloat16*)out,
                                                                  rows, delta)));
    FM_CUDA_TRY(cudaGetLastError());
    return FASTMAX_OK;
  }
  unsigned blocks = (unsigned)((rows + 7) / 8);
  if (c.p.dtype == FASTMAX_F32)
    FM_LAUNCH("fm_delta", c.stream,
              (delta_kernel<float><<<blocks, 256, 0, c.stream>>>((const float*)go, (const float*)out,
                                                                  rows, c.p.d, delta)));
  else
    FM_LAUNCH("fm_delta", c.stream,
              (delta_kernel<__nv_bfloat16><<<blocks, 256, 0, c.stream>>>(
                  (const __nv_bfloat16*)go, (const __nv_bfloat16*)out, rows, c.p.d, delta)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

// ---------------------------------------------------------------------------
// Backward preparation for the tensor-core family: the upstream gradient scaled
// by 1/den (rounded to bf16, it becomes a matrix operand) and the scaled row dot
// dvec = (grad_out . out)/den, so that w_ij = gs_i . v_j - dvec_i.  One warp per
// row of 64 or 128 elements, one or two bf16 pairs per lane.
template <int D>
__global__ void __launch_bounds__(256) gprep_kernel(const __nv_bfloat16* __restrict__ go,
                                                    const __nv_bfloat16* __restrict__ out,
                                                    const float* __restrict__ den, size_t rows,
                                                    __nv_bfloat16* __restrict__ gs,
                                                    float* __restrict__ dvec, int n, int out_heads) {
  constexpr int LPR = D / 8;        // lanes per row, 16 bytes (8 elements) each
  constexpr int RPW = 32 / LPR;     // rows per warp and step
  constexpr int STEPS = 2;          // independent steps per warp: more bytes in flight
  const int lane = threadIdx.x & 31, sub = lane / LPR, part = lane % LPR;
  const size_t row0 = ((size_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * (RPW * STEPS) + sub;
  uint4 g[STEPS], o[STEPS];
#pragma unroll
  for (int t = 0; t < STEPS; ++t) {
    const size_t row = row0 + (size_t)t * RPW;
    if (row < rows) {
      // grad_out and out may be (batch, n, heads, D) arrays; gs, dvec and den are always (heads, n, .)
      const size_t src = out_heads > 0 ? out_row((int)(row / n), (int)(row % n), n, out_heads) : row;
      g[t] = __ldg((const uint4*)(go + src * D) + part);
      o[t] = __ldg((const uint4*)(out + src * D) + part);
    } else {
      g[t] = make_uint4(0u, 0u, 0u, 0u);
      o[t] = g[t];
    }
  }
#pragma unroll
  for (int t = 0; t < STEPS; ++t) {
    const size_t row = row0 + (size_t)t * RPW;
    const uint32_t gw[4] = {g[t].x, g[t].y, g[t].z, g[t].w}, ow[4] = {o[t].x, o[t].y, o[t].z, o[t].w};
    // dvec is formed from the ROUNDED gs values: the gradient kernels subtract it from gs . v, and with
    // both built from the same bf16 numbers the difference is gs . (v - out) exactly, so the rounding of
    // gs acts like a 2^-9 relative change of grad_out instead of an absolute error that survives the
    // cancellation (early causal rows, where out is close to the few values seen, showed it)
    const float inv = (row < rows) ? 1.0f / __ldg(den + row) : 0.f;
    uint32_t gr[4];
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      gr[e] = pack_bf16x2(__uint_as_float(gw[e] << 16) * inv, __uint_as_float(gw[e] & 0xFFFF0000u) * inv);
      s = fmaf(__uint_as_float(gr[e] << 16), __uint_as_float(ow[e] << 16), s);
      s = fmaf(__uint_as_float(gr[e] & 0xFFFF0000u), __uint_as_float(ow[e] & 0xFFFF0000u), s);
    }
#pragma unroll
    for (int m = LPR / 2; m >= 1; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
    if (row < rows) {
      ((uint4*)(gs + row * D))[part] = make_uint4(gr[0], gr[1], gr[2], gr[3]);
      if (part == 0) dvec[row] = s;
    }
  }
}

int launch_gprep(const Ctx& c, const void* go, const void* out, const float* den, void* gs,
                 float* dvec) {
  size_t rows = (size_t)c.p.bh * c.p.nq;
  if (rows == 0) return FASTMAX_OK;
  if ((c.p.d != 64 && c.p.d != 128) || c.p.dtype != FASTMAX_BF16)
    return fail(FASTMAX_E_UNSUPPORTED, "gprep handles bf16 rows of 64 or 128 elements");
  if ((((uintptr_t)go | (uintptr_t)out | (uintptr_t)gs) & 15) != 0)
    return fail(FASTMAX_E_ARG, "the tensor-core family needs 16-byte aligned tensors");
  // a block of 8 warps covers 8 x (rows per warp-step) x 2 steps rows
  const size_t rows_per_block = 8 * (32 / (c.p.d / 8)) * 2;
  unsigned blocks = (unsigned)((rows + rows_per_block - 1) / rows_per_block);
  if (c.p.d == 64)
    FM_LAUNCH("fm_gprep", c.stream,
              (gprep_kernel<64><<<blocks, 256, 0, c.stream>>>((const __nv_bfloat16*)go,
                                                              (const __nv_bfloat16*)out, den, rows,
                                                              (__nv_bfloat16*)gs, dvec, c.p.nq, c.out_heads)));
  else
    FM_LAUNCH("fm_gprep", c.stream,
              (gprep_kernel<128><<<blocks, 256, 0, c.stream>>>((const __nv_bfloat16*)go,
                                                               (const __nv_bfloat16*)out, den, rows,
                                                               (__nv_bfloat16*)gs, dvec, c.p.nq, c.out_heads)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

// ---------------------------------------------------------------------------
// Gradient of x_hat = lim * x / m, m = ||x_r|| the largest row norm of the head:
//   dx_n = (lim/m) dx_hat_n  -  [n == r] (sum_n dx_hat_n . x_hat_n) x_r / m^2 .
// The attention kernels already wrote (lim/m) dx_hat and accumulated
// dots[head] = sum_n (lim/m) dx_hat_n . x_n, which equals the bracketed sum, so
// only row r of each head is corrected here.  The reference's CUDA backward
// has no such term; autograd through its PyTorch path (example.py:105-108) does.
template <typename T>
__global__ void norm_fixup_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                  const stat_t* __restrict__ stats,
                                  const float* __restrict__ dots, T* __restrict__ gq,
                                  T* __restrict__ gk, int bh, int nq, int nk, int d,
                                  int row_offset) {
  int head = blockIdx.x;
  const T* x;
  T* g;
  int n;
  if (head < bh) { x = q + (size_t)head * nq * d; g = gq + (size_t)head * nq * d; n = nq; }
  else { x = k + (size_t)(head - bh) * nk * d; g = gk + (size_t)(head - bh) * nk * d; n = nk; }
  stat_t s = stats[head];
  int r = stat_row(s) - row_offset;
  float m2 = stat_norm2(s);
  if (r < 0 || r >= n) return;
  float coef = dots[head] / m2;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    size_t i = (size_t)r * d + c;
    stf(g + i, ldf(g + i) - coef * ldf(x + i));
  }
}

int launch_norm_fixup(const Ctx& c, const void* q, const void* k, const stat_t* stats,
                      const float* dots, void* gq, void* gk, int row_offset) {
  const fastmax_problem& p = c.p;
  int heads = p.bh + p.bhkv;
  if (heads == 0) return FASTMAX_OK;
  if (p.dtype == FASTMAX_F32)
    FM_LAUNCH("fm_norm_fixup", c.stream,
              (norm_fixup_kernel<float><<<heads, 128, 0, c.stream>>>(
                  (const float*)q, (const float*)k, stats, dots, (float*)gq, (float*)gk, p.bh, p.nq,
                  p.nk, p.d, row_offset)));
  else
    FM_LAUNCH("fm_norm_fixup", c.stream,
              (norm_fixup_kernel<__nv_bfloat16><<<heads, 128, 0, c.stream>>>(
                  (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, stats, dots, (__nv_bfloat16*)gq,
                  (__nv_bfloat16*)gk, p.bh, p.nq, p.nk, p.d, row_offset)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

// ---------------------------------------------------------------------------
// Sequence sharding: after an all-gather of the per-shard moment totals into (world, floats), a shard
// needs the sum over the shards before it (forward, grad_q) or after it (grad_k, grad_v).  HBM-bound:
// reads (number of shards summed) x floats, writes floats; 16-byte accesses, grid-stride.
__global__ void __launch_bounds__(256) sum_totals_kernel(const float4* __restrict__ gathered, int first, int last,
                                                         size_t quads, float4* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (size_t)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = first; r < last; ++r) {
      const float4 v = __ldg(gathered + (size_t)r * quads + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    out[i] = acc;
  }
}

int launch_sum_totals(const float* gathered, int world, int rank, int reverse, size_t floats, float* out,
                      cudaStream_t stream) {
  const int first = reverse ? rank + 1 : 0, last = reverse ? world : rank;
  if (floats == 0) return FASTMAX_OK;
  if (floats % 4 != 0 || (((uintptr_t)gathered | (uintptr_t)out) & 15) != 0)
    return fail(FASTMAX_E_ARG, "totals must be 16-byte aligned and a multiple of 4 floats long");
  const size_t quads = floats / 4;
  const unsigned blocks = (unsigned)((quads + 255) / 256 < 148 * 8 ? (quads + 255) / 256 : 148 * 8);
  FM_LAUNCH("fm_sum_totals", stream,
            (sum_totals_kernel<<<blocks, 256, 0, stream>>>((const float4*)gathered, first, last, quads, (float4*)out)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

}  // namespace fm
