// The transformer call site around the attention: packed qkv -> rotary
// embedding -> per-head q, k, v, and the way back.
//
// The reference's caller (model.py:472-499, 557-603) receives one projection
// `qkv` of shape (B, T, G, Q+2, hs) -- G key/value groups, Q query heads per
// group -- permutes it to (B, G, Q+2, T, hs), splits it, expands k and v to the
// query head count, rotates the first `rope_n` features of q and k
// (apply_rope, model.py:812-825) and calls `.contiguous()` on the three views
// (model.py:572-574) before the attention; the result (B, H, T, hs) is
// transposed back to (B, T, H, hs) (model.py:603).  That is a dozen elementwise
// passes over HBM.  Here each direction is one pass:
//
//   qkv_split_rope      reads qkv once, writes q (B*H, T, hs), k and v
//                       (B*G, T, hs; not expanded: the attention kernels take
//                       grouped heads) with the rotation applied in fp32;
//   qkv_merge_rope_grad reads grad_q, grad_k, grad_v once and writes the
//                       gradient of qkv with the transposed rotation;
//   swap_middle_axes    (B, X, Y, hs) -> (B, Y, X, hs), for the attention output
//                       and its incoming gradient;
//   scale_by_noise      y = x * (1 + dropout * noise), the reference's output
//                       dropout (fastmax_cuda_forward.cu:271-280).
//
// All four are HBM-bound copies: 16-byte accesses where the shapes allow (a
// rotated width that is only a multiple of 8 falls back to 8-byte accesses in
// bf16, so that a piece never straddles the two halves of the rotation), two
// to four pieces loaded per thread before the first store, 32-bit index
// arithmetic inside a token, grid-stride over a grid sized to the SM count.
// Measured on B200 in bf16 (B=8, T=4096, H=32, hs=64): split and merge move
// 806 MB in 0.23-0.24 ms (3.4-3.5 TB/s; 4.0 TB/s at hs=128), the axis swap and
// the noise scaling run at 5.4-5.6 TB/s.
#include "fm_common.cuh"

namespace fm {
namespace {

// V consecutive elements of type T moved as one access: 16 bytes (float x 4, bf16 x 8) or, where
// the rotated width is only a multiple of 8, bf16 x 4.
template <typename T, int V> struct Pack;
template <> struct Pack<float, 4> {
  float4 r;
  __device__ __forceinline__ void load(const float* p) { r = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = r; }
  __device__ __forceinline__ void get(float* f) const { f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w; }
  __device__ __forceinline__ void set(const float* f) { r = make_float4(f[0], f[1], f[2], f[3]); }
};
__device__ __forceinline__ void unpack2(unsigned w, float* f) {
  f[0] = __uint_as_float(w << 16);
  f[1] = __uint_as_float(w & 0xFFFF0000u);
}
__device__ __forceinline__ unsigned pack2(const float* f) {
  __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]);
  return *reinterpret_cast<unsigned*>(&a);
}
template <> struct Pack<__nv_bfloat16, 4> {
  uint2 r;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { r = *reinterpret_cast<const uint2*>(p); }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint2*>(p) = r; }
  __device__ __forceinline__ void get(float* f) const { unpack2(r.x, f); unpack2(r.y, f + 2); }
  __device__ __forceinline__ void set(const float* f) { r.x = pack2(f); r.y = pack2(f + 2); }
};
template <> struct Pack<__nv_bfloat16, 8> {
  uint4 r;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { r = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = r; }
  __device__ __forceinline__ void get(float* f) const {
    unpack2(r.x, f); unpack2(r.y, f + 2); unpack2(r.z, f + 4); unpack2(r.w, f + 6);
  }
  __device__ __forceinline__ void set(const float* f) {
    r.x = pack2(f); r.y = pack2(f + 2); r.z = pack2(f + 4); r.w = pack2(f + 6);
  }
};

struct SiteArgs {
  long long batch, n;   // B, T
  int groups, qper, d;  // G, Q, hs
  int rope;             // rotated leading features (0 = none), a multiple of 8
};

// Where the vector (b, t, g, j) of the packed projection lives in the per-head
// arrays: j < Q is query head g*Q+j, j == Q the group's key, j == Q+1 its value.
template <typename T>
__device__ __forceinline__ T* head_row(T* q, T* k, T* v, const SiteArgs& a, long long b, long long t, int g,
                                       int j) {
  if (j < a.qper) return q + (((b * a.groups + g) * a.qper + j) * a.n + t) * a.d;
  T* base = (j == a.qper) ? k : v;
  return base + ((b * a.groups + g) * a.n + t) * a.d;
}

constexpr int kInFlight = 2;  // pieces a thread loads before it computes and stores

// GRAD = false: per-head arrays <- packed projection, rotation R(t).
// GRAD = true : packed gradient <- per-head gradients, rotation R(t)^T.
// With x = (x1, x2) the two halves of the rotated features, cos = (c1, c2), sin = (s1, s2):
//   y1 = x1 c1 - x2 s1,  y2 = x2 c2 + x1 s2       (model.py:812-825)
//   gx1 = gy1 c1 + gy2 s2,  gx2 = gy2 c2 - gy1 s1
// One token (b, t) per CTA pass: its G*(Q+2) vectors are contiguous in the packed array, so the
// index arithmetic inside a token is 32-bit and the packed side is one contiguous run.
template <typename T, int V, bool GRAD>
__global__ void __launch_bounds__(256) qkv_site_kernel(const T* __restrict__ packed_in, T* __restrict__ packed_out,
                                                       T* __restrict__ q, T* __restrict__ k, T* __restrict__ v,
                                                       const float* __restrict__ cs, const float* __restrict__ sn,
                                                       const SiteArgs a) {
  const int qd = a.d / V, total = a.qper + 2, half = a.rope / 2;
  const int per_tok = a.groups * total * qd;  // V-element pieces per token
  const long long tokens = a.batch * a.n;
  for (long long bt = blockIdx.x; bt < tokens; bt += gridDim.x) {
    const long long b = bt / a.n, t = bt - b * a.n;
    const long long pbase = bt * (long long)per_tok * V;
    const float* ct = cs + t * a.rope;
    const float* st = sn + t * a.rope;
    for (int w0 = threadIdx.x; w0 < per_tok; w0 += kInFlight * blockDim.x) {
      Pack<T, V> x[kInFlight], y[kInFlight];
      T* dst[kInFlight];
      int c[kInFlight];
      bool rot[kInFlight], live[kInFlight];
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const int w = w0 + u * blockDim.x;
        live[u] = w < per_tok;
        rot[u] = false;
        if (!live[u]) continue;
        const int vec = w / qd;
        c[u] = (w - vec * qd) * V;
        const int g = vec / total, j = vec - g * total;
        T* hrow = head_row(q, k, v, a, b, t, g, j);
        const long long pvec = pbase + (long long)vec * a.d;  // start of the vector in the packed array
        const T* src = GRAD ? hrow : packed_in + pvec;
        dst[u] = (GRAD ? packed_out + pvec : hrow) + c[u];
        x[u].load(src + c[u]);
        rot[u] = c[u] < a.rope && j <= a.qper;
        if (rot[u]) y[u].load(src + (c[u] < half ? c[u] + half : c[u] - half));
      }
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        if (!live[u]) continue;
        if (rot[u]) {
          const bool lo = c[u] < half;
          const int pc = lo ? c[u] + half : c[u] - half;
          float xf[V], yf[V], cc[V], ss[V];
          x[u].get(xf);
          y[u].get(yf);
          // cos at the feature's own index; sin at its own index going forward, at the partner's going back
#pragma unroll
          for (int e = 0; e < V; e += 4) {
            const float4 c4 = *reinterpret_cast<const float4*>(ct + c[u] + e);
            const float4 s4 = *reinterpret_cast<const float4*>(st + (GRAD ? pc : c[u]) + e);
            cc[e] = c4.x; cc[e + 1] = c4.y; cc[e + 2] = c4.z; cc[e + 3] = c4.w;
            ss[e] = s4.x; ss[e + 1] = s4.y; ss[e + 2] = s4.z; ss[e + 3] = s4.w;
          }
          const float sign = (lo != GRAD) ? -1.0f : 1.0f;
#pragma unroll
          for (int e = 0; e < V; ++e) xf[e] = xf[e] * cc[e] + sign * yf[e] * ss[e];
          x[u].set(xf);
        }
        x[u].store(dst[u]);
      }
    }
  }
}

struct SwapArgs {
  long long batch, x, y;
  int d;
};

constexpr int kSwapPieces = 4;  // pieces per thread, all loaded before the first store

// dst[b, iy, ix, :] = src[b, ix, iy, :].  A source row (b, ix) is y*d contiguous elements; CTAs take
// chunks of 256 * kSwapPieces pieces of a row and write them as runs of d elements.
template <typename T, int V>
__global__ void __launch_bounds__(256) swap_axes_kernel(const T* __restrict__ src, T* __restrict__ dst,
                                                        const SwapArgs a, const long long chunks_per_row) {
  const int qd = a.d / V;
  const long long rows = a.batch * a.x, per_row = a.y * qd;
  for (long long cid = blockIdx.x; cid < rows * chunks_per_row; cid += gridDim.x) {
    const long long row = cid / chunks_per_row, chunk = cid - row * chunks_per_row;
    const long long b = row / a.x, ix = row - b * a.x;
    const T* s = src + row * per_row * V;
    T* d0 = dst + (b * a.y * a.x + ix) * a.d;
    Pack<T, V> v[kSwapPieces];
    long long w[kSwapPieces];
#pragma unroll
    for (int u = 0; u < kSwapPieces; ++u) {
      w[u] = chunk * (256 * kSwapPieces) + u * 256 + threadIdx.x;
      if (w[u] < per_row) v[u].load(s + w[u] * V);
    }
#pragma unroll
    for (int u = 0; u < kSwapPieces; ++u) {
      if (w[u] >= per_row) continue;
      const long long iy = w[u] / qd;
      const int c = (int)(w[u] - iy * qd) * V;
      v[u].store(d0 + iy * a.x * a.d + c);
    }
  }
}

constexpr int kVec = 4;  // elements per access of the noise kernel

template <typename T>
__global__ void __launch_bounds__(256) noise_kernel(const T* x, const T* __restrict__ noise, T* y, float dropout,
                                                    long long count) {  // y may be x
  const long long quads = count / kVec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < quads;
       idx += (long long)gridDim.x * blockDim.x) {
    Pack<T, 4> a, b;
    a.load(x + idx * kVec);
    b.load(noise + idx * kVec);
    float af[4], bf[4];
    a.get(af);
    b.get(bf);
#pragma unroll
    for (int e = 0; e < 4; ++e) af[e] *= 1.0f + dropout * bf[e];
    a.set(af);
    a.store(y + idx * kVec);
  }
  // ragged tail (count not a multiple of 4)
  for (long long i = quads * kVec + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x)
    stf(y + i, (float)x[i] * (1.0f + dropout * (float)noise[i]));
}

// The reference's packed forward result (rows of d + 1 floats, the denominator last): the first d
// channels of every row are scaled by 1 + dropout * noise, the denominator is left alone
// (reference apply_dropout, fastmax_cuda_forward.cu:271-280).  One thread per element of noise.
template <typename TN>
__global__ void __launch_bounds__(256) packed_noise_kernel(float* o, const TN* __restrict__ noise, float dropout,
                                                           long long rows, int d) {
  const long long count = rows * d;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / d;
    o[i + r] *= 1.0f + dropout * ldf(noise + i);
  }
}

int grid_for(long long work_items, int* blocks) {
  int dev = 0, sms = 0;
  FM_CUDA_TRY(cudaGetDevice(&dev));
  FM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const long long need = (work_items + 255) / 256;
  const long long cap = (long long)sms * 8;  // 8 CTAs of 256 threads per SM, grid-stride beyond that
  *blocks = (int)(need < 1 ? 1 : (need < cap ? need : cap));
  return FASTMAX_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int check_site(int dtype, long long batch, long long n, int groups, int qper, int d, int rope, const float* cs,
               const float* sn) {
  if (dtype != FASTMAX_F32 && dtype != FASTMAX_BF16)
    return fail(FASTMAX_E_ARG, "dtype %d is neither FASTMAX_F32 nor FASTMAX_BF16", dtype);
  if (batch < 0 || n < 0 || groups < 1 || qper < 1) return fail(FASTMAX_E_ARG, "bad batch, length, groups or heads per group");
  if (d < 8 || d % 8) return fail(FASTMAX_E_ARG, "head size %d is not a positive multiple of 8", d);
  if (rope < 0 || rope > d || rope % 8)
    return fail(FASTMAX_E_ARG, "rotated feature count %d is not a multiple of 8 within the head size %d", rope, d);
  if (rope && (!cs || !sn)) return fail(FASTMAX_E_ARG, "cos / sin tables are NULL");
  if (rope && (!aligned16(cs) || !aligned16(sn))) return fail(FASTMAX_E_ARG, "cos / sin tables are not 16-byte aligned");
  return FASTMAX_OK;
}

template <bool GRAD>
int launch_site(const void* packed_in, void* packed_out, void* q, void* k, void* v, const float* cs,
                const float* sn, long long batch, long long n, int groups, int qper, int d, int rope, int dtype,
                cudaStream_t st) {
  int rc = check_site(dtype, batch, n, groups, qper, d, rope, cs, sn);
  if (rc) return rc;
  const void* ptrs[] = {GRAD ? packed_out : packed_in, q, k, v};
  for (const void* p : ptrs) {
    if (!p) return fail(FASTMAX_E_ARG, "NULL array");
    if (!aligned16(p)) return fail(FASTMAX_E_ARG, "array is not 16-byte aligned");
  }
  SiteArgs a{batch, n, groups, qper, d, rope};
  if (batch * n == 0) return FASTMAX_OK;
  int blocks;
  if ((rc = grid_for(batch * n * 256, &blocks))) return rc;   // one CTA per token, grid-stride beyond the cap
  const char* name = GRAD ? "fm_qkv_merge_rope_grad" : "fm_qkv_split_rope";
  typedef __nv_bfloat16 bf;
  if (dtype == FASTMAX_F32)
    FM_LAUNCH(name, st, (qkv_site_kernel<float, 4, GRAD><<<blocks, 256, 0, st>>>(
                            (const float*)packed_in, (float*)packed_out, (float*)q, (float*)k, (float*)v, cs, sn, a)));
  else if (rope % 16 == 0)   // both halves of the rotated features are multiples of 8: 16-byte accesses
    FM_LAUNCH(name, st, (qkv_site_kernel<bf, 8, GRAD><<<blocks, 256, 0, st>>>(
                            (const bf*)packed_in, (bf*)packed_out, (bf*)q, (bf*)k, (bf*)v, cs, sn, a)));
  else
    FM_LAUNCH(name, st, (qkv_site_kernel<bf, 4, GRAD><<<blocks, 256, 0, st>>>(
                            (const bf*)packed_in, (bf*)packed_out, (bf*)q, (bf*)k, (bf*)v, cs, sn, a)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

}  // namespace
}  // namespace fm

using namespace fm;

int fastmax_b200_qkv_split_rope(const void* qkv, const float* cos_table, const float* sin_table, void* q, void* k,
                                void* v, long long batch, long long n, int groups, int q_per_group, int d,
                                int rope_n, int dtype, void* stream) {
  return launch_site<false>(qkv, nullptr, q, k, v, cos_table, sin_table, batch, n, groups, q_per_group, d, rope_n,
                            dtype, (cudaStream_t)stream);
}

int fastmax_b200_qkv_merge_rope_grad(const void* grad_q, const void* grad_k, const void* grad_v,
                                     const float* cos_table, const float* sin_table, void* grad_qkv,
                                     long long batch, long long n, int groups, int q_per_group, int d, int rope_n,
                                     int dtype, void* stream) {
  return launch_site<true>(nullptr, grad_qkv, const_cast<void*>(grad_q), const_cast<void*>(grad_k),
                           const_cast<void*>(grad_v), cos_table, sin_table, batch, n, groups, q_per_group, d,
                           rope_n, dtype, (cudaStream_t)stream);
}

int fastmax_b200_swap_middle_axes(const void* src, void* dst, long long batch, long long x, long long y, int d,
                                  int dtype, void* stream) {
  if (dtype != FASTMAX_F32 && dtype != FASTMAX_BF16)
    return fail(FASTMAX_E_ARG, "dtype %d is neither FASTMAX_F32 nor FASTMAX_BF16", dtype);
  if (batch < 0 || x < 0 || y < 0 || d < 8 || d % 8) return fail(FASTMAX_E_ARG, "bad shape");
  if (!src || !dst || !aligned16(src) || !aligned16(dst) || src == dst)
    return fail(FASTMAX_E_ARG, "arrays must be distinct, non-NULL and 16-byte aligned");
  SwapArgs a{batch, x, y, d};
  if (batch * x * y == 0) return FASTMAX_OK;
  const int v = dtype == FASTMAX_F32 ? 4 : 8;
  const long long per_row = y * (d / v);
  const long long chunks_per_row = (per_row + 256 * kSwapPieces - 1) / (256 * kSwapPieces);
  int blocks, rc;
  if ((rc = grid_for(batch * x * chunks_per_row * 256, &blocks))) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == FASTMAX_F32)
    FM_LAUNCH("fm_swap_axes", st, (swap_axes_kernel<float, 4><<<blocks, 256, 0, st>>>((const float*)src, (float*)dst,
                                                                                       a, chunks_per_row)));
  else
    FM_LAUNCH("fm_swap_axes", st, (swap_axes_kernel<__nv_bfloat16, 8><<<blocks, 256, 0, st>>>(
                                      (const __nv_bfloat16*)src, (__nv_bfloat16*)dst, a, chunks_per_row)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

int fastmax_b200_scale_by_noise(const void* x, const void* noise, void* y, float dropout, size_t count, int dtype,
                                void* stream) {
  if (dtype != FASTMAX_F32 && dtype != FASTMAX_BF16)
    return fail(FASTMAX_E_ARG, "dtype %d is neither FASTMAX_F32 nor FASTMAX_BF16", dtype);
  if (count == 0) return FASTMAX_OK;
  if (!x || !noise || !y || !aligned16(x) || !aligned16(noise) || !aligned16(y))
    return fail(FASTMAX_E_ARG, "arrays must be non-NULL and 16-byte aligned");
  int blocks, rc;
  if ((rc = grid_for((long long)(count / kVec + 1), &blocks))) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == FASTMAX_F32)
    FM_LAUNCH("fm_scale_by_noise", st, (noise_kernel<float><<<blocks, 256, 0, st>>>(
                                           (const float*)x, (const float*)noise, (float*)y, dropout, (long long)count)));
  else
    FM_LAUNCH("fm_scale_by_noise", st,
              (noise_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)noise,
                                                                   (__nv_bfloat16*)y, dropout, (long long)count)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}
int fastmax_b200_scale_packed_by_noise(float* o_packed, const void* noise, float dropout, long long rows, int d,
                                       int noise_dtype, void* stream) {
  if (noise_dtype != FASTMAX_F32 && noise_dtype != FASTMAX_BF16)
    return fail(FASTMAX_E_ARG, "dtype %d is neither FASTMAX_F32 nor FASTMAX_BF16", noise_dtype);
  if (rows < 0 || d <= 0) return fail(FASTMAX_E_ARG, "bad shape");
  if (rows == 0) return FASTMAX_OK;
  if (!o_packed || !noise) return fail(FASTMAX_E_ARG, "NULL array");
  int blocks, rc;
  if ((rc = grid_for(rows * d, &blocks))) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (noise_dtype == FASTMAX_F32)
    FM_LAUNCH("fm_scale_packed_by_noise", st,
              (packed_noise_kernel<float><<<blocks, 256, 0, st>>>(o_packed, (const float*)noise, dropout, rows, d)));
  else
    FM_LAUNCH("fm_scale_packed_by_noise", st,
              (packed_noise_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(o_packed, (const __nv_bfloat16*)noise,
                                                                          dropout, rows, d)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}
