// Token-by-token (decode) Fastmax attention against a persistent moment state.
//
// The reference's model decodes with a key/value cache: every new token calls the
// attention with one query row and all cached keys (model.py:501-504, 828-852), so
// the cost per token grows with the length.  The factorised form needs no cache:
// per key/value head keep
//
//   S0[c]       = sum_j            vt_j[c]
//   S1[a][c]    = sum_j k_j[a]     vt_j[c]
//   S2[a][b][c] = sum_j k_j[a] k_j[b] vt_j[c]          (p = 2 only)
//
// with vt_j = (v_j, 1), over the RAW keys; the max-norm scaling lim / max_j |k_j|
// multiplies whole blocks (S1 by s, S2 by s^2), so it is applied when a query reads
// the state and the running maximum is one float in the state's header.  A query
// row is normalised by its own norm, as it is when the reference's attention is
// called with a single query row.  One step adds the new token to the state and
// reads it:  num[c] = a0 S0[c] + a1 s (q.S1)[c] + a2 s^2 (q(x)q . S2)[c],
// out = num[:d] / num[d]  -- the last row of causal attention over the tokens so far
// (fastmax_cuda_forward.cu:109, 132-150 with nq = 1).
//
// The state is fp32, F = (d^2 +) d + 1 rows of d+1 floats (second-order rows first, the
// constant row last) after a 4-word header {max |k|^2, token count (int32 bits), 0, 0} per key/value head.
// A step reads and writes it once: HBM-bound, 2 * 4 * F * (d+1) bytes per key/value head
// per token, independent of the length.  A thread owns one column c of one block of rows
// (a CTA's threads cover whole rows, so state accesses are contiguous), keeps the block
// in registers across the tokens of a call, and adds its share of the read-out to a small
// fp32 array with one atomicAdd per (query head, column, CTA).  Measured on B200 (1024
// heads, d = 64, p = 2, bf16 inputs): 0.50 ms per token for the 1.11 GB state, 4.4 TB/s.
#include "fm_common.cuh"

namespace fm {
namespace {

constexpr int kBlockA = 4;      // a thread's block of state rows: 4 values of a ...
constexpr int kBlockB = 16;     // ... times 16 consecutive values of b
constexpr int kTokBatch = 32;   // tokens staged in shared memory per pass (prompt processing)
constexpr int kHeader = 4;

struct DecArgs {
  int bh, bhkv, ratio, p, normalize;
  float a0, a1, a2, lim;
  long long n_new;       // tokens to add
  int rows;              // F
  long long head_floats; // kHeader + F * (d + 1)
};

template <int D> struct DecCfg {
  static constexpr int DV = D + 1;
  static constexpr int RPB = 256 / DV;          // row blocks per CTA
  static constexpr int THREADS = RPB * DV;
  static constexpr int KS = D + 16;             // (k, 1, 0 x 15): a 16-float window may start at D
  static constexpr int NB2 = (D / kBlockA) * (D / kBlockB);   // second-order blocks per head
  static constexpr int NB1 = D / kBlockB;                     // first-order blocks per head
};

// Sum of squares of x[0..D) by one warp; the result is valid in every lane.
template <int D>
__device__ __forceinline__ float warp_norm2(const float* x, int lane) {
  float n2 = 0.0f;
#pragma unroll
  for (int e = lane; e < D; e += 32) n2 = fmaf(x[e], x[e], n2);
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) n2 += __shfl_xor_sync(0xffffffffu, n2, m);
  return n2;
}

// 16 bytes of T from global memory as fp32 values.
__device__ __forceinline__ void load16_to_f32(const float* src, float* dst) {
  const float4 w = __ldg(reinterpret_cast<const float4*>(src));
  dst[0] = w.x; dst[1] = w.y; dst[2] = w.z; dst[3] = w.w;
}
__device__ __forceinline__ void load16_to_f32(const __nv_bfloat16* src, float* dst) {
  const uint4 w = __ldg(reinterpret_cast<const uint4*>(src));
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    dst[2 * e] = __uint_as_float(ww[e] << 16);
    dst[2 * e + 1] = __uint_as_float(ww[e] & 0xFFFF0000u);
  }
}

// Row order of a head's state: the d*d second-order rows (a, b) first (p = 2), then the d
// first-order rows, then the constant row.  A thread owns one column c of one block of rows:
// (a0..a0+3) x (b0..b0+15) of the second order, or 16 first-order rows, or the constant row.
// feature(a, b) = kx[a] * kx[b] with kx = (k, 1, 0, ...): per token the thread forms four
// products kx[a] * vt[c] and reads 16 values kx[b] (five 16-byte shared-memory loads and one
// scalar one) for its 64 multiply-adds, so prompt processing is bound by the FMA pipe rather
// than by shared memory; a decode step just streams the 64 accumulators through once.
template <typename T, int D, bool READ>
__global__ void __launch_bounds__(DecCfg<D>::THREADS) decode_kernel(const DecArgs a, const T* __restrict__ q,
                                                                    const T* __restrict__ k, const T* __restrict__ v,
                                                                    float* __restrict__ state, float* __restrict__ num) {
  typedef DecCfg<D> C;
  __shared__ __align__(16) float ks[kTokBatch][C::KS];
  __shared__ float vs[kTokBatch][D + 1];   // (v, 1)
  __shared__ float red[C::RPB][C::DV];
  __shared__ float s_q2;
  __shared__ int s_kmax2_bits;   // max |k|^2 as its bit pattern: non-negative floats order like integers
  const int tid = threadIdx.x, r = tid / C::DV, c = tid - r * C::DV, lane = tid & 31;
  const int head = blockIdx.y;
  float* hs = state + head * a.head_floats;

  // this thread's block
  const int nb2 = (a.p == 2) ? C::NB2 : 0, n2rows = (a.p == 2) ? D * D : 0;
  const int sb = blockIdx.x * C::RPB + r;
  int a0 = D, b0 = D, kind = 0, nu = 0, ni = 0;   // nu x ni valid rows
  int row00 = 0, ustride = 0;                     // row of (u, i) = row00 + u * ustride + i
  if (sb < nb2) {
    a0 = (sb / C::NB1) * kBlockA; b0 = (sb % C::NB1) * kBlockB; kind = 2; nu = kBlockA; ni = kBlockB;
    row00 = a0 * D + b0; ustride = D;
  } else if (sb < nb2 + C::NB1) {
    b0 = (sb - nb2) * kBlockB; kind = 1; nu = 1; ni = kBlockB; row00 = n2rows + b0;
  } else if (sb == nb2 + C::NB1) {
    nu = 1; ni = 1; row00 = n2rows + D;           // the constant row: kx[D] * kx[D] = 1
  }

  float* const base = hs + kHeader + (long long)row00 * C::DV + c;   // row (u, i) at base[(u * ustride + i) * DV]
  const int ustep = ustride * C::DV;
  float s[kBlockA][kBlockB];
#pragma unroll
  for (int u = 0; u < kBlockA; ++u) {
    const float* pu = base + u * ustep;
#pragma unroll
    for (int i = 0; i < kBlockB; ++i) s[u][i] = (u < nu && i < ni) ? pu[i * C::DV] : 0.0f;
  }
  if (tid == 0) s_kmax2_bits = __float_as_int(hs[0]);
  __syncthreads();

  const T* kh = k + (long long)head * a.n_new * D;
  const T* vh = v + (long long)head * a.n_new * D;
  for (long long t0 = 0; t0 < a.n_new; t0 += kTokBatch) {
    const int nt = (int)((a.n_new - t0 < kTokBatch) ? a.n_new - t0 : kTokBatch);
    // stage the batch: 16-byte loads of k and v, converted to fp32; then the (1, 0, ...) tails
    constexpr int EPV = 16 / (int)sizeof(T), VPT = D / EPV;   // elements per load, loads per token
    for (int e = tid; e < nt * VPT; e += C::THREADS) {
      const int tok = e / VPT, x = (e - tok * VPT) * EPV;
      load16_to_f32(kh + (t0 + tok) * D + x, &ks[tok][x]);
      load16_to_f32(vh + (t0 + tok) * D + x, &vs[tok][x]);
    }
    for (int e = tid; e < nt * 16; e += C::THREADS) {
      const int tok = e >> 4, j = e & 15;
      ks[tok][D + j] = j == 0 ? 1.0f : 0.0f;
      if (j == 0) vs[tok][D] = 1.0f;
    }
    __syncthreads();
    {   // running maximum of |k|^2, the tokens spread over the CTA's full warps
      constexpr int kFullWarps = C::THREADS / 32;
      const int warp = tid >> 5;
      if (warp < kFullWarps) {
        float m = 0.0f;
        for (int tok = warp; tok < nt; tok += kFullWarps) m = fmaxf(m, warp_norm2<D>(ks[tok], lane));
        if (lane == 0) atomicMax(&s_kmax2_bits, __float_as_int(m));
      }
    }
    for (int tok = 0; tok < nt; ++tok) {
      const float vc = vs[tok][c];
      const float4 ka = *reinterpret_cast<const float4*>(&ks[tok][a0]);   // (1, 0, 0, 0) when a0 == D
      const float t[kBlockA] = {ka.x * vc, ka.y * vc, ka.z * vc, ka.w * vc};
      const float4* kb = reinterpret_cast<const float4*>(&ks[tok][b0]);
#pragma unroll
      for (int i4 = 0; i4 < kBlockB / 4; ++i4) {
        const float4 b4 = kb[i4];
#pragma unroll
        for (int u = 0; u < kBlockA; ++u) {
          s[u][4 * i4 + 0] = fmaf(t[u], b4.x, s[u][4 * i4 + 0]);
          s[u][4 * i4 + 1] = fmaf(t[u], b4.y, s[u][4 * i4 + 1]);
          s[u][4 * i4 + 2] = fmaf(t[u], b4.z, s[u][4 * i4 + 2]);
          s[u][4 * i4 + 3] = fmaf(t[u], b4.w, s[u][4 * i4 + 3]);
        }
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int u = 0; u < kBlockA; ++u) {
    float* pu = base + u * ustep;
#pragma unroll
    for (int i = 0; i < kBlockB; ++i)
      if (u < nu && i < ni) pu[i * C::DV] = s[u][i];
  }
  // every CTA of the head holds the same maximum; the first one records it
  if (blockIdx.x == 0 && tid == 0) {
    hs[0] = __int_as_float(s_kmax2_bits);
    // the token count is an integer bit pattern in the float slot: exact past 2^24 tokens
    hs[1] = __int_as_float(__float_as_int(hs[1]) + (int)a.n_new);
  }
  if (!READ) return;

  float* qx = &ks[0][0];   // (q, 1, 0 x 15), reusing the key staging
  for (int g = 0; g < a.ratio; ++g) {
    const int qh = head * a.ratio + g;
    __syncthreads();
    for (int x = tid; x < C::KS; x += C::THREADS) qx[x] = x < D ? ldf(q + (long long)qh * D + x) : (x == D ? 1.0f : 0.0f);
    __syncthreads();
    if (tid < 32) {
      const float n2 = warp_norm2<D>(qx, lane);
      if (lane == 0) s_q2 = n2;
    }
    __syncthreads();
    const float sc = a.normalize ? (a.lim * rsqrtf(s_q2)) * (a.lim * rsqrtf(__int_as_float(s_kmax2_bits))) : 1.0f;
    const float coef = kind == 0 ? a.a0 : (kind == 1 ? a.a1 * sc : a.a2 * sc * sc);
    float part = 0.0f;
#pragma unroll
    for (int u = 0; u < kBlockA; ++u) {
      const float cu = coef * qx[a0 + u];
#pragma unroll
      for (int i = 0; i < kBlockB; ++i) part = fmaf((u < nu && i < ni) ? cu * qx[b0 + i] : 0.0f, s[u][i], part);
    }
    red[r][c] = part;
    __syncthreads();
    if (r == 0) {
      float tot = 0.0f;
#pragma unroll
      for (int rr = 0; rr < C::RPB; ++rr) tot += red[rr][c];
      atomicAdd(num + (long long)qh * C::DV + c, tot);
    }
  }
}

template <typename T, int D>
__global__ void decode_finish_kernel(const float* __restrict__ num, T* __restrict__ out, int bh) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= bh * D) return;
  const int h = idx / D, c = idx - h * D;
  stf(out + idx, num[(long long)h * (D + 1) + c] / num[(long long)h * (D + 1) + D]);
}

int rows_of(const fastmax_problem& p) { return 1 + p.d + (p.p == 2 ? p.d * p.d : 0); }

int check_decode(const fastmax_problem* prob) {
  int rc = check_problem(prob);
  if (rc) return rc;
  if (prob->d != 32 && prob->d != 64 && prob->d != 128)
    return fail(FASTMAX_E_ARG, "the decode state supports head dimensions 32, 64 and 128, got %d", prob->d);
  return FASTMAX_OK;
}

template <typename T, int D, bool READ>
int launch_decode(const fastmax_problem& p, const void* q, const void* k, const void* v, long long n_new,
                  float* state, float* num, void* out, cudaStream_t st) {
  typedef DecCfg<D> C;
  DecArgs a{p.bh, p.bhkv, p.bhkv ? p.bh / p.bhkv : 1, p.p, p.normalize, p.a0, p.a1, p.a2, p.lim, n_new, rows_of(p),
            kHeader + (long long)rows_of(p) * (D + 1)};
  if (p.bhkv == 0) return FASTMAX_OK;
  if (READ) FM_CUDA_TRY(cudaMemsetAsync(num, 0, sizeof(float) * (size_t)p.bh * (D + 1), st));
  const int blocks_per_head = (p.p == 2 ? C::NB2 : 0) + C::NB1 + 1;
  dim3 grid((blocks_per_head + C::RPB - 1) / C::RPB, p.bhkv);
  FM_LAUNCH(READ ? "fm_decode_step" : "fm_decode_append", st,
            (decode_kernel<T, D, READ><<<grid, C::THREADS, 0, st>>>(a, (const T*)q, (const T*)k, (const T*)v, state, num)));
  FM_CUDA_TRY(cudaGetLastError());
  if (READ) {
    const int total = p.bh * D;
    FM_LAUNCH("fm_decode_finish", st,
              (decode_finish_kernel<T, D><<<(total + 255) / 256, 256, 0, st>>>(num, (T*)out, p.bh)));
    FM_CUDA_TRY(cudaGetLastError());
  }
  return FASTMAX_OK;
}

template <bool READ>
int dispatch_decode(const fastmax_problem& p, const void* q, const void* k, const void* v, long long n_new,
                    float* state, float* num, void* out, cudaStream_t st) {
#define FM_DEC(TT, DD) return launch_decode<TT, DD, READ>(p, q, k, v, n_new, state, num, out, st)
  if (p.dtype == FASTMAX_F32) {
    if (p.d == 32) FM_DEC(float, 32);
    if (p.d == 64) FM_DEC(float, 64);
    FM_DEC(float, 128);
  }
  if (p.d == 32) FM_DEC(__nv_bfloat16, 32);
  if (p.d == 64) FM_DEC(__nv_bfloat16, 64);
  FM_DEC(__nv_bfloat16, 128);
#undef FM_DEC
}

}  // namespace
}  // namespace fm

using namespace fm;

size_t fastmax_b200_decode_state_bytes(const fastmax_problem* prob) {
  if (!prob || prob->bhkv < 0 || prob->d <= 0) return 0;
  return sizeof(float) * (size_t)prob->bhkv * (kHeader + (size_t)rows_of(*prob) * (prob->d + 1));
}

size_t fastmax_b200_decode_scratch_bytes(const fastmax_problem* prob) {
  if (!prob || prob->bh < 0 || prob->d <= 0) return 0;
  return sizeof(float) * (size_t)prob->bh * (prob->d + 1);
}

int fastmax_b200_decode_append(const fastmax_problem* prob, const void* k, const void* v, long long n_new,
                               void* state, void* stream) {
  int rc = check_decode(prob);
  if (rc) return rc;
  if (n_new < 0) return fail(FASTMAX_E_ARG, "negative token count");
  if (n_new == 0 || prob->bhkv == 0) return FASTMAX_OK;
  if (!k || !v || !state) return fail(FASTMAX_E_ARG, "NULL array");
  if (((uintptr_t)k | (uintptr_t)v) & 15) return fail(FASTMAX_E_ARG, "k and v must be 16-byte aligned");
  return dispatch_decode<false>(*prob, nullptr, k, v, n_new, (float*)state, nullptr, nullptr, (cudaStream_t)stream);
}

int fastmax_b200_decode_step(const fastmax_problem* prob, const void* q, const void* k, const void* v, void* state,
                             void* scratch, void* out, void* stream) {
  int rc = check_decode(prob);
  if (rc) return rc;
  if (prob->bh == 0) return FASTMAX_OK;
  if (!q || !k || !v || !state || !scratch || !out) return fail(FASTMAX_E_ARG, "NULL array");
  if (((uintptr_t)k | (uintptr_t)v) & 15) return fail(FASTMAX_E_ARG, "k and v must be 16-byte aligned");
  return dispatch_decode<true>(*prob, q, k, v, 1, (float*)state, (float*)scratch, out, (cudaStream_t)stream);
}
