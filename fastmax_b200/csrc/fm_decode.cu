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
// The state is fp32, F = (d^2 +) d + 1 rows of d+1 floats (second-order rows first, the constant
// row last) after a 4-float header {max |k|^2, tokens, 0, 0} per key/value head.  A step reads and writes it once:
// HBM-bound, 2 * 4 * F * (d+1) bytes per key/value head per token, independent of
// the length.  CTAs take slices of rows; a thread owns one column c of a few rows
// (a CTA's threads cover whole rows, so state accesses are contiguous), keeps
// them in registers across the tokens of a call, and adds its share of the
// read-out to a small fp32 array with one atomicAdd per (query head, column, CTA).
#include "fm_common.cuh"

namespace fm {
namespace {

constexpr int kIter = 16;      // state rows per thread: one aligned block of 16 consecutive rows
constexpr int kTokBatch = 32;  // tokens staged in shared memory per pass (prompt processing)
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
  static constexpr int RPB = 256 / DV;          // 16-row blocks per CTA
  static constexpr int THREADS = RPB * DV;
  static constexpr int ROWS = RPB * kIter;      // rows per CTA
  static constexpr int KS = D + 16;             // (k, 1, 0 x 15): a 16-float window may start at D
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

// Row order of a head's state: the d*d second-order rows (a, b) first (p = 2), then the d
// first-order rows, then the constant row.  d is a multiple of 16, so every aligned block of 16
// rows has one `a` and 16 consecutive `b`: feature(row i of the block) = kx[ia] * kx[ib0 + i] with
// kx = (k, 1, 0, ...).  A thread owns one column c of one block: per token one product
// kx[ia] * vt[c] and four 16-byte shared-memory loads feed its 16 multiply-adds.
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
  const int blk = blockIdx.x * C::ROWS + r * kIter;   // first row of this thread's block
  float* hs = state + head * a.head_floats;

  const int n2rows = (a.p == 2) ? D * D : 0;
  int ia = D, ib0 = D, kind = 0;                      // the constant row (and padding behind it)
  if (blk < n2rows) { ia = blk / D; ib0 = blk % D; kind = 2; }
  else if (blk < n2rows + D) { ib0 = blk - n2rows; kind = 1; }

  float s[kIter];
#pragma unroll
  for (int i = 0; i < kIter; ++i) s[i] = (blk + i < a.rows) ? hs[kHeader + (long long)(blk + i) * C::DV + c] : 0.0f;
  if (tid == 0) s_kmax2_bits = __float_as_int(hs[0]);
  __syncthreads();

  const T* kh = k + (long long)head * a.n_new * D;
  const T* vh = v + (long long)head * a.n_new * D;
  for (long long t0 = 0; t0 < a.n_new; t0 += kTokBatch) {
    const int nt = (int)((a.n_new - t0 < kTokBatch) ? a.n_new - t0 : kTokBatch);
    for (int e = tid; e < nt * C::KS; e += C::THREADS) {
      const int tok = e / C::KS, x = e - tok * C::KS;
      ks[tok][x] = x < D ? ldf(kh + (t0 + tok) * D + x) : (x == D ? 1.0f : 0.0f);
      if (x <= D) vs[tok][x] = x < D ? ldf(vh + (t0 + tok) * D + x) : 1.0f;
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
#pragma unroll 2
    for (int tok = 0; tok < nt; ++tok) {
      const float t = ks[tok][ia] * vs[tok][c];
      const float4* kb = reinterpret_cast<const float4*>(&ks[tok][ib0]);
#pragma unroll
      for (int i4 = 0; i4 < kIter / 4; ++i4) {
        const float4 b4 = kb[i4];
        s[4 * i4 + 0] = fmaf(t, b4.x, s[4 * i4 + 0]);
        s[4 * i4 + 1] = fmaf(t, b4.y, s[4 * i4 + 1]);
        s[4 * i4 + 2] = fmaf(t, b4.z, s[4 * i4 + 2]);
        s[4 * i4 + 3] = fmaf(t, b4.w, s[4 * i4 + 3]);
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < kIter; ++i)
    if (blk + i < a.rows) hs[kHeader + (long long)(blk + i) * C::DV + c] = s[i];
  // every CTA of the head holds the same maximum; the first one records it
  if (blockIdx.x == 0 && tid == 0) {
    hs[0] = __int_as_float(s_kmax2_bits);
    hs[1] += (float)a.n_new;
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
    const float coef = (kind == 0 ? a.a0 : (kind == 1 ? a.a1 * sc : a.a2 * sc * sc)) * qx[ia];
    float part = 0.0f;
#pragma unroll
    for (int i = 0; i < kIter; ++i) part = fmaf((blk + i < a.rows) ? coef * qx[ib0 + i] : 0.0f, s[i], part);
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
  dim3 grid((a.rows + C::ROWS - 1) / C::ROWS, p.bhkv);
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
  return dispatch_decode<false>(*prob, nullptr, k, v, n_new, (float*)state, nullptr, nullptr, (cudaStream_t)stream);
}

int fastmax_b200_decode_step(const fastmax_problem* prob, const void* q, const void* k, const void* v, void* state,
                             void* scratch, void* out, void* stream) {
  int rc = check_decode(prob);
  if (rc) return rc;
  if (prob->bh == 0) return FASTMAX_OK;
  if (!q || !k || !v || !state || !scratch || !out) return fail(FASTMAX_E_ARG, "NULL array");
  return dispatch_decode<true>(*prob, q, k, v, 1, (float*)state, (float*)scratch, out, (cudaStream_t)stream);
}
