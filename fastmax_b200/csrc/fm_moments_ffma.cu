// Moment-state form of Fastmax attention on CUDA cores (fp32 math): the
// factorisation the reference evaluates (fastmax_cuda_forward.cu:25-197 for the
// first order, `old stuff/fastmax_cuda_forward_quad.cu`:57-268 for the second,
// and the matching backward files), restated as three data-parallel kernels
// instead of a serial walk over the sequence.
//
// With feature rows  phi(x) = [ x_a x_b (a,b < D) | x_a (a < D) | 1 ]  (F = D^2 + D + 1 rows)
// and value columns  zt = [ z_0 .. z_{D-1}, e ]  (e = 1 for key/value states,
// e = -grad_out.out/den for query/gradient states; DVP = D+1 rounded up to 4):
//
//   chunk_state   T_c[f][col] = sum_{j in chunk c} phi_f(y_j) zt_j[col]
//   prefix        P_c = base + sum_{c' < c} T_c'   (or the suffix sum), total = sum_c T_c
//   readout A     r_i[col] = sum_f w_f phi_f(x_i) P[f][col]            (numerator | denominator, grad_v)
//   readout B     r_i[a]   = sum_{b,col} k_b xe_i[b] P[(a,b)][col] ut_i[col]   (grad_q, grad_k)
//
// where the weights w = (A2 | A1 | A0) and k = (2 A2 | A1) carry the polynomial
// coefficients times the per-head normalisation scales, so q and k are read as
// stored.  States hold raw (unscaled) features.  The causal pass uses these
// kernels for everything before a token's own chunk and the score-form kernels
// for the chunk itself; the unmasked pass reads every token against the total.
#include "fm_common.cuh"

namespace fm {
namespace {

template <int D>
struct MC {
  static constexpr int DV = D + 1;
  static constexpr int DVP = (D + 1 + 3) / 4 * 4;
  static constexpr int F = D * D + D + 1;
  static constexpr int CW = DVP / 4;              // columns per thread (4 column groups)
  static constexpr int FPT = (D >= 128) ? 2 : 4;  // feature rows / tokens per thread
  static constexpr int TILE = 64 * FPT;           // feature rows (chunk_state) or tokens (readouts) per CTA
};

// row f of the state -> indices into xe = [x_0 .. x_{D-1}, 1] whose product is the feature
template <int D>
__device__ __forceinline__ void feature_index(int f, int& ia, int& ib) {
  if (f < D * D) { ia = f / D; ib = f % D; }
  else if (f < D * D + D) { ia = f - D * D; ib = D; }
  else { ia = D; ib = D; }
}

// Loads `rows` token rows of x into xe[row][D+1] (last entry 1), zero rows past n.
template <int D, typename T>
__device__ __forceinline__ void load_xe(float* xe, const T* x, int tok0, int rows, int n) {
  for (int idx = threadIdx.x; idx < rows * (D + 1); idx += blockDim.x) {
    const int r = idx / (D + 1), c = idx % (D + 1);
    const bool ok = tok0 + r < n;
    xe[idx] = (c == D) ? 1.f : (ok ? ldf(x + (size_t)(tok0 + r) * D + c) : 0.f);
  }
}
// Loads the extended value rows zt[row][DVP]; ext = 0: [z, 1]; ext = 1: [z/den, -delta/den].
// Rows past n and the padding columns are zero.
template <int D, typename T>
__device__ __forceinline__ void load_zt(float* zt, const T* z, const float* den, const float* delta,
                                        int ext, int tok0, int rows, int n) {
  constexpr int DVP = MC<D>::DVP;
  for (int idx = threadIdx.x; idx < rows * DVP; idx += blockDim.x) {
    const int r = idx / DVP, c = idx % DVP;
    const int tok = tok0 + r;
    float v = 0.f;
    if (tok < n && c <= D) {
      if (ext == 0) v = (c < D) ? ldf(z + (size_t)tok * D + c) : 1.f;
      else {
        const float inv = 1.0f / den[tok];
        v = (c < D) ? ldf(z + (size_t)tok * D + c) * inv : -delta[tok] * inv;
      }
    }
    zt[idx] = v;
  }
}

// ---------------------------------------------------------------------------------
struct StateArgs {
  const void* y;       // (heads, n, D) feature source
  const void* z;       // (heads, n, D) values
  const float* den;    // ext = 1: (heads, n)
  const float* delta;  // ext = 1: (heads, n)
  float* state;        // (heads, nchunk, F, DVP)
  int n, chunk, nchunk, ext, f_begin;
  int f_store;         // first row that is stored (d*d when p == 1: the second-order rows do not exist)
};

template <int D, typename T>
__global__ void __launch_bounds__(256) chunk_state_kernel(const StateArgs a) {
  using M = MC<D>;
  constexpr int TJ = 32;
  __shared__ float ye[TJ * (D + 1)];
  __shared__ float zt[TJ * M::DVP];
  const int head = blockIdx.z, chunk = blockIdx.y;
  const int fg = threadIdx.x >> 2, cg = threadIdx.x & 3;
  const int f0 = a.f_begin + blockIdx.x * M::TILE + fg * M::FPT;
  int ia[M::FPT], ib[M::FPT];
#pragma unroll
  for (int k = 0; k < M::FPT; ++k) feature_index<D>(min(f0 + k, M::F - 1), ia[k], ib[k]);
  float acc[M::FPT][M::CW];
#pragma unroll
  for (int k = 0; k < M::FPT; ++k)
#pragma unroll
    for (int c = 0; c < M::CW; ++c) acc[k][c] = 0.f;
  const T* y = (const T*)a.y + (size_t)head * a.n * D;
  const T* z = (const T*)a.z + (size_t)head * a.n * D;
  const float* den = a.den ? a.den + (size_t)head * a.n : nullptr;
  const float* delta = a.delta ? a.delta + (size_t)head * a.n : nullptr;
  const int t_end = min(a.n, (chunk + 1) * a.chunk);
  for (int t0 = chunk * a.chunk; t0 < t_end; t0 += TJ) {
    __syncthreads();
    load_xe<D, T>(ye, y, t0, TJ, t_end);
    load_zt<D, T>(zt, z, den, delta, a.ext, t0, TJ, t_end);
    __syncthreads();
#pragma unroll 4
    for (int j = 0; j < TJ; ++j) {
      float phi[M::FPT];
#pragma unroll
      for (int k = 0; k < M::FPT; ++k) phi[k] = ye[j * (D + 1) + ia[k]] * ye[j * (D + 1) + ib[k]];
#pragma unroll
      for (int c = 0; c < M::CW; ++c) {
        const float zv = zt[j * M::DVP + cg * M::CW + c];
#pragma unroll
        for (int k = 0; k < M::FPT; ++k) acc[k][c] = fmaf(phi[k], zv, acc[k][c]);
      }
    }
  }
  float* st = a.state + ((size_t)head * a.nchunk + chunk) * (M::F - a.f_store) * M::DVP;
#pragma unroll
  for (int k = 0; k < M::FPT; ++k) {
    const int f = f0 + k;
    if (f < M::F)
#pragma unroll
      for (int c = 0; c < M::CW; ++c) st[(size_t)(f - a.f_store) * M::DVP + cg * M::CW + c] = acc[k][c];
  }
}

// ---------------------------------------------------------------------------------
// Exclusive running sum over the chunks of every head (forward or reverse), started
// from `base` (per head, may be null); `total` (may be null) gets this shard's own sum.
// With write == 0 the states are left as they are and only the total is produced.
// One thread owns four consecutive state elements (`per` is a multiple of 4: the column count is).
__global__ void __launch_bounds__(256) prefix_kernel(float* state,
                                                     const float* __restrict__ base,
                                                     float* __restrict__ total, int nchunk,
                                                     size_t per, size_t first, int reverse,
                                                     int write) {
  const size_t e = first + ((size_t)blockIdx.x * 256 + threadIdx.x) * 4;
  const int head = blockIdx.y;
  if (e >= per) return;
  float4 run = base ? *(const float4*)(base + (size_t)head * per + e) : make_float4(0.f, 0.f, 0.f, 0.f);
  const float4 start = run;
  // batches of 8 chunks: the loads of a batch are independent and in flight together
  for (int i0 = 0; i0 < nchunk; i0 += 8) {
    float4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u;
      const int c = reverse ? nchunk - 1 - i : i;
      // without a total the last chunk in scan order is added to nothing that is kept (and may not have been built)
      v[u] = (i < nchunk && (total || i + 1 < nchunk))
                 ? __ldcs((const float4*)(state + ((size_t)head * nchunk + c) * per + e))
                 : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u;
      if (i < nchunk) {
        const int c = reverse ? nchunk - 1 - i : i;
        if (write) *(float4*)(state + ((size_t)head * nchunk + c) * per + e) = run;
        run.x += v[u].x; run.y += v[u].y; run.z += v[u].z; run.w += v[u].w;
      }
    }
  }
  if (total)
    *(float4*)(total + (size_t)head * per + e) =
        make_float4(run.x - start.x, run.y - start.y, run.z - start.z, run.w - start.w);
}

// ---------------------------------------------------------------------------------
struct ReadArgs {
  const void* x;        // (heads, n, D) tokens that read the state
  const float* state;   // (heads, nchunk, F, DVP) prefix states, or one total per head
  int state_per_chunk;  // 1: token t reads state[t / chunk]; 0: every token reads state[0]
  float* o_add;         // (heads, n, D) result (fp32)
  float* den_add;       // readout A: (heads, n) column D of the result, may be null
  const void* u;        // readout B: (heads, n, D) second token operand
  const float* den;     // readout B with ext = 1
  const float* delta;
  const stat_t* stat_q;
  const stat_t* stat_k;
  int n, chunk, nchunk, ext, f_begin, f_store;
  int accumulate;       // add to o_add / den_add instead of overwriting them
  float a0, a1, a2, lim;
};

// readout A: r_i[col] = sum_f w_f phi_f(x_i) P[f][col]
template <int D, typename T>
__global__ void __launch_bounds__(256) readout_a_kernel(const ReadArgs a) {
  using M = MC<D>;
  constexpr int FT = 32;  // state rows staged per step
  extern __shared__ float sm[];
  float* xe = sm;                           // [TILE][D+1]
  float* pt = xe + M::TILE * (D + 1);       // [FT][DVP]
  const int head = blockIdx.y, tok0 = blockIdx.x * M::TILE;
  const int tg = threadIdx.x >> 2, cg = threadIdx.x & 3;
  const float c = stat_scale(a.stat_q, head, a.lim) * stat_scale(a.stat_k, head, a.lim);
  const float A0 = a.a0, A1 = a.a1 * c, A2 = a.a2 * c * c;
  const int chunk = a.state_per_chunk ? tok0 / a.chunk : 0;
  const float* st = a.state + ((size_t)head * (a.state_per_chunk ? a.nchunk : 1) + chunk) * (M::F - a.f_store) * M::DVP
                    - (size_t)a.f_store * M::DVP;   // indexed by the absolute row number below
  load_xe<D, T>(xe, (const T*)a.x + (size_t)head * a.n * D, tok0, M::TILE, a.n);
  float acc[M::FPT][M::CW];
#pragma unroll
  for (int k = 0; k < M::FPT; ++k)
#pragma unroll
    for (int cc = 0; cc < M::CW; ++cc) acc[k][cc] = 0.f;
  for (int fb = a.f_begin; fb < M::F; fb += FT) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < FT * M::DVP; idx += 256) {
      const int f = fb + idx / M::DVP;
      pt[idx] = (f < M::F) ? st[(size_t)f * M::DVP + idx % M::DVP] : 0.f;
    }
    __syncthreads();
    const int fe = min(FT, M::F - fb);
    for (int fr = 0; fr < fe; ++fr) {
      const int f = fb + fr;
      int ia, ib;
      feature_index<D>(f, ia, ib);
      const float w = (f < D * D) ? A2 : ((f < D * D + D) ? A1 : A0);
      float phi[M::FPT];
#pragma unroll
      for (int k = 0; k < M::FPT; ++k) {
        const float* xr = xe + (tg * M::FPT + k) * (D + 1);
        phi[k] = w * xr[ia] * xr[ib];
      }
#pragma unroll
      for (int cc = 0; cc < M::CW; ++cc) {
        const float pv = pt[fr * M::DVP + cg * M::CW + cc];
#pragma unroll
        for (int k = 0; k < M::FPT; ++k) acc[k][cc] = fmaf(phi[k], pv, acc[k][cc]);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < M::FPT; ++k) {
    const int tok = tok0 + tg * M::FPT + k;
    if (tok >= a.n) continue;
    const size_t row = (size_t)head * a.n + tok;
#pragma unroll
    for (int cc = 0; cc < M::CW; ++cc) {
      const int col = cg * M::CW + cc;
      if (col < D) a.o_add[row * D + col] = acc[k][cc] + (a.accumulate ? a.o_add[row * D + col] : 0.f);
      else if (col == D && a.den_add) a.den_add[row] = acc[k][cc] + (a.accumulate ? a.den_add[row] : 0.f);
    }
  }
}

// readout B: r_i[a] = sum_{b <= D} kappa_b xe_i[b] sum_col P[row(a,b)][col] ut_i[col],
// row(a,b) = a D + b and kappa = 2 A2 for b < D; row(a,D) = D^2 + a and kappa = A1.
template <int D, typename T>
__global__ void __launch_bounds__(256) readout_b_kernel(const ReadArgs a) {
  using M = MC<D>;
  constexpr int AW = D / 4;  // output channels per thread, interleaved: a = m*4 + ag
  extern __shared__ float sm[];
  float* xe = sm;                          // [TILE][D+1]
  float* ut = xe + M::TILE * (D + 1);      // [TILE][DVP]
  float* pt = ut + M::TILE * M::DVP;       // [D][DVP]
  const int head = blockIdx.y, tok0 = blockIdx.x * M::TILE;
  const int tg = threadIdx.x >> 2, ag = threadIdx.x & 3;
  const float c = stat_scale(a.stat_q, head, a.lim) * stat_scale(a.stat_k, head, a.lim);
  const float A1 = a.a1 * c, A22 = 2.f * a.a2 * c * c;
  const int chunk = a.state_per_chunk ? tok0 / a.chunk : 0;
  const float* st = a.state + ((size_t)head * (a.state_per_chunk ? a.nchunk : 1) + chunk) * (M::F - a.f_store) * M::DVP
                    - (size_t)a.f_store * M::DVP;   // indexed by the absolute row number below
  load_xe<D, T>(xe, (const T*)a.x + (size_t)head * a.n * D, tok0, M::TILE, a.n);
  load_zt<D, T>(ut, (const T*)a.u + (size_t)head * a.n * D, a.den ? a.den + (size_t)head * a.n : nullptr,
                a.delta ? a.delta + (size_t)head * a.n : nullptr, a.ext, tok0, M::TILE, a.n);
  float acc[M::FPT][AW];
#pragma unroll
  for (int k = 0; k < M::FPT; ++k)
#pragma unroll
    for (int m = 0; m < AW; ++m) acc[k][m] = 0.f;
  const int b_begin = (a.f_begin >= D * D) ? D : 0;  // first order only: skip the quadratic rows
  for (int b = b_begin; b <= D; ++b) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < D * M::DVP; idx += 256) {
      const int ar = idx / M::DVP;
      const size_t row = (b < D) ? (size_t)ar * D + b : (size_t)D * D + ar;
      pt[idx] = st[row * M::DVP + idx % M::DVP];
    }
    __syncthreads();
    const float kappa = (b < D) ? A22 : A1;
    float xb[M::FPT];
#pragma unroll
    for (int k = 0; k < M::FPT; ++k) xb[k] = kappa * xe[(tg * M::FPT + k) * (D + 1) + b];
#pragma unroll 2
    for (int col = 0; col <= D; ++col) {
      float psi[M::FPT];
#pragma unroll
      for (int k = 0; k < M::FPT; ++k) psi[k] = xb[k] * ut[(tg * M::FPT + k) * M::DVP + col];
#pragma unroll
      for (int m = 0; m < AW; ++m) {
        const float pv = pt[(m * 4 + ag) * M::DVP + col];
#pragma unroll
        for (int k = 0; k < M::FPT; ++k) acc[k][m] = fmaf(psi[k], pv, acc[k][m]);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < M::FPT; ++k) {
    const int tok = tok0 + tg * M::FPT + k;
    if (tok >= a.n) continue;
    const size_t row = (size_t)head * a.n + tok;
#pragma unroll
    for (int m = 0; m < AW; ++m)
      a.o_add[row * D + m * 4 + ag] = acc[k][m] + (a.accumulate ? a.o_add[row * D + m * 4 + ag] : 0.f);
  }
}

// ---------------------------------------------------------------------------------
// Turns fp32 result rows into the output element type.  mode 0: out = num/den and den
// is written (unmasked forward); mode 1: plain conversion plus the per-head dot with x
// that the normalisation gradient needs (unmasked gradients).
template <typename T>
__global__ void __launch_bounds__(256) finalize_kernel(const float* __restrict__ r,
                                                       const float* __restrict__ den_in,
                                                       const T* __restrict__ x, T* __restrict__ out,
                                                       float* __restrict__ den_out,
                                                       float* __restrict__ dots, int n, int d,
                                                       int mode) {
  const int head = blockIdx.y;
  const size_t row0 = (size_t)head * n;
  float part = 0.f;
  for (size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x; idx < (size_t)n * d;
       idx += (size_t)gridDim.x * 256) {
    const size_t g = row0 * d + idx;
    float v = r[g];
    if (mode == 0) {
      const float dn = den_in[row0 + idx / d];
      v /= dn;
      if (idx % d == 0) den_out[row0 + idx / d] = dn;
    } else if (dots) {
      part = fmaf(v, ldf(x + g), part);
    }
    stf(out + g, v);
  }
  if (mode == 1 && dots) {
    // one atomic per CTA: thousands of them on one address per head serialise in L2
    __shared__ float warp_part[8];
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) part += __shfl_xor_sync(0xffffffffu, part, m);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) s += warp_part[w];
      atomicAdd(dots + head, s);
    }
  }
}

template <int D>
size_t readout_smem(bool b) {
  using M = MC<D>;
  size_t f = (size_t)M::TILE * (D + 1);
  if (b) f += (size_t)M::TILE * M::DVP + (size_t)D * M::DVP;
  else f += (size_t)32 * M::DVP;
  return f * sizeof(float);
}

}  // namespace

// ---- host-visible helpers ---------------------------------------------------------------
MomentDims moment_dims(int d, int p) {
  MomentDims m;
  m.dvp = (d + 1 + 3) / 4 * 4;
  m.f0 = (p == 1) ? d * d : 0;
  m.f = d * d + d + 1 - m.f0;
  return m;
}

#define FM_DISPATCH_D(d, CALL)                                                         \
  switch (d) {                                                                         \
    case 8: { constexpr int DD = 8; CALL; } break;                                     \
    case 16: { constexpr int DD = 16; CALL; } break;                                   \
    case 32: { constexpr int DD = 32; CALL; } break;                                   \
    case 64: { constexpr int DD = 64; CALL; } break;                                   \
    case 128: { constexpr int DD = 128; CALL; } break;                                 \
    default: return fail(FASTMAX_E_ARG, "head dimension %d is not one of 8,16,32,64,128", d); \
  }

int moments_chunk_state(const Ctx& c, int heads, int n, int chunk, const void* y, const void* z,
                        const float* den, const float* delta, int ext, float* state, int first_order_only) {
  if (heads == 0 || n == 0) return FASTMAX_OK;
  StateArgs a;
  a.y = y; a.z = z; a.den = den; a.delta = delta; a.state = state;
  a.n = n; a.chunk = chunk; a.nchunk = (n + chunk - 1) / chunk; a.ext = ext;
  a.f_begin = (c.p.p == 1 || first_order_only) ? c.p.d * c.p.d : 0;
  a.f_store = moment_dims(c.p.d, c.p.p).f0;
  const bool f32 = c.p.dtype == FASTMAX_F32;
  FM_DISPATCH_D(c.p.d, {
    using M = MC<DD>;
    dim3 grid((M::F - a.f_begin + M::TILE - 1) / M::TILE, a.nchunk, heads);
    if (f32) FM_LAUNCH("fm_moments_state", c.stream, (chunk_state_kernel<DD, float><<<grid, 256, 0, c.stream>>>(a)));
    else FM_LAUNCH("fm_moments_state", c.stream, (chunk_state_kernel<DD, __nv_bfloat16><<<grid, 256, 0, c.stream>>>(a)));
  });
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

int moments_prefix(const Ctx& c, int heads, int nchunk, float* state, const float* base, float* total,
                   int reverse, int write, int first_row) {
  if (heads == 0 || nchunk == 0) return FASTMAX_OK;
  const MomentDims m = moment_dims(c.p.d, c.p.p);
  const size_t per = (size_t)m.f * m.dvp;
  const size_t first = (size_t)first_row * m.dvp;   // rows before it are left alone (dvp is a multiple of 4)
  if ((((uintptr_t)state | (uintptr_t)base | (uintptr_t)total) & 15) != 0)
    return fail(FASTMAX_E_ARG, "moment states and totals must be 16-byte aligned");
  dim3 grid((unsigned)((per - first + 1023) / 1024), heads);   // four elements per thread
  FM_LAUNCH("fm_moments_prefix", c.stream,
            (prefix_kernel<<<grid, 256, 0, c.stream>>>(state, base, total, nchunk, per, first, reverse, write)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

int moments_readout(const Ctx& c, int mode_b, int heads, int n, int chunk, int state_per_chunk,
                    const void* x, const void* u, const float* den, const float* delta, int ext,
                    const float* state, const stat_t* stats, float* o_add, float* den_add,
                    int first_order_only) {
  if (heads == 0 || n == 0) return FASTMAX_OK;
  const fastmax_problem& p = c.p;
  ReadArgs a;
  a.x = x; a.state = state; a.state_per_chunk = state_per_chunk; a.o_add = o_add; a.den_add = den_add;
  a.u = u; a.den = den; a.delta = delta;
  a.stat_q = p.normalize ? stats : nullptr;
  a.stat_k = p.normalize ? stats + p.bh : nullptr;
  a.n = n; a.chunk = chunk; a.nchunk = (n + chunk - 1) / chunk; a.ext = ext;
  a.f_begin = (p.p == 1 || first_order_only) ? p.d * p.d : 0;
  a.f_store = moment_dims(p.d, p.p).f0;
  a.accumulate = first_order_only;   // the second-order part was written by the tensor-core read-out
  a.a0 = p.a0; a.a1 = p.a1; a.a2 = (p.p == 2) ? p.a2 : 0.f; a.lim = p.lim;
  const bool f32 = p.dtype == FASTMAX_F32;
  FM_DISPATCH_D(p.d, {
    using M = MC<DD>;
    dim3 grid((n + M::TILE - 1) / M::TILE, heads);
    const size_t sm = readout_smem<DD>(mode_b != 0);
    if (mode_b) {
      if (f32) {
        FM_CUDA_TRY(cudaFuncSetAttribute(readout_b_kernel<DD, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
        FM_LAUNCH("fm_moments_readout_b", c.stream, (readout_b_kernel<DD, float><<<grid, 256, sm, c.stream>>>(a)));
      } else {
        FM_CUDA_TRY(cudaFuncSetAttribute(readout_b_kernel<DD, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
        FM_LAUNCH("fm_moments_readout_b", c.stream, (readout_b_kernel<DD, __nv_bfloat16><<<grid, 256, sm, c.stream>>>(a)));
      }
    } else {
      if (f32) {
        FM_CUDA_TRY(cudaFuncSetAttribute(readout_a_kernel<DD, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
        FM_LAUNCH("fm_moments_readout_a", c.stream, (readout_a_kernel<DD, float><<<grid, 256, sm, c.stream>>>(a)));
      } else {
        FM_CUDA_TRY(cudaFuncSetAttribute(readout_a_kernel<DD, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
        FM_LAUNCH("fm_moments_readout_a", c.stream, (readout_a_kernel<DD, __nv_bfloat16><<<grid, 256, sm, c.stream>>>(a)));
      }
    }
  });
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

int moments_finalize(const Ctx& c, int heads, int n, const float* r, const float* den_in, const void* x,
                     void* out, float* den_out, float* dots, int mode) {
  if (heads == 0 || n == 0) return FASTMAX_OK;
  const int d = c.p.d;
  // enough CTAs to fill the device a few times over; with the per-head dot, few CTAs per head
  // when there are many heads, since each ends in an atomic on the head's word
  const size_t most = dots ? (size_t)max(8, (4096 + heads - 1) / heads) : (size_t)1024;
  dim3 grid((unsigned)min(most, ((size_t)n * d + 255) / 256), heads);
  if (c.p.dtype == FASTMAX_F32)
    FM_LAUNCH("fm_moments_finalize", c.stream,
              (finalize_kernel<float><<<grid, 256, 0, c.stream>>>(r, den_in, (const float*)x, (float*)out,
                                                                   den_out, dots, n, d, mode)));
  else
    FM_LAUNCH("fm_moments_finalize", c.stream,
              (finalize_kernel<__nv_bfloat16><<<grid, 256, 0, c.stream>>>(
                  r, den_in, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, den_out, dots, n, d, mode)));
  FM_CUDA_TRY(cudaGetLastError());
  return FASTMAX_OK;
}

}  // namespace fm
