// Shared declarations of the fastmax_b200 library (internal).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fastmax_b200.h"

namespace fm {

// Records the calling thread's error message and returns `code`.
int fail(int code, const char* fmt, ...);

#define FM_CUDA_TRY(expr)                                                              \
  do {                                                                                 \
    cudaError_t _e = (expr);                                                           \
    if (_e != cudaSuccess)                                                             \
      return ::fm::fail(FASTMAX_E_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

// ---- launch accounting ------------------------------------------------------
// Every kernel launch of the library goes through FM_LAUNCH: it counts the
// launch and, while profiling is enabled, brackets it with CUDA events on the
// launch stream so a caller can read per-kernel device times afterwards.
void prof_before(const char* name, cudaStream_t s);
void prof_after(cudaStream_t s);
#define FM_LAUNCH(name, stream, ...)      \
  do {                                    \
    ::fm::prof_before(name, stream);      \
    __VA_ARGS__;                          \
    ::fm::prof_after(stream);             \
  } while (0)

// ---- element access -------------------------------------------------------
__device__ __forceinline__ float ldf(const float* p) { return __ldg(p); }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// ---- per-head statistics ---------------------------------------------------
// One 64-bit word per head: high 32 bits = bit pattern of max_n ||x_n||^2 (a
// non-negative float, so unsigned order equals numeric order), low 32 bits =
// 0xFFFFFFFF - row index, so an atomicMax keeps the largest norm and, among
// equal norms, the lowest row.  Words of q heads come first, then k heads.
typedef unsigned long long stat_t;

__host__ __device__ __forceinline__ float stat_norm2(stat_t s) {
#ifdef __CUDA_ARCH__
  return __uint_as_float((unsigned)(s >> 32));
#else
  union { unsigned u; float f; } c;
  c.u = (unsigned)(s >> 32);
  return c.f;
#endif
}
__host__ __device__ __forceinline__ int stat_row(stat_t s) {
  return (int)(0xFFFFFFFFu - (unsigned)(s & 0xFFFFFFFFull));
}
// lim / max_n ||x_n||  (1 when the problem is not normalised: st == nullptr)
__device__ __forceinline__ float stat_scale(const stat_t* st, int head, float lim) {
  return st ? lim / sqrtf(stat_norm2(st[head])) : 1.0f;
}

// FASTMAX_OK if the problem description is valid, else the error code (message recorded).
int check_problem(const fastmax_problem* p);

// ---- kernel launchers (each returns FASTMAX_OK or an error code) ------------
struct Ctx {
  fastmax_problem p;
  cudaStream_t stream;
  // > 0: the forward's result and the upstream gradient are (batch, n, out_heads, d) arrays -- the
  // layout the model's output projection consumes -- instead of (batch * out_heads, n, d); only the
  // tensor-core score kernels and the gradient preparation pass honour it (see fastmax_b200_forward_bt)
  int out_heads = 0;
  // Causal moment family, one call for the whole sequence: the chunk whose state nothing reads (the last
  // one in scan order: no later chunk exists and no total is asked for) is not built, and the tokens of
  // the chunk whose running sum is empty (the first in scan order, when no base is added) get zeros
  // without a read-out.  -1: no such chunk.  Honoured by the tensor-core moment kernels.
  int skip_chunk = -1;
  int zero_chunk = -1;
};
// Row of head `head`, token `row` in a (heads, n, .) array, or in a (batch, n, out_heads, .) array
__host__ __device__ __forceinline__ size_t out_row(int head, int row, int n, int out_heads) {
  return out_heads > 0 ? ((size_t)(head / out_heads) * n + row) * out_heads + head % out_heads
                       : (size_t)head * n + row;
}

// Row statistics of q and k into `stats` (zeroes it first).
// row_offset is added to the row indices that are recorded (a sequence shard's first token).
int launch_rowmax(const Ctx& c, const void* q, const void* k, stat_t* stats, int row_offset = 0);

// delta[h,i] = grad_out[h,i,:] . out[h,i,:]
int launch_delta(const Ctx& c, const void* grad_out, const void* out, float* delta);

// Adds the gradient of the max-norm scaling to one row per head of grad_q/grad_k.
// Rows are looked up as (recorded row - row_offset); heads whose row lies outside this shard are skipped.
int launch_norm_fixup(const Ctx& c, const void* q, const void* k, const stat_t* stats,
                      const float* dots, void* grad_q, void* grad_k, int row_offset = 0);

// Where the forward writes: out has row stride `o_stride` elements and is fp32
// when `out_f32` (the reference's packed layout), else the input element type.
struct FwdOut {
  void* out;
  float* den;
  int o_stride;
  int den_stride;
  int out_f32;
};

// gs[h,i,:] = grad_out[h,i,:] / den[h,i]  (bf16) and dvec[h,i] = (grad_out[h,i,:] . out[h,i,:]) / den[h,i]
int launch_gprep(const Ctx& c, const void* grad_out, const void* out, const float* den, void* gs,
                 float* dvec);
// true when every stage of the moment family runs on tensor cores for this problem (then grad_out
// and out are read by the gradient preparation pass only)
bool moments_all_tc(const fastmax_problem& p);

// Tensor-core score-form family (bf16, head dimension 64 or 128, bh a multiple of bhkv).
bool dense_tc_supports(const fastmax_problem& p);
struct ChunkAdd;
int dense_tc_forward(const Ctx& c, const void* q, const void* k, const void* v,
                     const stat_t* stats, void* out, float* den, const ChunkAdd* ca = nullptr);
int dense_tc_backward(const Ctx& c, const void* q, const void* k, const void* v, const void* gs,
                      const float* dvec, const stat_t* stats, float* dots, void* grad_q,
                      void* grad_k, void* grad_v, const ChunkAdd* ca = nullptr);
// Copies the device-side protocol status word to *out (synchronises the stream); *_reset clears it.
// wait_selftest launches one warp that waits, with the given clock limit, on a barrier nobody arrives at.
int tc_wait_selftest(long long limit_clocks, cudaStream_t stream);
int tc_status(int* out, cudaStream_t stream);
int tc_status_reset(cudaStream_t stream);
// Ping-pong kernels for d == 64 (fm_dense_tc_wide.cu): forward, grad_q, and grad_k / grad_v in one kernel.
bool dense_tc_wide_supports(const fastmax_problem& p);
int dense_tc_wide_backward(const Ctx& c, const void* q, const void* k, const void* v, const void* gs,
                           const float* dvec, const stat_t* stats, float* dots, void* grad_q,
                           void* grad_k, void* grad_v, const ChunkAdd* ca = nullptr);
int dense_tc_wide_forward(const Ctx& c, const void* q, const void* k, const void* v, const stat_t* stats,
                          void* out, float* den, const ChunkAdd* ca = nullptr);
int tc_wide_status(int* out, cudaStream_t stream);
int tc_wide_status_reset(cudaStream_t stream);
// backward for d == 128: grad_q, and grad_k / grad_v in one kernel (fm_dense_tc_dkdv128.cu)
bool dense_tc_dkdv128_supports(const fastmax_problem& p);
int dense_tc_backward128(const Ctx& c, const void* q, const void* k, const void* v, const void* gs,
                         const float* dvec, const stat_t* stats, float* dots, void* grad_q, void* grad_k,
                         void* grad_v, const ChunkAdd* ca = nullptr);
int tc_dkdv128_status(int* out, cudaStream_t stream);
int tc_dkdv128_status_reset(cudaStream_t stream);

// Optional coupling of the score-form kernels to the moment-state form: columns are
// restricted to the row's own chunk of `chunk` tokens (0 = no restriction; needs
// nq == nk and chunk % 256 == 0), and fp32 contributions of everything outside the
// chunk are added before the result is divided / rounded.
struct ChunkAdd {
  int chunk = 0;
  const float* out_add = nullptr;   // forward: (bh, nq, d) numerator part
  const float* den_add = nullptr;   // forward: (bh, nq) denominator part
  const float* gq_add = nullptr;    // backward: (bh, nq, d)
  const float* gk_add = nullptr;    // backward: (bhkv, nk, d)
  const float* gv_add = nullptr;    // backward: (bhkv, nk, d)
};

int dense_ffma_forward(const Ctx& c, const void* q, const void* k, const void* v,
                       const stat_t* stats, const FwdOut& o, const ChunkAdd& ca = ChunkAdd());
int dense_ffma_backward(const Ctx& c, const void* q, const void* k, const void* v,
                        const float* den, const stat_t* stats, const void* grad_out,
                        const float* delta, float* dots, void* grad_q, void* grad_k,
                        void* grad_v, const ChunkAdd& ca = ChunkAdd());

// ---- moment-state form (fm_moments_ffma.cu) ---------------------------------------
struct MomentDims {
  int f;    // state rows that are stored: d*d + d + 1, or d + 1 when p == 1
  int f0;   // number of the first stored row (d*d when p == 1, else 0)
  int dvp;  // state columns: d + 1 rounded up to a multiple of 4
};
MomentDims moment_dims(int d, int p = 2);
// state[h][c][f][col] = sum over the tokens of chunk c of feature_f(y) * [z | e];  ext 0: e = 1,
// ext 1: z and e scaled: [z/den | -delta/den].
int moments_chunk_state(const Ctx& c, int heads, int n, int chunk, const void* y, const void* z,
                        const float* den, const float* delta, int ext, float* state,
                        int first_order_only = 0);
// exclusive running sum over chunks (reverse = suffix), started from base; total = own sum; state rows
// before first_row are neither read nor written
int moments_prefix(const Ctx& c, int heads, int nchunk, float* state, const float* base, float* total,
                   int reverse, int write, int first_row = 0);
int moments_readout(const Ctx& c, int mode_b, int heads, int n, int chunk, int state_per_chunk,
                    const void* x, const void* u, const float* den, const float* delta, int ext,
                    const float* state, const stat_t* stats, float* o_add, float* den_add,
                    int first_order_only = 0);

// second-order part on tensor cores (fm_moments_tc.cu): bf16, d == 64, p == 2
bool moments_tc_supports(const fastmax_problem& p);
size_t moments_tc_state_bytes(int mats);
int moments_tc_chunk_state(const Ctx& c, int heads, int n, int chunk, const void* y, const void* z,
                           const float* dvec, float* state);
int moments_tc_convert(const Ctx& c, int mats, const float* state, void* state_bf16);
int moments_tc_prefix_convert(const Ctx& c, int heads, int nchunk, const float* state, const float* base,
                              int reverse, void* state_bf16);
int moments_tc_readout(const Ctx& c, int mode, int heads, int n, int chunk, int state_per_chunk,
                       const void* x, const void* u, const float* uvec, const void* state_bf16,
                       const stat_t* stats, float* out_a, float* den_a, float* out_b,
                       const float* state_f32 = nullptr);
int moments_tc_status(int* out, cudaStream_t stream);
int moments_tc_status_reset(cudaStream_t stream);

// first-order part on tensor cores (fm_first_tc.cu): bf16, d in {64, 128}
bool first_tc_supports(const fastmax_problem& p);
size_t first_tc_copy_bytes(const fastmax_problem& p, int mats);
int first_tc_chunk_state(const Ctx& c, int heads, int n, int chunk, const void* y, const void* z,
                         const float* dvec, float* state);
int first_tc_convert(const Ctx& c, int mats, const float* state, void* s1b);
int first_tc_readout(const Ctx& c, int type_b, int heads, int n, int chunk, int per_chunk, const void* tile,
                     const void* x, const float* uvec, const float* state, const void* s1b,
                     const stat_t* stats, float* o_add, float* den_add, int accumulate, int final = 0,
                     void* out_final = nullptr, float* den_final = nullptr, float* dots = nullptr);
int first_tc_status(int* out, cudaStream_t stream);
int first_tc_status_reset(cudaStream_t stream);
// host orchestration of the moment family (fm_moments.cu)
struct MomFwdWs { size_t states, total, o_add, den_add, s16, bytes; };
struct MomBwdWs { size_t dots, delta, dvec, gs, states, total, gq_add, gk_add, gv_add, s16, bytes; };
int moments_chunk(const fastmax_problem& p);
bool moments_supports(const fastmax_problem& p);
size_t moment_state_bytes(const fastmax_problem& p, int n);
size_t moment_total_bytes(const fastmax_problem& p);
size_t state16_bytes(const fastmax_problem& p, int n);   // bf16 operand copies of the states of n tokens
size_t moment_kept16_bytes(const fastmax_problem& p);    // bf16 second-order copies kept beside the fp32 states
MomFwdWs moments_fwd_layout(const fastmax_problem& p);
MomBwdWs moments_bwd_layout(const fastmax_problem& p);
int moments_forward(const Ctx& c, const void* q, const void* k, const void* v, const stat_t* stats,
                    const FwdOut& o, void* workspace, float* total_keep = nullptr);
int moments_forward_finish(const Ctx& c, const void* q, const void* k, const void* v,
                           const stat_t* stats, float* kv_states, const float* s_base,
                           float* o_add, float* den_add, void* s16, const FwdOut& o,
                           void* second16 = nullptr);
// chunk states of (y, z | e) with the best kernels for the problem; gs/dvec are the bf16
// gradient rows and grad_out.out/den when ext == 1 and the tensor-core path is used
int moments_build_states(const Ctx& c, int n, const void* y, const void* z, const float* den,
                         const float* delta, int ext, const void* gs, const float* dvec, float* states);
int moments_backward(const Ctx& c, const void* q, const void* k, const void* v, const void* out,
                     const float* den, const stat_t* stats, const void* grad_out, void* grad_q,
                     void* grad_k, void* grad_v, void* workspace, const float* kv_total_kept = nullptr);
int moments_backward_finish(const Ctx& c, const void* q, const void* k, const void* v,
                            const float* den, const stat_t* stats, const void* grad_out,
                            const float* delta, const float* dvec, const void* gs,
                            const float* s_states, float* r_states, const float* r_base,
                            float* gq_add, float* gk_add, float* gv_add, void* s16, float* dots,
                            void* grad_q, void* grad_k, void* grad_v, bool dq_far_done = false);
int moments_backward_dq_far(const Ctx& c, const void* q, const float* den, const stat_t* stats,
                            const void* grad_out, const float* delta, const float* dvec, const void* gs,
                            const float* s_states, float* gq_add, void* s16);
// out[i] = sum of gathered[r][i] over r < rank (r > rank when reverse); gathered is (world, floats)
int launch_sum_totals(const float* gathered, int world, int rank, int reverse, size_t floats, float* out,
                      cudaStream_t stream);
// unmasked passes from given total states (this device's, or the sum over all sequence shards)
int moments_forward_total(const Ctx& c, const void* q, const stat_t* stats, const float* total, float* o_add,
                          float* den_add, void* s16, const FwdOut& o);
int moments_backward_total(const Ctx& c, const void* q, const void* k, const void* v, const float* den,
                           const stat_t* stats, const void* grad_out, const float* delta, const float* dvec,
                           const void* gs, const float* kv_total, const float* qg_total, float* gq_add,
                           float* gk_add, float* gv_add, void* s16, float* dots, void* grad_q, void* grad_k,
                           void* grad_v);
int moments_finalize(const Ctx& c, int heads, int n, const float* r, const float* den_in, const void* x,
                     void* out, float* den_out, float* dots, int mode);

}  // namespace fm
