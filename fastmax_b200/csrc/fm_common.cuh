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
};

// Row statistics of q and k into `stats` (zeroes it first).
int launch_rowmax(const Ctx& c, const void* q, const void* k, stat_t* stats);

// delta[h,i] = grad_out[h,i,:] . out[h,i,:]
int launch_delta(const Ctx& c, const void* grad_out, const void* out, float* delta);

// Adds the gradient of the max-norm scaling to one row per head of grad_q/grad_k.
int launch_norm_fixup(const Ctx& c, const void* q, const void* k, const stat_t* stats,
                      const float* dots, void* grad_q, void* grad_k);

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

// Tensor-core score-form family (bf16, head dimension 64, bh == bhkv).
bool dense_tc_supports(const fastmax_problem& p);
int dense_tc_forward(const Ctx& c, const void* q, const void* k, const void* v,
                     const stat_t* stats, void* out, float* den);
int dense_tc_backward(const Ctx& c, const void* q, const void* k, const void* v, const void* gs,
                      const float* dvec, const stat_t* stats, float* dots, void* grad_q,
                      void* grad_k, void* grad_v);
// Copies the device-side protocol status word to *out (synchronises the stream).
int tc_status(int* out, cudaStream_t stream);

int dense_ffma_forward(const Ctx& c, const void* q, const void* k, const void* v,
                       const stat_t* stats, const FwdOut& o);
int dense_ffma_backward(const Ctx& c, const void* q, const void* k, const void* v,
                        const float* den, const stat_t* stats, const void* grad_out,
                        const float* delta, float* dots, void* grad_q, void* grad_k,
                        void* grad_v);

}  // namespace fm
