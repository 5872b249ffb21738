// Backward pass that needs no scratch buffer from the caller and never asks CUDA
// for memory: its scratch is a fixed array that is part of the library image.
//
// Who this is for.  Some programs that embed this library cannot hand it a
// workspace or let it obtain one: an inference server or training framework that
// has already claimed all device memory for its own arena (so a cudaMalloc made
// on its behalf fails, or succeeds only by evicting cached blocks), and
// latency-critical loops for which the device-wide synchronisation that
// cudaMalloc and cudaFree imply is not acceptable.  For them the scratch lives
// in a file-scope __device__ array that the driver reserves on a GPU when this
// library's code is loaded there, and that stays reserved until the process exits.
// With CUDA's default lazy module loading that happens at the first call on that
// GPU, which also looks the array's address up (with that GPU current).  A host
// that is about to hand the rest of the GPU to its own arena, or to start a stream
// capture, should therefore make one call first; an empty problem (bh == 0, all
// pointers NULL) does the set-up and nothing else.  Setting
// CUDA_MODULE_LOADING=EAGER moves the reservation to library load.
//
// Limits.  The array is kStaticScratchBytes (8 MiB) per GPU; a problem whose
// scratch does not fit is rejected with FASTMAX_E_WORKSPACE.  Every call on a
// GPU uses the same array, so two calls that overlap on that GPU (different
// streams, different host threads) race; issue them on one stream or order them
// yourself.  The array keeps whatever the previous call left there; the part
// that must start at zero is cleared at the start of each call.
#include <mutex>

#include "fm_common.cuh"

namespace fm {
namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;
// In host code this name is only a handle for the runtime's symbol calls; the
// device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the array on the current device; looked up once per device.
int static_scratch(void** out) {
  int dev = -1;
  FM_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(FASTMAX_E_DEVICE, "device ordinal %d is out of range", dev);
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p)
      return fail(FASTMAX_E_CUDA, "cudaGetSymbolAddress(static scratch) failed on device %d: %s", dev,
                  cudaGetErrorString(e));
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return FASTMAX_OK;
}

size_t align256(size_t x) { return (x + 255) / 256 * 256; }

}  // namespace
}  // namespace fm

using namespace fm;

extern "C" {

size_t fastmax_b200_static_scratch_bytes(void) { return kStaticScratchBytes; }

int fastmax_b200_backward_static(const fastmax_problem* prob, const void* q, const void* k,
                                 const void* v, const void* out, const float* den,
                                 const void* stats, const void* grad_out, void* grad_q,
                                 void* grad_k, void* grad_v, void* stream) {
  int rc = check_problem(prob);
  if (rc) return rc;
  const fastmax_problem& p = *prob;
  // The device check and the per-device address lookup come before everything else, so that
  // a call with an empty problem (bh == 0) is a cheap way to do the one-time set-up early:
  // under CUDA's lazy module loading it is this lookup that makes the driver reserve the
  // array on the current GPU.
  int major = 0, dev = 0;
  FM_CUDA_TRY(cudaGetDevice(&dev));
  FM_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return fail(FASTMAX_E_DEVICE, "device %d is not compute capability 10.x", dev);
  void* base = nullptr;
  if ((rc = static_scratch(&base))) return rc;
  if (p.bh == 0 || (p.nq == 0 && p.nk == 0)) return FASTMAX_OK;
  if (!q || !k || !v || !out || !den || !grad_out || !grad_q || !grad_k || !grad_v)
    return fail(FASTMAX_E_ARG, "NULL tensor pointer");
  if (p.normalize && !stats) return fail(FASTMAX_E_ARG, "normalize needs the forward's stats buffer");
  if (p.impl != FASTMAX_IMPL_AUTO && p.impl != FASTMAX_IMPL_DENSE_FFMA)
    return fail(FASTMAX_E_UNSUPPORTED, "the static-scratch backward runs the CUDA-core score family only");
  // scratch layout: [per-head dot accumulators: bh + bhkv floats][row dots: bh * nq floats]
  const size_t dots_bytes = align256(sizeof(float) * (size_t)(p.bh + p.bhkv));
  const size_t need = dots_bytes + align256(sizeof(float) * (size_t)p.bh * p.nq);
  if (need > kStaticScratchBytes)
    return fail(FASTMAX_E_WORKSPACE,
                "this problem needs %zu bytes of scratch but the built-in array holds %zu "
                "(bh*nq must stay below about %zu); use fastmax_b200_backward with a caller buffer",
                need, kStaticScratchBytes, (kStaticScratchBytes - dots_bytes) / sizeof(float));
  Ctx c{p, (cudaStream_t)stream};
  float* dots = (float*)base;
  float* delta = (float*)((char*)base + dots_bytes);
  // the accumulators are added to with atomics and must start at zero; the row dots are fully rewritten
  if (p.normalize) FM_CUDA_TRY(cudaMemsetAsync(dots, 0, sizeof(float) * (size_t)(p.bh + p.bhkv), c.stream));
  if ((rc = launch_delta(c, grad_out, out, delta))) return rc;
  if ((rc = dense_ffma_backward(c, q, k, v, den, (const stat_t*)stats, grad_out, delta, dots, grad_q,
                                grad_k, grad_v)))
    return rc;
  if (p.normalize) return launch_norm_fixup(c, q, k, (const stat_t*)stats, dots, grad_q, grad_k);
  return FASTMAX_OK;
}

}  // extern "C"
