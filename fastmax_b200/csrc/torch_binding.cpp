// torch C++ extension module `fastmax_cuda`: the reference's extension boundary
// (reference fastmax_cuda.cpp:17-37) on top of the fastmax_b200 C ABI.
//
//   forwardpass(q, k, v, drop_noise, [rpe_matrix,] mask, dropout, normalize, temperature,
//               a0, a1, a2, lim, p) -> o
//   backwardpass(q, k, v, o, grad_output, mask, a0, a1, a2, p) -> [gradq, gradk, gradv]
//
// Same contract as the reference: q (bh, nq, d), k and v (bhkv, nk, d), contiguous CUDA
// tensors (float32, or bfloat16 here); o is (bh, nq, d+1) float32 whose last channel is
// the denominator and whose first d channels are the divided output.  Both forwardpass
// arities of the reference's callers are exported (with and without rpe_matrix, which is
// accepted and unused, as in every kernel version of the reference).  Differences, all on
// purpose: inputs are never modified (the reference rescales q and k in place when
// normalize is set and divides grad_output in place), work is issued on the current
// stream of the tensors' device without device-wide synchronisation, and p = 2 is
// computed (the reference's current kernels silently ignore it).
//
// normalize.  backwardpass has no normalize, lim or temperature argument in the
// reference: there forwardpass leaves the rescaled q and k behind in the caller's
// tensors, the wrapper saves those and backwardpass differentiates the attention of
// what it is handed (reference example.py:36-47, 69; model.py:29-75).  Here q and k stay
// as the caller wrote them, so forwardpass has to tell backwardpass what it did: the
// tensor it returns owns a few hundred extra bytes behind its (b*h, n, d+1) elements that
// hold the per-head max-norm statistics, and a host-side table keyed by that storage's
// address remembers (normalize, lim, shape).  backwardpass looks `o` up; if it finds the
// record and the storage still has the recorded size, it runs the normalised backward --
// gradients with respect to the caller's own q and k, including the derivative of the
// max-norm scaling, which is what autograd through the reference's PyTorch path returns.
// An `o` that forwardpass did not make (or a copy of it) falls back to the unnormalised
// backward of the q and k given.  The record lives as long as the address is not reused by
// a later forwardpass result; the table keeps the most recent 65536 results.
//
// dropout.  forwardpass multiplies channels 0..d-1 of o by 1 + dropout * drop_noise, as the
// reference does (fastmax_cuda_forward.cu:271-280, 396-399); backwardpass, like the
// reference's, then works from the o it is given.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <cstdint>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "fastmax_b200.h"

namespace {

void check_input(const torch::Tensor& x, const char* name) {
  TORCH_CHECK(x.device().is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(x.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(x.dim() == 3, name, " must be (b*h, n, d)");
  TORCH_CHECK(x.scalar_type() == torch::kFloat32 || x.scalar_type() == torch::kBFloat16, name,
              " must be float32 or bfloat16");
}

fastmax_problem make_problem(const torch::Tensor& q, const torch::Tensor& k, bool mask, bool normalize,
                             double temperature, double a0, double a1, double a2, double lim, int64_t p) {
  TORCH_CHECK(p == 1 || p == 2, "p must be 1 or 2, got: ", p);
  fastmax_problem pr;
  pr.dtype = q.scalar_type() == torch::kFloat32 ? FASTMAX_F32 : FASTMAX_BF16;
  pr.bh = (int32_t)q.size(0);
  pr.bhkv = (int32_t)k.size(0);
  pr.nq = (int32_t)q.size(1);
  pr.nk = (int32_t)k.size(1);
  pr.d = (int32_t)q.size(2);
  pr.mask = mask;
  pr.normalize = normalize;
  pr.p = (int32_t)p;
  pr.impl = FASTMAX_IMPL_AUTO;
  pr.a0 = (float)a0;
  pr.a1 = (float)a1;
  pr.a2 = (float)a2;
  pr.lim = (float)lim;
  pr.temperature = (float)temperature;
  pr.chunk = 0;
  return pr;
}

void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == FASTMAX_OK, what, " failed (code ", rc, "): ", fastmax_b200_last_error());
}

// What forwardpass did, for the backwardpass that will be handed its result.
struct FwdRecord {
  int64_t bh, bhkv, nq, nk, d;
  size_t storage_bytes;   // of the tensor forwardpass returned (elements + statistics)
  size_t stats_offset;    // byte offset of the statistics inside that storage
  bool normalize;
  float lim;
  uint64_t seq;
};
std::mutex g_rec_mu;
std::unordered_map<const void*, FwdRecord> g_rec;
uint64_t g_rec_seq = 0;
constexpr size_t kMaxRecords = 65536;

void remember(const void* key, FwdRecord r) {
  std::lock_guard<std::mutex> lk(g_rec_mu);
  r.seq = ++g_rec_seq;
  g_rec[key] = r;
  if (g_rec.size() > kMaxRecords) {   // drop the older half
    const uint64_t cut = g_rec_seq - kMaxRecords / 2;
    for (auto it = g_rec.begin(); it != g_rec.end();) it = it->second.seq <= cut ? g_rec.erase(it) : ++it;
  }
}
bool recall(const void* key, FwdRecord* r) {
  std::lock_guard<std::mutex> lk(g_rec_mu);
  auto it = g_rec.find(key);
  if (it == g_rec.end()) return false;
  *r = it->second;
  return true;
}

torch::Tensor forward_impl(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v,
                           const c10::optional<torch::Tensor>& drop_noise, bool mask, double dropout, bool normalize,
                           double temperature, double a0, double a1, double a2, double lim, int64_t p) {
  check_input(q, "q");
  check_input(k, "k");
  check_input(v, "v");
  TORCH_CHECK(k.sizes() == v.sizes() && q.size(2) == k.size(2) && q.scalar_type() == k.scalar_type() &&
                  q.scalar_type() == v.scalar_type() && q.device() == k.device() && q.device() == v.device(),
              "q, k and v disagree in shape, dtype or device");
  TORCH_CHECK(dropout >= 0.0, "dropout must be non-negative, got: ", dropout);
  c10::cuda::CUDAGuard guard(q.device());
  fastmax_problem pr = make_problem(q, k, mask, normalize, temperature, a0, a1, a2, lim, p);
  // one storage: the (bh, nq, d+1) result, then (256-byte aligned) the statistics of this call
  const int64_t elems = q.size(0) * q.size(1) * (q.size(2) + 1);
  const size_t stats_offset = ((size_t)elems * sizeof(float) + 255) / 256 * 256;
  const size_t stats_bytes = std::max<size_t>(fastmax_b200_stats_bytes(&pr), 8);
  const int64_t total_floats = (int64_t)((stats_offset + stats_bytes + 3) / 4);
  auto buf = torch::empty({total_floats}, q.options().dtype(torch::kFloat32));
  auto o = buf.narrow(0, 0, elems).view({q.size(0), q.size(1), q.size(2) + 1});
  void* stats = (char*)buf.data_ptr() + stats_offset;
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  check_rc(fastmax_b200_forward_packed(&pr, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr<float>(), stats,
                                       nullptr, 0, stream),
           "fastmax forwardpass");
  if (dropout > 0.0) {
    TORCH_CHECK(drop_noise.has_value() && drop_noise->defined(), "dropout > 0 needs drop_noise");
    const torch::Tensor& nz = *drop_noise;
    TORCH_CHECK(nz.device() == q.device() && nz.is_contiguous() && nz.numel() == q.numel() &&
                    (nz.scalar_type() == torch::kFloat32 || nz.scalar_type() == torch::kBFloat16),
                "drop_noise must be a contiguous float32 or bfloat16 CUDA tensor with as many elements as q");
    check_rc(fastmax_b200_scale_packed_by_noise(o.data_ptr<float>(), nz.data_ptr(), (float)dropout,
                                                q.size(0) * q.size(1), (int)q.size(2),
                                                nz.scalar_type() == torch::kFloat32 ? FASTMAX_F32 : FASTMAX_BF16,
                                                stream),
             "fastmax forwardpass (dropout)");
  }
  remember(buf.storage().data(), FwdRecord{q.size(0), k.size(0), q.size(1), k.size(1), q.size(2),
                                           buf.storage().nbytes(), stats_offset, normalize, (float)lim, 0});
  return o;
}

torch::Tensor forwardpass13(torch::Tensor q, torch::Tensor k, torch::Tensor v, c10::optional<torch::Tensor> drop_noise,
                            bool mask, double dropout, bool normalize, double temperature, double a0, double a1,
                            double a2, double lim, int64_t p) {
  return forward_impl(q, k, v, drop_noise, mask, dropout, normalize, temperature, a0, a1, a2, lim, p);
}

torch::Tensor forwardpass14(torch::Tensor q, torch::Tensor k, torch::Tensor v, c10::optional<torch::Tensor> drop_noise,
                            c10::optional<torch::Tensor> rpe_matrix, bool mask, double dropout, bool normalize,
                            double temperature, double a0, double a1, double a2, double lim, int64_t p) {
  (void)rpe_matrix;
  return forward_impl(q, k, v, drop_noise, mask, dropout, normalize, temperature, a0, a1, a2, lim, p);
}

std::vector<torch::Tensor> backwardpass(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor o,
                                        torch::Tensor grad_output, bool mask, double a0, double a1, double a2,
                                        int64_t p) {
  check_input(q, "q");
  check_input(k, "k");
  check_input(v, "v");
  TORCH_CHECK(o.device() == q.device() && o.dim() == 3 && o.size(0) == q.size(0) && o.size(1) == q.size(1) &&
                  o.size(2) == q.size(2) + 1 && o.scalar_type() == torch::kFloat32,
              "o must be the (b*h, n, d+1) float32 tensor forwardpass returned");
  TORCH_CHECK(grad_output.device() == q.device() && grad_output.sizes() == q.sizes(),
              "grad_output must have the shape of q");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t d = q.size(2);
  // did forwardpass make this o, and with which normalisation?
  FwdRecord rec;
  const void* stats = nullptr;
  bool normalize = false;
  float lim = 1.0f;
  if (o.storage_offset() == 0 && o.is_contiguous() && recall(o.storage().data(), &rec) &&
      rec.storage_bytes == o.storage().nbytes() && rec.bh == q.size(0) && rec.bhkv == k.size(0) &&
      rec.nq == q.size(1) && rec.nk == k.size(1) && rec.d == d && rec.normalize) {
    normalize = true;
    lim = rec.lim;
    stats = (const char*)o.storage().data() + rec.stats_offset;
  }
  fastmax_problem pr = make_problem(q, k, mask, normalize, 1.0, a0, a1, a2, lim, p);
  auto out = o.slice(2, 0, d).to(q.scalar_type()).contiguous();
  auto den = o.select(2, d).contiguous();
  auto go = grad_output.to(q.scalar_type()).contiguous();
  auto gq = torch::empty_like(q), gk = torch::empty_like(k), gv = torch::empty_like(v);
  const size_t wsb = fastmax_b200_backward_workspace_bytes(&pr);
  auto ws = torch::empty({(int64_t)std::max<size_t>(wsb, 1)}, q.options().dtype(torch::kUInt8));
  check_rc(fastmax_b200_backward(&pr, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                 den.data_ptr<float>(), stats, go.data_ptr(), gq.data_ptr(), gk.data_ptr(),
                                 gv.data_ptr(), ws.data_ptr(), wsb, at::cuda::getCurrentCUDAStream().stream()),
           "fastmax backwardpass");
  return {gq, gk, gv};
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("forwardpass", &forwardpass13, "forwardpass");
  m.def("forwardpass", &forwardpass14, "forwardpass (with rpe_matrix)");
  m.def("backwardpass", &backwardpass, "backwardpass");
}
