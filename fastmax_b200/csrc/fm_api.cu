// C ABI of the fastmax_b200 library: argument validation, workspace layout and
// dispatch to the kernel families.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <atomic>
#include <initializer_list>
#include <mutex>
#include <string>
#include <vector>

#include "fm_common.cuh"

namespace fm {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// ---- launch accounting ------------------------------------------------------
struct ProfRec {
  const char* name;
  cudaEvent_t e0, e1;
};
static std::atomic<unsigned long long> g_launches{0};
static std::atomic<int> g_prof_on{0};
static std::mutex g_prof_mu;
static std::vector<ProfRec> g_prof;
static thread_local int g_prof_open = -1;
static const size_t kProfMax = 1u << 16;

void prof_before(const char* name, cudaStream_t s) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  g_prof_open = -1;
  if (!g_prof_on.load(std::memory_order_relaxed)) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (g_prof.size() >= kProfMax) return;
  ProfRec r{name, nullptr, nullptr};
  if (cudaEventCreate(&r.e0) != cudaSuccess || cudaEventCreate(&r.e1) != cudaSuccess) return;
  cudaEventRecord(r.e0, s);
  g_prof.push_back(r);
  g_prof_open = (int)g_prof.size() - 1;
}

void prof_after(cudaStream_t s) {
  if (g_prof_open < 0) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if ((size_t)g_prof_open < g_prof.size()) cudaEventRecord(g_prof[g_prof_open].e1, s);
  g_prof_open = -1;
}

static void prof_clear() {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  for (auto& r : g_prof) {
    if (r.e0) cudaEventDestroy(r.e0);
    if (r.e1) cudaEventDestroy(r.e1);
  }
  g_prof.clear();
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static int validate(const fastmax_problem* p) {
  if (!p) return fail(FASTMAX_E_ARG, "problem is NULL");
  if (p->dtype != FASTMAX_F32 && p->dtype != FASTMAX_BF16)
    return fail(FASTMAX_E_ARG, "dtype %d is neither FASTMAX_F32 nor FASTMAX_BF16", p->dtype);
  if (p->p != 1 && p->p != 2) return fail(FASTMAX_E_ARG, "p must be 1 or 2, got: %d", p->p);
  if (p->d != 8 && p->d != 16 && p->d != 32 && p->d != 64 && p->d != 128)
    return fail(FASTMAX_E_ARG, "head dimension %d is not one of 8,16,32,64,128", p->d);
  if (p->bh < 0 || p->bhkv < 0 || p->nq < 0 || p->nk < 0)
    return fail(FASTMAX_E_ARG, "negative size");
  if (p->bh > 0 && (p->bhkv <= 0 || p->bh % p->bhkv != 0))
    return fail(FASTMAX_E_ARG, "bh=%d is not a multiple of bhkv=%d", p->bh, p->bhkv);
  if (p->nq > (1 << 22) || p->nk > (1 << 22))
    return fail(FASTMAX_E_ARG, "sequence longer than 4194304 tokens");
  if (p->mask && p->nk < p->nq)
    return fail(FASTMAX_E_ARG, "causal attention needs nk >= nq (nq=%d, nk=%d)", p->nq, p->nk);
  if (p->nq > 0 && p->nk == 0) return fail(FASTMAX_E_ARG, "no keys (nk == 0)");
  if (p->impl < FASTMAX_IMPL_AUTO || p->impl > FASTMAX_IMPL_MOMENTS_FFMA)
    return fail(FASTMAX_E_ARG, "unknown impl %d", p->impl);
  if (p->chunk < 0 || p->chunk % 256 != 0)
    return fail(FASTMAX_E_ARG, "chunk=%d is not a non-negative multiple of 256", p->chunk);
  return FASTMAX_OK;
}

// Argument check shared with other translation units of the library.
int check_problem(const fastmax_problem* p) { return validate(p); }

static int check_device() {
  int dev = 0;
  FM_CUDA_TRY(cudaGetDevice(&dev));
  int major = 0;
  FM_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10)
    return fail(FASTMAX_E_DEVICE, "device %d has compute capability %d.x; this library is built for sm_100a only",
                dev, major);
  return FASTMAX_OK;
}

// Family actually used for a problem.  `packed` = forward into the reference's
// float32 (d+1)-channel layout, which only the CUDA-core family writes.
// Rough time of one pass per (token, head) in arbitrary units: score form grows with the
// number of keys a row sees, the moment form is constant plus its own chunk in score form.
static bool moments_faster(const fastmax_problem& p, bool tc_ok) {
  if (!moments_supports(p)) return false;
  const double d = p.d, F = d + (p.p == 2 ? d * d : 0.0);
  // Constants fitted to this library's kernels on a B200 (bf16, d = 64, p = 2, causal): the score family takes
  // 5.6 ns per token and head at 10^4 keys; the moment family 4.1 ns for its states and read-outs plus 2.0 ns
  // for the score kernels of a 2048-token chunk (short rows run at 0.58 of the long-row rate), the former
  // times the share of chunks that build and read states.  The two families then break even near 9 300 keys,
  // as measured (score against moment family for the same number of token-heads, 8192 keys: 20.3 / 22.8 ms;
  // 9216: 22.6 / 23.0; 10000: 60.9 / 54.5).
  const double rate_score = tc_ok ? 800e12 : 25e12;
  const double rate_state = p.p == 2 ? (moments_tc_supports(p) ? 930e12 : 20e12) : (first_tc_supports(p) ? 450e12 : 20e12);
  const double rate_chunk = tc_ok ? 0.58 * rate_score : rate_score;
  // Unmasked with nq != nk: the score form costs nq * nk pairs, the moment form one state per key and one
  // read-out per query row (and the mirror image backward), so per token of the mean length the score form
  // sees nq * nk / mean(nq, nk) keys.  Few query rows against many keys therefore stay on the score family.
  const double keys = p.mask ? 0.5 * p.nk : (double)p.nq * p.nk / (0.5 * ((double)p.nq + p.nk));
  const double chunk_keys = p.mask ? 0.5 * moments_chunk(p) : 0.0;
  const double per_key = 14.0 * (d + 0.5);
  const double t_score = keys * per_key / rate_score;
  // causal: one chunk in nchunk builds no state and one reads none (see Ctx::skip_chunk, zero_chunk)
  const int L = moments_chunk(p);
  const double used = p.mask ? 1.0 - 1.0 / (double)((p.nk + L - 1) / L) : 1.0;
  double t_mom = used * 14.0 * F * (d + 1) / rate_state + chunk_keys * per_key / rate_chunk;
  // unmasked: the fp32 result rows take one more pass (5.5 ns per token and head in all), and each head
  // pays about a third of a chunk's time once, for its totals (break-even measured near 5 500 keys)
  if (!p.mask) t_mom *= 1.3 * (1.0 + 0.33 * L / (0.5 * ((double)p.nq + p.nk)));
  return t_mom < t_score && p.nk > moments_chunk(p);
}

static int pick_impl(const fastmax_problem& p, bool packed, int* impl) {
  int want = p.impl;
  const bool tc_ok = dense_tc_supports(p) && !packed;
  if (want == FASTMAX_IMPL_AUTO) {
    want = tc_ok ? FASTMAX_IMPL_DENSE_TC : FASTMAX_IMPL_DENSE_FFMA;
    if (!packed && moments_faster(p, tc_ok)) want = FASTMAX_IMPL_MOMENTS;
  }
  if (want == FASTMAX_IMPL_MOMENTS || want == FASTMAX_IMPL_MOMENTS_FFMA) {
    if (!moments_supports(p) || packed)
      return fail(FASTMAX_E_UNSUPPORTED,
                  "the moment family needs bh == bhkv, nq == nk when causal, and the plain output layout");
    *impl = FASTMAX_IMPL_MOMENTS;   // callers branch on the family; the state kernels look at p.impl
    return FASTMAX_OK;
  }
  if (want == FASTMAX_IMPL_DENSE_TC && !tc_ok)
    return fail(FASTMAX_E_UNSUPPORTED,
                "the tensor-core score family needs bf16, d in {64, 128} and the plain output layout");
  if (want != FASTMAX_IMPL_DENSE_FFMA && want != FASTMAX_IMPL_DENSE_TC)
    return fail(FASTMAX_E_UNSUPPORTED, "kernel family %d is not available in this build", want);
  *impl = want;
  return FASTMAX_OK;
}

// The tensor-core kernels read through TMA, which needs 16-byte aligned base addresses; when the
// library chose that family itself (AUTO) and a tensor is not aligned, the CUDA-core family
// serves the call instead of failing it.
static bool aligned16(std::initializer_list<const void*> ptrs) {
  for (const void* q : ptrs)
    if (((uintptr_t)q & 15) != 0) return false;
  return true;
}

// Backward workspace: [dots: bh+bhkv floats][delta or dvec: bh*nq floats]
// [gs: bh*nq*d bf16, tensor-core family only], 256-byte aligned parts.
struct BwdWs {
  size_t dots_off, delta_off, gs_off, total;
};
static BwdWs bwd_layout(const fastmax_problem& p) {
  BwdWs w;
  w.dots_off = 0;
  w.delta_off = align_up(sizeof(float) * (size_t)(p.bh + p.bhkv), 256);
  w.gs_off = w.delta_off + align_up(sizeof(float) * (size_t)p.bh * p.nq, 256);
  w.total = w.gs_off;
  if (dense_tc_supports(p)) w.total += align_up((size_t)2 * p.bh * p.nq * p.d, 256);
  return w;
}
// the workspace must serve whichever family AUTO picks
static size_t fwd_ws_bytes(const fastmax_problem& p) {
  return moments_supports(p) ? moments_fwd_layout(p).bytes : 0;
}
static size_t bwd_ws_bytes(const fastmax_problem& p) {
  size_t a = bwd_layout(p).total;
  if (moments_supports(p)) { size_t b = moments_bwd_layout(p).bytes; if (b > a) a = b; }
  return a;
}

}  // namespace fm

using namespace fm;

extern "C" {

int fastmax_b200_version(void) { return 200; }

const char* fastmax_b200_last_error(void) { return g_err; }

unsigned long long fastmax_b200_launch_count(void) { return g_launches.load(); }

int fastmax_b200_device_status(int* status, void* stream) {
  if (!status) return fail(FASTMAX_E_ARG, "status is NULL");
  int a = 0, b = 0, f = 0, w = 0, rc;
  if ((rc = tc_status(&a, (cudaStream_t)stream))) return rc;
  if ((rc = tc_wide_status(&w, (cudaStream_t)stream))) return rc;
  if (!a) a = w;
  if ((rc = tc_dkdv128_status(&w, (cudaStream_t)stream))) return rc;
  if (!a) a = w;
  if ((rc = moments_tc_status(&b, (cudaStream_t)stream))) return rc;
  if ((rc = first_tc_status(&f, (cudaStream_t)stream))) return rc;
  *status = a ? a : (b ? b : f);
  return FASTMAX_OK;
}

int fastmax_b200_device_status_reset(void* stream) {
  int rc;
  cudaStream_t s = (cudaStream_t)stream;
  if ((rc = tc_status_reset(s))) return rc;
  if ((rc = tc_wide_status_reset(s))) return rc;
  if ((rc = tc_dkdv128_status_reset(s))) return rc;
  if ((rc = moments_tc_status_reset(s))) return rc;
  return first_tc_status_reset(s);
}

int fastmax_b200_wait_selftest(long long limit_clocks, void* stream) {
  int rc = check_device();
  if (rc) return rc;
  return tc_wait_selftest(limit_clocks, (cudaStream_t)stream);
}

int fastmax_b200_profile_enable(int on) {
  g_prof_on.store(0);
  prof_clear();
  g_prof_on.store(on ? 1 : 0);
  return FASTMAX_OK;
}

int fastmax_b200_profile_count(void) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  return (int)g_prof.size();
}

int fastmax_b200_profile_get(int i, char* name, int name_len, float* ms) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (i < 0 || (size_t)i >= g_prof.size()) return fail(FASTMAX_E_ARG, "profile record %d out of range", i);
  const ProfRec& r = g_prof[i];
  if (name && name_len > 0) {
    strncpy(name, r.name, (size_t)name_len - 1);
    name[name_len - 1] = 0;
  }
  if (ms) {
    FM_CUDA_TRY(cudaEventSynchronize(r.e1));
    FM_CUDA_TRY(cudaEventElapsedTime(ms, r.e0, r.e1));
  }
  return FASTMAX_OK;
}

// Problems on the moment family leave behind the statistic words what the backward pass would otherwise
// rebuild from k and v: unmasked, the total key/value state; causal, the exclusive prefixes of the key/value
// chunk states -- the latter only while they are no larger than twice the tensors autograd holds anyway
// (q, k, v, out), which is the case for the tensor-core configurations (1.1 MB of state per 2048-token chunk
// and head at d = 64 against 1 MB of tokens).
static size_t stats_words_bytes(const fastmax_problem& p) {
  return align_up(sizeof(stat_t) * (size_t)(p.bh + p.bhkv), 256);
}
static size_t kept_bytes(const fastmax_problem& p) {
  if (!p.mask) return moment_total_bytes(p);
  const size_t states = moment_state_bytes(p, p.nk) + moment_kept16_bytes(p);
  const size_t es = p.dtype == FASTMAX_BF16 ? 2 : 4;
  const size_t held = es * (size_t)p.d * (2 * (size_t)p.bh * p.nq + 2 * (size_t)p.bhkv * p.nk);
  return states <= 2 * held ? states : 0;
}
static bool keeps_total(const fastmax_problem& p, int impl) {
  return impl == FASTMAX_IMPL_MOMENTS && kept_bytes(p) > 0;
}

size_t fastmax_b200_stats_bytes(const fastmax_problem* p) {
  if (!p || p->bh < 0 || p->bhkv < 0) return 0;
  int impl;
  if (validate(p) == FASTMAX_OK && p->bh > 0 && pick_impl(*p, false, &impl) == FASTMAX_OK && keeps_total(*p, impl))
    return stats_words_bytes(*p) + kept_bytes(*p);
  return sizeof(stat_t) * (size_t)(p->bh + p->bhkv);
}

int fastmax_b200_selected_impl(const fastmax_problem* p, int32_t* impl) {
  if (!impl) return fail(FASTMAX_E_ARG, "null impl pointer");
  int rc = validate(p);
  if (rc) return rc;
  int got = 0;
  if ((rc = pick_impl(*p, false, &got))) return rc;
  *impl = got;
  return FASTMAX_OK;
}

// Sized for the family the call will run: the moment family needs room for its states.
size_t fastmax_b200_forward_workspace_bytes(const fastmax_problem* p) {
  if (validate(p)) return 0;
  int impl;
  if (pick_impl(*p, false, &impl)) return 0;
  return impl == FASTMAX_IMPL_MOMENTS ? fwd_ws_bytes(*p) : 0;
}

size_t fastmax_b200_backward_workspace_bytes(const fastmax_problem* p) {
  if (validate(p)) return 0;
  int impl;
  if (pick_impl(*p, false, &impl)) return 0;
  return impl == FASTMAX_IMPL_MOMENTS ? bwd_ws_bytes(*p) : bwd_layout(*p).total;
}

// Whether a problem can take its result and upstream gradient in the (batch, n, heads, d) layout:
// the last kernel of the forward must be a tensor-core score kernel and grad_out / out must be read
// by the gradient preparation pass alone.
static int bt_layout_ok(const fastmax_problem& p, int heads_per_batch, int impl) {
  if (heads_per_batch <= 0 || p.bh % heads_per_batch != 0)
    return fail(FASTMAX_E_ARG, "heads_per_batch=%d does not divide bh=%d", heads_per_batch, p.bh);
  const bool ok = dense_tc_supports(p) &&
                  (impl == FASTMAX_IMPL_DENSE_TC || (impl == FASTMAX_IMPL_MOMENTS && p.mask && moments_all_tc(p)));
  if (!ok)
    return fail(FASTMAX_E_UNSUPPORTED,
                "the (batch, n, heads, d) layout needs the tensor-core kernels (bf16, d in {64, 128}; the moment "
                "family only when causal); use the plain layout and swap the axes");
  return FASTMAX_OK;
}

static int forward_impl(const fastmax_problem* prob, const void* q, const void* k, const void* v,
                        const FwdOut& o, void* stats, void* workspace, size_t workspace_bytes,
                        void* stream, int heads_per_batch = 0) {
  int rc = validate(prob);
  if (rc) return rc;
  const fastmax_problem& p = *prob;
  if (p.bh == 0 || p.nq == 0) return FASTMAX_OK;
  if (!q || !k || !v || !o.out || !o.den) return fail(FASTMAX_E_ARG, "NULL tensor pointer");
  if (p.normalize && !stats) return fail(FASTMAX_E_ARG, "normalize needs a stats buffer");
  if ((rc = check_device())) return rc;
  int impl;
  if ((rc = pick_impl(p, o.out_f32 != 0, &impl))) return rc;
  if (p.impl == FASTMAX_IMPL_AUTO && impl == FASTMAX_IMPL_DENSE_TC && !aligned16({q, k, v, o.out}))
    impl = FASTMAX_IMPL_DENSE_FFMA;
  if (heads_per_batch && (rc = bt_layout_ok(p, heads_per_batch, impl))) return rc;
  Ctx c{p, (cudaStream_t)stream};
  c.out_heads = heads_per_batch;
  if (p.normalize && (rc = launch_rowmax(c, q, k, (stat_t*)stats))) return rc;
  if (impl == FASTMAX_IMPL_MOMENTS) {
    const size_t need = moments_fwd_layout(p).bytes;
    if (!workspace || workspace_bytes < need)
      return fail(FASTMAX_E_WORKSPACE, "forward workspace too small: need %zu bytes, got %zu", need,
                  workspace_bytes);
    float* keep = (stats && keeps_total(p, impl)) ? (float*)((char*)stats + stats_words_bytes(p)) : nullptr;
    return moments_forward(c, q, k, v, (const stat_t*)stats, o, workspace, keep);
  }
  if (impl == FASTMAX_IMPL_DENSE_TC)
    return dense_tc_forward(c, q, k, v, (const stat_t*)stats, o.out, o.den);
  return dense_ffma_forward(c, q, k, v, (const stat_t*)stats, o);
}

int fastmax_b200_forward(const fastmax_problem* prob, const void* q, const void* k, const void* v,
                         void* out, float* den, void* stats, void* workspace,
                         size_t workspace_bytes, void* stream) {
  FwdOut o{out, den, prob ? prob->d : 0, 1, 0};
  return forward_impl(prob, q, k, v, o, stats, workspace, workspace_bytes, stream);
}

int fastmax_b200_forward_bt(const fastmax_problem* prob, const void* q, const void* k, const void* v,
                            void* out_bt, float* den, void* stats, int32_t heads_per_batch, void* workspace,
                            size_t workspace_bytes, void* stream) {
  if (heads_per_batch <= 0) return fail(FASTMAX_E_ARG, "heads_per_batch must be positive");
  FwdOut o{out_bt, den, prob ? prob->d : 0, 1, 0};
  return forward_impl(prob, q, k, v, o, stats, workspace, workspace_bytes, stream, heads_per_batch);
}

int fastmax_b200_bt_layout_supported(const fastmax_problem* prob, int32_t heads_per_batch) {
  if (validate(prob)) return 0;
  int impl;
  if (pick_impl(*prob, false, &impl)) return 0;
  return bt_layout_ok(*prob, heads_per_batch, impl) == FASTMAX_OK;
}

int fastmax_b200_forward_packed(const fastmax_problem* prob, const void* q, const void* k,
                                const void* v, float* o_packed, void* stats, void* workspace,
                                size_t workspace_bytes, void* stream) {
  int d = prob ? prob->d : 0;
  FwdOut o{o_packed, o_packed ? o_packed + d : nullptr, d + 1, d + 1, 1};
  return forward_impl(prob, q, k, v, o, stats, workspace, workspace_bytes, stream);
}

static int backward_impl(const fastmax_problem* prob, const void* q, const void* k, const void* v,
                         const void* out, const float* den, const void* stats,
                         const void* grad_out, void* grad_q, void* grad_k, void* grad_v,
                         void* workspace, size_t workspace_bytes, void* stream, int heads_per_batch) {
  int rc = validate(prob);
  if (rc) return rc;
  const fastmax_problem& p = *prob;
  if (p.bh == 0 || (p.nq == 0 && p.nk == 0)) return FASTMAX_OK;
  if (!q || !k || !v || !out || !den || !grad_out || !grad_q || !grad_k || !grad_v)
    return fail(FASTMAX_E_ARG, "NULL tensor pointer");
  if (p.normalize && !stats) return fail(FASTMAX_E_ARG, "normalize needs the forward's stats buffer");
  int impl;
  if ((rc = pick_impl(p, false, &impl))) return rc;
  if (p.impl == FASTMAX_IMPL_AUTO && impl == FASTMAX_IMPL_DENSE_TC &&
      !aligned16({q, k, v, out, grad_out, grad_q, grad_k, grad_v}))
    impl = FASTMAX_IMPL_DENSE_FFMA;
  if (heads_per_batch && (rc = bt_layout_ok(p, heads_per_batch, impl))) return rc;
  BwdWs w = bwd_layout(p);
  const size_t need = impl == FASTMAX_IMPL_MOMENTS ? moments_bwd_layout(p).bytes : w.total;
  if (need > 0 && (!workspace || workspace_bytes < need))
    return fail(FASTMAX_E_WORKSPACE, "backward workspace too small: need %zu bytes, got %zu", need,
                workspace_bytes);
  if ((rc = check_device())) return rc;
  Ctx c{p, (cudaStream_t)stream};
  c.out_heads = heads_per_batch;
  if (impl == FASTMAX_IMPL_MOMENTS)
    return moments_backward(c, q, k, v, out, den, (const stat_t*)stats, grad_out, grad_q, grad_k, grad_v,
                            workspace,
                            (stats && keeps_total(p, impl)) ? (const float*)((const char*)stats + stats_words_bytes(p))
                                                            : nullptr);
  float* dots = (float*)((char*)workspace + w.dots_off);
  float* delta = (float*)((char*)workspace + w.delta_off);
  if (p.normalize)
    FM_CUDA_TRY(cudaMemsetAsync(dots, 0, sizeof(float) * (size_t)(p.bh + p.bhkv), c.stream));
  if (impl == FASTMAX_IMPL_DENSE_TC) {
    void* gs = (char*)workspace + w.gs_off;
    if ((rc = launch_gprep(c, grad_out, out, den, gs, delta))) return rc;
    if ((rc = dense_tc_backward(c, q, k, v, gs, delta, (const stat_t*)stats, dots, grad_q, grad_k,
                                grad_v)))
      return rc;
  } else {
    if ((rc = launch_delta(c, grad_out, out, delta))) return rc;
    if ((rc = dense_ffma_backward(c, q, k, v, den, (const stat_t*)stats, grad_out, delta, dots,
                                  grad_q, grad_k, grad_v)))
      return rc;
  }
  if (p.normalize)
    return launch_norm_fixup(c, q, k, (const stat_t*)stats, dots, grad_q, grad_k);
  return FASTMAX_OK;
}

int fastmax_b200_backward(const fastmax_problem* prob, const void* q, const void* k, const void* v,
                          const void* out, const float* den, const void* stats,
                          const void* grad_out, void* grad_q, void* grad_k, void* grad_v,
                          void* workspace, size_t workspace_bytes, void* stream) {
  return backward_impl(prob, q, k, v, out, den, stats, grad_out, grad_q, grad_k, grad_v, workspace, workspace_bytes,
                       stream, 0);
}

int fastmax_b200_backward_bt(const fastmax_problem* prob, const void* q, const void* k, const void* v,
                             const void* out_bt, const float* den, const void* stats, const void* grad_out_bt,
                             int32_t heads_per_batch, void* grad_q, void* grad_k, void* grad_v, void* workspace,
                             size_t workspace_bytes, void* stream) {
  if (heads_per_batch <= 0) return fail(FASTMAX_E_ARG, "heads_per_batch must be positive");
  return backward_impl(prob, q, k, v, out_bt, den, stats, grad_out_bt, grad_q, grad_k, grad_v, workspace,
                       workspace_bytes, stream, heads_per_batch);
}

// ---- sequence sharding ------------------------------------------------------------------
static int validate_shard(const fastmax_problem* prob) {
  int rc = validate(prob);
  if (rc) return rc;
  if (prob->nq != prob->nk || prob->bh != prob->bhkv)
    return fail(FASTMAX_E_ARG, "a sequence shard needs nq == nk and bh == bhkv");
  return check_device();
}
static size_t shard_s16_bytes(const fastmax_problem& p) { return state16_bytes(p, p.nq); }
struct ShardFwdWs { size_t o_add, den_add, s16, bytes; };
static ShardFwdWs shard_fwd_layout(const fastmax_problem& p) {
  ShardFwdWs w;
  w.o_add = 0;
  w.den_add = align_up(sizeof(float) * (size_t)p.bh * p.nq * p.d, 256);
  w.s16 = w.den_add + align_up(sizeof(float) * (size_t)p.bh * p.nq, 256);
  w.bytes = w.s16 + shard_s16_bytes(p);
  return w;
}
struct ShardBwdWs { size_t gq, gk, gv, dvec, gs, s16, bytes; };
static ShardBwdWs shard_bwd_layout(const fastmax_problem& p) {
  ShardBwdWs w;
  const size_t t = align_up(sizeof(float) * (size_t)p.bh * p.nq * p.d, 256);
  w.gq = 0;
  w.gk = t;
  w.gv = 2 * t;
  w.dvec = 3 * t;
  w.gs = w.dvec + align_up(sizeof(float) * (size_t)p.bh * p.nq, 256);
  w.s16 = w.gs + (dense_tc_supports(p) ? align_up((size_t)2 * p.bh * p.nq * p.d, 256) : 0);
  w.bytes = w.s16 + shard_s16_bytes(p);
  return w;
}

size_t fastmax_b200_moment_state_bytes(const fastmax_problem* p) {
  return validate(p) ? 0 : moment_state_bytes(*p, p->nk);
}
size_t fastmax_b200_moment_total_bytes(const fastmax_problem* p) {
  return validate(p) ? 0 : moment_total_bytes(*p);
}
size_t fastmax_b200_shard_forward_workspace_bytes(const fastmax_problem* p) {
  return validate(p) ? 0 : shard_fwd_layout(*p).bytes;
}
size_t fastmax_b200_shard_backward_workspace_bytes(const fastmax_problem* p) {
  return validate(p) ? 0 : shard_bwd_layout(*p).bytes;
}

int fastmax_b200_shard_rowmax(const fastmax_problem* prob, const void* q, const void* k,
                              int32_t row_offset, void* stats, void* stream) {
  int rc = validate_shard(prob);
  if (rc) return rc;
  if (!q || !k || !stats) return fail(FASTMAX_E_ARG, "NULL tensor pointer");
  Ctx c{*prob, (cudaStream_t)stream};
  return launch_rowmax(c, q, k, (stat_t*)stats, row_offset);
}

int fastmax_b200_shard_kv_state(const fastmax_problem* prob, const void* k, const void* v,
                                float* kv_states, float* kv_total, void* stream) {
  int rc = validate_shard(prob);
  if (rc) return rc;
  if (!k || !v || !kv_states || !kv_total) return fail(FASTMAX_E_ARG, "NULL tensor pointer");
  const fastmax_problem& p = *prob;
  Ctx c{p, (cudaStream_t)stream};
  const int L = moments_chunk(p);
  if ((rc = moments_build_states(c, p.nk, k, v, nullptr, nullptr, 0, nullptr, nullptr, kv_states))) return rc;
  return moments_prefix(c, p.bh, (p.nk + L - 1) / L, kv_states, nullptr, kv_total, 0, 0);
}

int fastmax_b200_shard_forward(const fastmax_problem* prob, const void* q, const void* k,
                               const void* v, const void* stats, float* kv_states,
                               const float* s_base, void* out, float* den, void* workspace,
                               size_t workspace_bytes, void* stream) {
  int rc = validate_shard(prob);
  if (rc) return rc;
  const fastmax_problem& p = *prob;
  if (!q || !k || !v || !out || !den) return fail(FASTMAX_E_ARG, "NULL tensor pointer");
  if (p.mask && !kv_states) return fail(FASTMAX_E_ARG, "NULL tensor pointer");
  if (!p.mask && !s_base) return fail(FASTMAX_E_ARG, "an unmasked shard needs the total of all shards in s_base");
  if (p.normalize && !stats) return fail(FASTMAX_E_ARG, "normalize needs the reduced stats buffer");
  const ShardFwdWs w = shard_fwd_layout(p);
  if (!workspace || workspace_bytes < w.bytes)
    return fail(FASTMAX_E_WORKSPACE, "shard forward workspace too small: need %zu bytes, got %zu", w.bytes,
                workspace_bytes);
  Ctx c{p, (cudaStream_t)stream};
  FwdOut o{out, den, p.d, 1, 0};
  if (!p.mask)   // every query reads the total over all shards
    return moments_forward_total(c, q, (const stat_t*)stats, s_base, (float*)((char*)workspace + w.o_add),
                                 (float*)((char*)workspace + w.den_add), (char*)workspace + w.s16, o);
  return moments_forward_finish(c, q, k, v, (const stat_t*)stats, kv_states, s_base,
                                (float*)((char*)workspace + w.o_add),
                                (float*)((char*)workspace + w.den_add), (char*)workspace + w.s16, o);
}

int fastmax_b200_shard_qg_state(const fastmax_problem* prob, const void* q, const void* out,
                                const float* den, const void* grad_out, float* delta,
                                float* qg_states, float* qg_total, void* workspace,
                                size_t workspace_bytes, void* stream) {
  int rc = validate_shard(prob);
  if (rc) return rc;
  const fastmax_problem& p = *prob;
  if (!q || !out || !den || !grad_out || !delta || !qg_states || !qg_total)
    return fail(FASTMAX_E_ARG, "NULL tensor pointer");
  const ShardBwdWs w = shard_bwd_layout(p);
  if (!workspace || workspace_bytes < w.bytes)
    return fail(FASTMAX_E_WORKSPACE, "shard backward workspace too small: need %zu bytes, got %zu", w.bytes,
                workspace_bytes);
  Ctx c{p, (cudaStream_t)stream};
  const int L = moments_chunk(p);
  char* ws = (char*)workspace;
  float* dvec = (float*)(ws + w.dvec);
  void* gs = ws + w.gs;
  if ((rc = launch_delta(c, grad_out, out, delta))) return rc;
  if (dense_tc_supports(p) && (rc = launch_gprep(c, grad_out, out, den, gs, dvec))) return rc;
  if ((rc = moments_build_states(c, p.nq, q, grad_out, den, delta, 1, gs, dvec, qg_states))) return rc;
  return moments_prefix(c, p.bh, (p.nq + L - 1) / L, qg_states, nullptr, qg_total, 1, 0);
}

int fastmax_b200_shard_backward(const fastmax_problem* prob, const void* q, const void* k,
                                const void* v, const void* out, const float* den,
                                const void* stats, const void* grad_out, const float* delta,
                                const float* kv_states, float* qg_states, const float* r_base,
                                float* dots, void* grad_q, void* grad_k, void* grad_v,
                                int32_t dq_far_done, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = validate_shard(prob);
  if (rc) return rc;
  const fastmax_problem& p = *prob;
  if (!q || !k || !v || !out || !den || !grad_out || !delta || !kv_states || !dots || !grad_q || !grad_k ||
      !grad_v)
    return fail(FASTMAX_E_ARG, "NULL tensor pointer");
  if (p.mask && !qg_states) return fail(FASTMAX_E_ARG, "NULL tensor pointer");
  if (!p.mask && !r_base)
    return fail(FASTMAX_E_ARG, "an unmasked shard needs the query/gradient total of all shards in r_base");
  if (p.normalize && !stats) return fail(FASTMAX_E_ARG, "normalize needs the reduced stats buffer");
  const ShardBwdWs w = shard_bwd_layout(p);
  if (!workspace || workspace_bytes < w.bytes)
    return fail(FASTMAX_E_WORKSPACE, "shard backward workspace too small: need %zu bytes, got %zu", w.bytes,
                workspace_bytes);
  Ctx c{p, (cudaStream_t)stream};
  char* ws = (char*)workspace;
  FM_CUDA_TRY(cudaMemsetAsync(dots, 0, sizeof(float) * (size_t)(p.bh + p.bhkv), c.stream));
  float* dvec = (float*)(ws + w.dvec);
  void* gs = ws + w.gs;
  // gs and dvec are still in the workspace when shard_dq_far ran on it
  if (!(dq_far_done && p.mask) && dense_tc_supports(p) && (rc = launch_gprep(c, grad_out, out, den, gs, dvec)))
    return rc;
  if (!p.mask)   // kv_states holds the key/value total of all shards, r_base the query/gradient total
    return moments_backward_total(c, q, k, v, den, (const stat_t*)stats, grad_out, delta, dvec, gs, kv_states,
                                  r_base, (float*)(ws + w.gq), (float*)(ws + w.gk), (float*)(ws + w.gv),
                                  ws + w.s16, p.normalize ? dots : nullptr, grad_q, grad_k, grad_v);
  return moments_backward_finish(c, q, k, v, den, (const stat_t*)stats, grad_out, delta, dvec, gs,
                                 kv_states, qg_states, r_base, (float*)(ws + w.gq), (float*)(ws + w.gk),
                                 (float*)(ws + w.gv), ws + w.s16, p.normalize ? dots : nullptr, grad_q, grad_k,
                                 grad_v, dq_far_done != 0);
}

int fastmax_b200_shard_dq_far(const fastmax_problem* prob, const void* q, const float* den, const void* stats,
                              const void* grad_out, const float* delta, const float* kv_states, void* workspace,
                              size_t workspace_bytes, void* stream) {
  int rc = validate_shard(prob);
  if (rc) return rc;
  const fastmax_problem& p = *prob;
  if (!p.mask) return fail(FASTMAX_E_ARG, "shard_dq_far applies to causal shards only");
  if (!q || !den || !grad_out || !delta || !kv_states) return fail(FASTMAX_E_ARG, "NULL tensor pointer");
  if (p.normalize && !stats) return fail(FASTMAX_E_ARG, "normalize needs the reduced stats buffer");
  const ShardBwdWs w = shard_bwd_layout(p);
  if (!workspace || workspace_bytes < w.bytes)
    return fail(FASTMAX_E_WORKSPACE, "shard backward workspace too small: need %zu bytes, got %zu", w.bytes,
                workspace_bytes);
  Ctx c{p, (cudaStream_t)stream};
  char* ws = (char*)workspace;
  return moments_backward_dq_far(c, q, den, (const stat_t*)stats, grad_out, delta, (const float*)(ws + w.dvec),
                                 ws + w.gs, kv_states, (float*)(ws + w.gq), ws + w.s16);
}

int fastmax_b200_shard_sum_totals(const float* gathered, int32_t world, int32_t rank, int32_t reverse,
                                  size_t floats_per_shard, float* out, void* stream) {
  if (!gathered || !out || world <= 0 || rank < 0 || rank >= world)
    return fail(FASTMAX_E_ARG, "bad arguments to shard_sum_totals");
  return launch_sum_totals(gathered, world, rank, reverse, floats_per_shard, out, (cudaStream_t)stream);
}

int fastmax_b200_shard_norm_fixup(const fastmax_problem* prob, const void* q, const void* k,
                                  const void* stats, const float* dots, int32_t row_offset,
                                  void* grad_q, void* grad_k, void* stream) {
  int rc = validate_shard(prob);
  if (rc) return rc;
  if (!q || !k || !stats || !dots || !grad_q || !grad_k) return fail(FASTMAX_E_ARG, "NULL tensor pointer");
  Ctx c{*prob, (cudaStream_t)stream};
  return launch_norm_fixup(c, q, k, (const stat_t*)stats, dots, grad_q, grad_k, row_offset);
}

}  // extern "C"
