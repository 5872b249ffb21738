// Host-side orchestration of the moment-state form: which kernels run, in which
// order, on which slices of the caller's workspace.  The same stages serve a
// whole sequence on one GPU and one contiguous shard of a sequence split over
// several GPUs; in the sharded case the caller exchanges the per-shard totals
// between the stages (see include/fastmax_b200.h).
#include "fm_common.cuh"

namespace fm {

static size_t up256(size_t x) { return (x + 255) / 256 * 256; }

int moments_chunk(const fastmax_problem& p) {
  // 2048 tokens per chunk: measured best for the tensor-core kernels (8.9 ms at 1024, 7.8 at 2048, 8.2 at
  // 4096 per step for 8 heads of 65536 tokens); fewer, larger chunks mean fewer states to build, scan and convert
  int L = p.chunk > 0 ? p.chunk : 2048;
  L = (L + 255) / 256 * 256;
  return L;
}

size_t moment_state_bytes(const fastmax_problem& p, int n) {
  const MomentDims m = moment_dims(p.d, p.p);
  const int L = moments_chunk(p);
  return up256(sizeof(float) * (size_t)p.bh * ((n + L - 1) / L) * m.f * m.dvp);
}
size_t moment_total_bytes(const fastmax_problem& p) {
  const MomentDims m = moment_dims(p.d, p.p);
  return up256(sizeof(float) * (size_t)p.bh * m.f * m.dvp);
}

// bf16 transposed copy of the second-order block of every chunk state (tensor-core read-out)
// layout: [second-order copies (tensor-core read-out)][first-order copies]
static size_t state16_second(const fastmax_problem& p, int mats) {
  return moments_tc_supports(p) ? up256(moments_tc_state_bytes(mats)) : 0;
}
size_t state16_bytes(const fastmax_problem& p, int n) {
  const int L = moments_chunk(p);
  const int mats = p.bh * ((n + L - 1) / L);
  return state16_second(p, mats) + (first_tc_supports(p) ? up256(first_tc_copy_bytes(p, mats)) : 0);
}

// second-order bf16 copies of the key/value chunk prefixes that a causal forward leaves for the backward
size_t moment_kept16_bytes(const fastmax_problem& p) {
  const int L = moments_chunk(p);
  return state16_second(p, p.bh * ((p.nk + L - 1) / L));
}

bool moments_all_tc(const fastmax_problem& p) {
  return dense_tc_supports(p) && first_tc_supports(p) && (p.p == 1 || moments_tc_supports(p));
}

bool moments_supports(const fastmax_problem& p) {
  return p.bh == p.bhkv && (!p.mask || p.nq == p.nk);
}

// Workspace of the one-call forward: [states][total][o_add][den_add]
MomFwdWs moments_fwd_layout(const fastmax_problem& p) {
  MomFwdWs w;
  w.states = 0;
  w.total = w.states + moment_state_bytes(p, p.nk);
  w.o_add = w.total + moment_total_bytes(p);
  w.den_add = w.o_add + up256(sizeof(float) * (size_t)p.bh * p.nq * p.d);
  w.s16 = w.den_add + up256(sizeof(float) * (size_t)p.bh * p.nq);
  w.bytes = w.s16 + state16_bytes(p, p.nk);
  return w;
}
// Workspace of the one-call backward:
// [dots][delta][dvec][gs][states][total][gq_add][gk_add][gv_add]
MomBwdWs moments_bwd_layout(const fastmax_problem& p) {
  MomBwdWs w;
  w.dots = 0;
  w.delta = up256(sizeof(float) * (size_t)(p.bh + p.bhkv));
  w.dvec = w.delta + up256(sizeof(float) * (size_t)p.bh * p.nq);
  w.gs = w.dvec + up256(sizeof(float) * (size_t)p.bh * p.nq);
  w.states = w.gs + (dense_tc_supports(p) ? up256((size_t)2 * p.bh * p.nq * p.d) : 0);
  w.total = w.states + moment_state_bytes(p, p.nk > p.nq ? p.nk : p.nq);
  w.gq_add = w.total + moment_total_bytes(p);
  w.gk_add = w.gq_add + up256(sizeof(float) * (size_t)p.bh * p.nq * p.d);
  w.gv_add = w.gk_add + up256(sizeof(float) * (size_t)p.bhkv * p.nk * p.d);
  w.s16 = w.gv_add + up256(sizeof(float) * (size_t)p.bhkv * p.nk * p.d);
  w.bytes = w.s16 + state16_bytes(p, p.nk > p.nq ? p.nk : p.nq);
  return w;
}

int moments_build_states(const Ctx& c, int n, const void* y, const void* z, const float* den,
                         const float* delta, int ext, const void* gs, const float* dvec, float* states) {
  const fastmax_problem& p = c.p;
  const int L = moments_chunk(p);
  const bool tc2 = moments_tc_supports(p), tc1 = first_tc_supports(p);
  int rc;
  // second-order rows: tensor cores where built, else everything on the CUDA cores
  if (p.p == 2) {
    if (!tc2) return moments_chunk_state(c, p.bh, n, L, y, z, den, delta, ext, states);
    if ((rc = moments_tc_chunk_state(c, p.bh, n, L, y, ext ? gs : z, ext ? dvec : nullptr, states))) return rc;
  }
  // first-order and constant rows
  if (tc1) return first_tc_chunk_state(c, p.bh, n, L, y, ext ? gs : z, ext ? dvec : nullptr, states);
  return moments_chunk_state(c, p.bh, n, L, y, z, den, delta, ext, states, 1);
}

// read-out of prefix (or total) states for n tokens; mode 0: type A, 1: type B, 2: both on x
// second16 (may be null): second-order bf16 copies that exist already (prefix_states, or kept by the forward)
static int read_states(const Ctx& c, int mode, int n, int per_chunk, const void* x, const void* u,
                       const float* den, const float* delta, int ext, const void* gs, const float* dvec,
                       const float* states, void* s16, const stat_t* stats, float* out_a, float* den_a,
                       float* out_b, const void* second16 = nullptr) {
  const fastmax_problem& p = c.p;
  const int L = moments_chunk(p);
  int rc;
  const bool tc2 = moments_tc_supports(p);
  const bool tc1 = first_tc_supports(p) && (p.p == 1 || tc2);
  const int mats = p.bh * (per_chunk ? (n + L - 1) / L : 1);
  if (tc2) {
    if (!second16 && (rc = moments_tc_convert(c, mats, states, s16))) return rc;
    // both kinds come out complete: the first-order and constant terms ride on the copy's last rows
    return moments_tc_readout(c, mode, p.bh, n, L, per_chunk, x, ext ? gs : u, ext ? dvec : nullptr,
                              second16 ? second16 : s16, stats, out_a, den_a, out_b, states);
  }
  if (tc1) {
    // first-order part on tensor cores; it adds to the second-order part when there is one
    void* s1b = (char*)s16 + state16_second(p, mats);
    if ((rc = first_tc_convert(c, mats, states, s1b))) return rc;
    if ((mode == 0 || mode == 2) && !tc2)
      if ((rc = first_tc_readout(c, 0, p.bh, n, L, per_chunk, x, x, nullptr, states, s1b, stats, out_a, den_a,
                                 tc2)))
        return rc;
    if (mode == 1 || mode == 2)
      if ((rc = first_tc_readout(c, 1, p.bh, n, L, per_chunk, ext ? gs : u, x, ext ? dvec : nullptr, states,
                                 s1b, stats, out_b, nullptr, tc2)))
        return rc;
    return FASTMAX_OK;
  }
  if ((mode == 0 || mode == 2) && !tc2)
    if ((rc = moments_readout(c, 0, p.bh, n, L, per_chunk, x, nullptr, nullptr, nullptr, 0, states, stats,
                              out_a, den_a, tc2)))
      return rc;
  if (mode == 1 || mode == 2)
    if ((rc = moments_readout(c, 1, p.bh, n, L, per_chunk, x, u, den, delta, ext, states, stats, out_b,
                              nullptr, tc2)))
      return rc;
  return FASTMAX_OK;
}

// p = 1 on tensor cores without a score-form part: the read-out of the total state is the
// result, so it is divided / rounded in the read-out kernel itself
static bool first_is_whole(const fastmax_problem& p) { return p.p == 1 && !p.mask && first_tc_supports(p); }
static int read_first_final(const Ctx& c, int type_b, int n, const void* tile, const void* x, const float* uvec,
                            const float* total, void* s16, const stat_t* stats, int final, void* out,
                            float* den_out, float* dots) {
  int rc;
  if ((rc = first_tc_convert(c, c.p.bh, total, s16))) return rc;
  return first_tc_readout(c, type_b, c.p.bh, n, moments_chunk(c.p), 0, tile, x, uvec, total, s16, stats, nullptr,
                          nullptr, 0, final, out, den_out, dots);
}

// Exclusive running sums over the chunks of every head (per-chunk mode).  With `fuse` and the tensor-core
// second-order part, the second-order rows go straight to their bf16 transposed copies at `second16` in one
// pass over the raw states and stay raw in `states` (nothing else reads them); only the first-order rows are
// summed in place.  *ready tells whether `second16` holds the copies.
static int prefix_states(const Ctx& c, int nchunk, float* states, const float* base, int reverse, bool fuse,
                         void* second16, bool* ready) {
  const fastmax_problem& p = c.p;
  *ready = fuse && p.p == 2 && moments_tc_supports(p);
  if (!*ready) return moments_prefix(c, p.bh, nchunk, states, base, nullptr, reverse, 1);
  int rc;
  // first the first-order rows in place: the copies carry them too (their last 64 rows)
  if ((rc = moments_prefix(c, p.bh, nchunk, states, base, nullptr, reverse, 1, p.d * p.d))) return rc;
  return moments_tc_prefix_convert(c, p.bh, nchunk, states, base, reverse, second16);
}

// Copies of the context that tell the tensor-core moment kernels which chunk's state nothing will read,
// and whose tokens read an empty running sum (see Ctx).
static Ctx skipping(const Ctx& c, int chunk) { Ctx r = c; r.skip_chunk = chunk; return r; }
static Ctx zeroing(const Ctx& c, int chunk) { Ctx r = c; r.zero_chunk = chunk; return r; }

// ---- forward -----------------------------------------------------------------------
// kv_states: raw chunk states of (k, v) for this shard (already built); s_base: sum of the
// totals of all earlier shards or null.  Turns the states into prefixes in place.
int moments_forward_finish(const Ctx& c, const void* q, const void* k, const void* v,
                           const stat_t* stats, float* kv_states, const float* s_base,
                           float* o_add, float* den_add, void* s16, const FwdOut& o, void* second16) {
  const fastmax_problem& p = c.p;
  const int L = moments_chunk(p);
  const int nchunk = (p.nk + L - 1) / L;
  int rc;
  // second16 != null: the caller does not need the fp32 second-order prefixes (see prefix_states)
  bool ready;
  if ((rc = prefix_states(c, nchunk, kv_states, s_base, 0, second16 != nullptr, second16, &ready))) return rc;
  // without a base the tokens of the first chunk have nothing before them
  if ((rc = read_states(zeroing(c, s_base ? -1 : 0), 0, p.nq, 1, q, nullptr, nullptr, nullptr, 0, nullptr, nullptr,
                        kv_states, s16, stats, o_add, den_add, nullptr, ready ? second16 : nullptr)))
    return rc;
  ChunkAdd ca;
  ca.chunk = L;
  ca.out_add = o_add;
  ca.den_add = den_add;
  if (dense_tc_supports(p) && !o.out_f32) return dense_tc_forward(c, q, k, v, stats, o.out, o.den, &ca);
  return dense_ffma_forward(c, q, k, v, stats, o, ca);
}

// total_keep (may be null): where the forward leaves what the backward would otherwise rebuild from k and v --
// unmasked: the total key/value state; causal: the chunk states of the keys and values (first-order rows as
// exclusive prefixes; with the tensor-core second-order part those rows stay raw and their prefixes follow
// as bf16 transposed copies, moment_kept16_bytes)
int moments_forward(const Ctx& c, const void* q, const void* k, const void* v, const stat_t* stats,
                    const FwdOut& o, void* workspace, float* total_keep) {
  const fastmax_problem& p = c.p;
  const int L = moments_chunk(p);
  const MomFwdWs w = moments_fwd_layout(p);
  char* ws = (char*)workspace;
  float* states = (p.mask && total_keep) ? total_keep : (float*)(ws + w.states);
  float* total = (!p.mask && total_keep) ? total_keep : (float*)(ws + w.total);
  float* o_add = (float*)(ws + w.o_add);
  float* den_add = (float*)(ws + w.den_add);
  int rc;
  void* s16 = ws + w.s16;
  // causal: nothing comes after the last chunk, so its state is not built
  const int last = (p.nk + L - 1) / L - 1;
  if ((rc = moments_build_states(p.mask ? skipping(c, last) : c, p.nk, k, v, nullptr, nullptr, 0, nullptr, nullptr,
                                 states)))
    return rc;
  if (p.mask) {
    // second-order prefixes go straight to their bf16 copies: behind the kept fp32 states when the
    // backward will want them again, else in the workspace
    void* second16 = total_keep ? (void*)((char*)total_keep + moment_state_bytes(p, p.nk)) : s16;
    return moments_forward_finish(c, q, k, v, stats, states, nullptr, o_add, den_add, s16, o, second16);
  }
  // unmasked: every query reads the total of all keys
  const int nchunk = (p.nk + L - 1) / L;
  if ((rc = moments_prefix(c, p.bh, nchunk, states, nullptr, total, 0, 0))) return rc;
  return moments_forward_total(c, q, stats, total, o_add, den_add, s16, o);
}

// Unmasked forward from a given total state (this device's keys, or the sum over all shards).
int moments_forward_total(const Ctx& c, const void* q, const stat_t* stats, const float* total, float* o_add,
                          float* den_add, void* s16, const FwdOut& o) {
  const fastmax_problem& p = c.p;
  int rc;
  if (o.out_f32 || o.o_stride != p.d)
    return fail(FASTMAX_E_UNSUPPORTED, "the moment family writes the plain output layout only");
  if (first_is_whole(p))
    return read_first_final(c, 0, p.nq, q, q, nullptr, total, s16, stats, 1, o.out, o.den, nullptr);
  if ((rc = read_states(c, 0, p.nq, 0, q, nullptr, nullptr, nullptr, 0, nullptr, nullptr, total, s16, stats,
                        o_add, den_add, nullptr)))
    return rc;
  return moments_finalize(c, p.bh, p.nq, o_add, den_add, nullptr, o.out, o.den, nullptr, 0);
}

// ---- backward ----------------------------------------------------------------------
// The part of grad_q that reads the key/value prefixes (everything before a token's own chunk).  It
// depends on nothing from later shards, so a sequence shard issues it while the query/gradient
// totals are being exchanged.
int moments_backward_dq_far(const Ctx& c, const void* q, const float* den, const stat_t* stats,
                            const void* grad_out, const float* delta, const float* dvec, const void* gs,
                            const float* s_states, float* gq_add, void* s16) {
  return read_states(c, 1, c.p.nq, 1, q, grad_out, den, delta, 1, gs, dvec, s_states, s16, stats, nullptr,
                     nullptr, gq_add);
}

// s_states: exclusive prefixes of the (k, v) chunk states (as left by the forward finish);
// r_states: raw chunk states of (q, grad_out/den | -delta/den); r_base: sum of the totals of
// all later shards or null.  Writes the three gradients without the normalisation row fix.
int moments_backward_finish(const Ctx& c, const void* q, const void* k, const void* v,
                            const float* den, const stat_t* stats, const void* grad_out,
                            const float* delta, const float* dvec, const void* gs,
                            const float* s_states, float* r_states, const float* r_base,
                            float* gq_add, float* gk_add, float* gv_add, void* s16, float* dots,
                            void* grad_q, void* grad_k, void* grad_v, bool dq_far_done) {
  const fastmax_problem& p = c.p;
  const int L = moments_chunk(p);
  const int nchunk = (p.nq + L - 1) / L;
  int rc;
  // grad_q reads the key/value prefixes with u = [grad_out/den | -delta/den]
  if (!dq_far_done &&
      (rc = moments_backward_dq_far(c, q, den, stats, grad_out, delta, dvec, gs, s_states, gq_add, s16)))
    return rc;
  // grad_k and grad_v read the suffix sums of the query/gradient states
  // (nothing reads r_states after this call, so their second-order rows may stay raw: prefix_states)
  bool ready;
  if ((rc = prefix_states(c, nchunk, r_states, r_base, 1, true, s16, &ready))) return rc;
  if ((rc = read_states(zeroing(c, r_base ? -1 : nchunk - 1), 2, p.nk, 1, k, v, nullptr, nullptr, 0, nullptr, nullptr,
                        r_states, s16, stats, gv_add, nullptr, gk_add, ready ? s16 : nullptr)))
    return rc;
  ChunkAdd ca;
  ca.chunk = L;
  ca.gq_add = gq_add;
  ca.gk_add = gk_add;
  ca.gv_add = gv_add;
  if (dense_tc_supports(p))
    return dense_tc_backward(c, q, k, v, gs, dvec, stats, dots, grad_q, grad_k, grad_v, &ca);
  return dense_ffma_backward(c, q, k, v, den, stats, grad_out, delta, dots, grad_q, grad_k, grad_v, ca);
}

// kv_total_kept (may be null): what the forward left behind (unmasked: the total key/value state; causal: the
// exclusive prefixes of the key/value chunk states); without it the states are rebuilt from k and v
int moments_backward(const Ctx& c, const void* q, const void* k, const void* v, const void* out,
                     const float* den, const stat_t* stats, const void* grad_out, void* grad_q,
                     void* grad_k, void* grad_v, void* workspace, const float* kv_total_kept) {
  const fastmax_problem& p = c.p;
  const int L = moments_chunk(p);
  const MomBwdWs w = moments_bwd_layout(p);
  char* ws = (char*)workspace;
  float* dots = (float*)(ws + w.dots);
  float* delta = (float*)(ws + w.delta);
  float* dvec = (float*)(ws + w.dvec);
  void* gs = ws + w.gs;
  float* states = (float*)(ws + w.states);
  float* total = (float*)(ws + w.total);
  float* gq_add = (float*)(ws + w.gq_add);
  float* gk_add = (float*)(ws + w.gk_add);
  float* gv_add = (float*)(ws + w.gv_add);
  void* s16 = ws + w.s16;
  int rc;
  if (p.normalize)
    FM_CUDA_TRY(cudaMemsetAsync(dots, 0, sizeof(float) * (size_t)(p.bh + p.bhkv), c.stream));
  const bool tc = dense_tc_supports(p);
  // the plain row dots feed the CUDA-core kernels only; when every stage runs on tensor cores they
  // all read gs / dvec and the pass over grad_out and out is skipped
  const bool all_tc = moments_all_tc(p);
  if (!all_tc && (rc = launch_delta(c, grad_out, out, delta))) return rc;
  if (tc && (rc = launch_gprep(c, grad_out, out, den, gs, dvec))) return rc;
  const int nck = (p.nk + L - 1) / L, ncq = (p.nq + L - 1) / L;
  if (p.mask) {
    // the key/value prefixes are rebuilt (the forward does not keep them), used for grad_q,
    // then the buffer is reused for the query/gradient states
    bool ready = false;
    const void* kv16 = nullptr;   // second-order bf16 copies of the key/value prefixes, where they exist already
    if (!kv_total_kept) {
      if ((rc = moments_build_states(skipping(c, nck - 1), p.nk, k, v, nullptr, nullptr, 0, nullptr, nullptr, states)))
        return rc;
      if ((rc = prefix_states(c, nck, states, nullptr, 0, true, s16, &ready))) return rc;
      if (ready) kv16 = s16;
    } else if (moment_kept16_bytes(p) > 0) {
      kv16 = (const char*)kv_total_kept + moment_state_bytes(p, p.nk);
    }
    // grad_q: the first chunk's tokens have no keys before their chunk; grad_k, grad_v: the last chunk's
    // tokens no queries after theirs, and nothing reads the query/gradient state of the first chunk
    if ((rc = read_states(zeroing(c, 0), 1, p.nq, 1, q, grad_out, den, delta, 1, gs, dvec,
                          kv_total_kept ? kv_total_kept : states, s16, stats, nullptr, nullptr, gq_add, kv16)))
      return rc;
    if ((rc = moments_build_states(skipping(c, 0), p.nq, q, grad_out, den, delta, 1, gs, dvec, states))) return rc;
    if ((rc = prefix_states(c, ncq, states, nullptr, 1, true, s16, &ready))) return rc;
    if ((rc = read_states(zeroing(c, ncq - 1), 2, p.nk, 1, k, v, nullptr, nullptr, 0, nullptr, nullptr, states, s16,
                          stats, gv_add, nullptr, gk_add, ready ? s16 : nullptr)))
      return rc;
    ChunkAdd ca;
    ca.chunk = L;
    ca.gq_add = gq_add;
    ca.gk_add = gk_add;
    ca.gv_add = gv_add;
    if (tc) rc = dense_tc_backward(c, q, k, v, gs, dvec, stats, dots, grad_q, grad_k, grad_v, &ca);
    else rc = dense_ffma_backward(c, q, k, v, den, stats, grad_out, delta, dots, grad_q, grad_k, grad_v, ca);
    if (rc) return rc;
  } else {
    // unmasked: totals only, no score-form part.  The two totals share one buffer, so grad_q is
    // read out before the query/gradient total replaces the key/value total.
    if (!kv_total_kept) {
      if ((rc = moments_build_states(c, p.nk, k, v, nullptr, nullptr, 0, nullptr, nullptr, states))) return rc;
      if ((rc = moments_prefix(c, p.bh, nck, states, nullptr, total, 0, 0))) return rc;
    }
    if ((rc = moments_backward_total(c, q, k, v, den, stats, grad_out, delta, dvec, gs,
                                     kv_total_kept ? kv_total_kept : total, nullptr, gq_add,
                                     gk_add, gv_add, s16, dots, grad_q, nullptr, nullptr)))
      return rc;
    if ((rc = moments_build_states(c, p.nq, q, grad_out, den, delta, 1, gs, dvec, states))) return rc;
    if ((rc = moments_prefix(c, p.bh, ncq, states, nullptr, total, 0, 0))) return rc;
    if ((rc = moments_backward_total(c, q, k, v, den, stats, grad_out, delta, dvec, gs, nullptr, total, gq_add,
                                     gk_add, gv_add, s16, dots, nullptr, grad_k, grad_v)))
      return rc;
  }
  if (p.normalize) return launch_norm_fixup(c, q, k, stats, dots, grad_q, grad_k);
  return FASTMAX_OK;
}

// Unmasked gradients from given total states (this device's, or the sums over all shards): grad_q
// from the key/value total when kv_total and grad_q are given, grad_k and grad_v from the
// query/gradient total when qg_total and grad_k are given.  Without the normalisation row fix.
int moments_backward_total(const Ctx& c, const void* q, const void* k, const void* v, const float* den,
                           const stat_t* stats, const void* grad_out, const float* delta, const float* dvec,
                           const void* gs, const float* kv_total, const float* qg_total, float* gq_add,
                           float* gk_add, float* gv_add, void* s16, float* dots, void* grad_q, void* grad_k,
                           void* grad_v) {
  const fastmax_problem& p = c.p;
  int rc;
  if (kv_total && grad_q) {
    if (first_is_whole(p)) {
      if ((rc = read_first_final(c, 1, p.nq, gs, q, dvec, kv_total, s16, stats, 2, grad_q, nullptr,
                                 p.normalize ? dots : nullptr)))
        return rc;
    } else {
      if ((rc = read_states(c, 1, p.nq, 0, q, grad_out, den, delta, 1, gs, dvec, kv_total, s16, stats, nullptr,
                            nullptr, gq_add)))
        return rc;
      if ((rc = moments_finalize(c, p.bh, p.nq, gq_add, nullptr, q, grad_q, nullptr,
                                 p.normalize ? dots : nullptr, 1)))
        return rc;
    }
  }
  if (qg_total && grad_k) {
    if (first_is_whole(p)) {
      if ((rc = read_first_final(c, 1, p.nk, v, k, nullptr, qg_total, s16, stats, 2, grad_k, nullptr,
                                 p.normalize ? dots + p.bh : nullptr)))
        return rc;
      if ((rc = read_first_final(c, 0, p.nk, k, k, nullptr, qg_total, s16, stats, 2, grad_v, nullptr, nullptr)))
        return rc;
    } else {
      if ((rc = read_states(c, 2, p.nk, 0, k, v, nullptr, nullptr, 0, nullptr, nullptr, qg_total, s16, stats,
                            gv_add, nullptr, gk_add)))
        return rc;
      if ((rc = moments_finalize(c, p.bh, p.nk, gk_add, nullptr, k, grad_k, nullptr,
                                 p.normalize ? dots + p.bh : nullptr, 1)))
        return rc;
      if ((rc = moments_finalize(c, p.bh, p.nk, gv_add, nullptr, nullptr, grad_v, nullptr, nullptr, 1)))
        return rc;
    }
  }
  return FASTMAX_OK;
}

}  // namespace fm
