/*
 * fastmax_b200 -- C ABI of the B200 (sm_100a) Fastmax attention library.
 *
 * Fastmax attention scores a query/key pair with the polynomial
 *     f(s) = a0 + a1*s + a2*s^2,   s = q.k      (a2 = 0 when p == 1)
 * and row-normalises:  out_i = sum_j f(s_ij) v_j / sum_j f(s_ij),
 * j over all keys (mask == 0) or over j <= i + (nk - nq) (mask == 1, causal).
 * With normalize != 0, q and k are first scaled per head to
 *     x <- lim * x / max_n ||x_n||_2,
 * and the backward pass differentiates through that scaling.
 *
 * This header is what a foreign-function binding of the reference project
 * would bind instead of its `forward_cuda` / `backward_cuda` launchers.  Every
 * pointer is a device pointer unless said otherwise; all tensors are dense,
 * row-major and contiguous:
 *     q, out, grad_out, grad_q : (bh,   nq, d)
 *     k, v, grad_k, grad_v     : (bhkv, nk, d)      bh % bhkv == 0
 *     den                      : (bh, nq) float32   row sums of f(s)
 * The library allocates no device memory: the caller passes every output and
 * scratch buffer, sized by the *_bytes queries below.  Calls are asynchronous
 * on the given CUDA stream (a `cudaStream_t` passed as `void*`) and never
 * synchronise the device.  Inputs are never written.
 *
 * Every function returns FASTMAX_OK (0) or a negative FASTMAX_E_* code;
 * `fastmax_b200_last_error()` gives the message of the calling thread's last
 * failure.
 */
#ifndef FASTMAX_B200_H
#define FASTMAX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  FASTMAX_OK = 0,
  FASTMAX_E_ARG = -1,       /* bad shape, dtype, p, head dimension, null pointer */
  FASTMAX_E_WORKSPACE = -2, /* scratch buffer smaller than the *_bytes query */
  FASTMAX_E_CUDA = -3,      /* a CUDA runtime call or a kernel launch failed */
  FASTMAX_E_UNSUPPORTED = -4, /* valid request that this build has no kernel for */
  FASTMAX_E_DEVICE = -5     /* the current device is not compute capability 10.x */
};

enum { FASTMAX_F32 = 0, FASTMAX_BF16 = 1 };

/* Kernel family selection.  AUTO picks the fastest family that supports the
 * problem; the others force one family (used by the parity tests to compare
 * families against each other). */
enum {
  FASTMAX_IMPL_AUTO = 0,
  FASTMAX_IMPL_DENSE_FFMA = 1,   /* tiled score form on CUDA cores, fp32 math */
  FASTMAX_IMPL_DENSE_TC = 2,     /* tiled score form on tcgen05 tensor cores (bf16) */
  FASTMAX_IMPL_MOMENTS = 3,      /* chunked moment-state form: states built and read on tcgen05 where a
                                    kernel exists (bf16: second order at d == 64, first order at d in
                                    {64, 128}), otherwise on CUDA cores; each chunk's own block in score
                                    form on the best family for the problem */
  FASTMAX_IMPL_MOMENTS_FFMA = 4  /* the same with every state kernel on CUDA cores (any d and dtype) */
};

/* One attention problem.  Mirrors the argument list of the reference's
 * forwardpass(q,k,v,drop_noise,[rpe_matrix,]mask,dropout,normalize,temperature,
 * a0,a1,a2,lim,p) (reference fastmax_cuda.cpp:17-24).  `temperature` is carried
 * for signature compatibility and has no effect, as in the reference's
 * pure-PyTorch path (reference example.py:102,110-111). */
typedef struct fastmax_problem {
  int32_t dtype;      /* FASTMAX_F32 or FASTMAX_BF16: element type of q,k,v,out,grads */
  int32_t bh;         /* batch*heads of q */
  int32_t bhkv;       /* batch*heads of k and v; bh % bhkv == 0 */
  int32_t nq;         /* query tokens */
  int32_t nk;         /* key tokens; causal needs nk >= nq */
  int32_t d;          /* head dimension: 8,16,32,64 or 128 */
  int32_t mask;       /* 0 = all keys, 1 = causal */
  int32_t normalize;  /* 0/1 */
  int32_t p;          /* polynomial order, 1 or 2 */
  int32_t impl;       /* FASTMAX_IMPL_* */
  float a0, a1, a2;
  float lim;
  float temperature;
  int32_t chunk;      /* moment family: tokens per chunk (multiple of 256); 0 = library default */
} fastmax_problem;

/* Library version (major*10000 + minor*100 + patch). */
int fastmax_b200_version(void);

/* Message of the calling thread's most recent failure ("" if none). */
const char* fastmax_b200_last_error(void);

/* Launch accounting (no counterpart in the reference, which times itself with
 * host clocks around device-wide synchronisations, test_fastmax.py:351-356).
 * launch_count: kernels this process has launched through the library so far.
 * profile_enable(1) discards earlier records and starts bracketing every
 * launch with CUDA events on its stream; profile_enable(0) stops and discards.
 * profile_get waits for record i to finish and returns its kernel name and
 * device time in milliseconds. */
unsigned long long fastmax_b200_launch_count(void);
int fastmax_b200_profile_enable(int on);
int fastmax_b200_profile_count(void);
int fastmax_b200_profile_get(int i, char* name, int name_len, float* ms);

/* Device-side protocol status (no counterpart in the reference).  The
 * tensor-core kernels bound every wait on a barrier; a wait that gives up stores
 * a non-zero code in a device word and the kernel winds down instead of
 * hanging.  This call synchronises `stream` and copies the word to *status
 * (host pointer): 0 means no kernel of this process gave up a wait since the last reset. */
int fastmax_b200_device_status(int* status, void* stream);
/* Clears the status word (synchronises `stream`), so that a later give-up can be told from
 * an earlier one. */
int fastmax_b200_device_status_reset(void* stream);
/* Exercises the give-up path without disturbing a real kernel: launches one warp that waits,
 * bounded by limit_clocks SM clocks (at most the kernels' own limit, about a second), on a
 * barrier that nothing ever completes.  The kernel returns once the limit has passed -- the
 * wait is re-armed in steps of up to 1.6 ms -- and fastmax_b200_device_status then reports 99.
 * Nothing faults and the context stays usable. */
int fastmax_b200_wait_selftest(long long limit_clocks, void* stream);

/* Bytes of the per-head statistics buffer that forward writes and backward
 * reads: the max row norms and their row indices and, for problems that run on
 * the moment family, the key/value moment states backward would otherwise
 * rebuild (unmasked: their total; causal: the per-chunk states and the bf16
 * copies of their running sums that the read-out multiplies, about 1.6 times
 * the size of q + k + v + out at d = 64).  backward must be given the buffer the
 * forward call of the same problem filled; with normalize == 0 it may be NULL,
 * and backward then recomputes what it needs.  Replaces the reference's
 * qnorms/knorms/qmaxes/kmaxes temporaries (reference fastmax_cuda_forward.cu:
 * 349-358), which it needs because it rescales q and k in place. */
size_t fastmax_b200_stats_bytes(const fastmax_problem* prob);

/* Which kernel family a forward or backward call with this problem runs, without
 * launching anything: one of FASTMAX_IMPL_DENSE_FFMA, FASTMAX_IMPL_DENSE_TC,
 * FASTMAX_IMPL_MOMENTS in *impl (prob->impl AUTO: the library's choice from its
 * rate model; a forced family: that family, or an error where it cannot serve the
 * problem).  Pure host arithmetic; needs no device.  The reference has one pair
 * of kernels per mask setting and no such choice (reference
 * fastmax_cuda_forward.cu:384-391). */
int fastmax_b200_selected_impl(const fastmax_problem* prob, int32_t* impl);

/* Bytes of scratch the forward / backward pass needs (may be 0). */
size_t fastmax_b200_forward_workspace_bytes(const fastmax_problem* prob);
size_t fastmax_b200_backward_workspace_bytes(const fastmax_problem* prob);

/* Forward pass.  Replaces forward_cuda (reference fastmax_cuda_forward.cu:
 * 297-411): normalisation (223-269), moment/score kernels (25-197, and the
 * second-order terms of `old stuff/fastmax_cuda_forward_quad.cu`:57-268) and
 * the division (199-210).  Writes out (element type of the inputs), den and
 * stats. */
int fastmax_b200_forward(const fastmax_problem* prob,
                         const void* q, const void* k, const void* v,
                         void* out, float* den, void* stats,
                         void* workspace, size_t workspace_bytes,
                         void* stream);

/* The same passes with the result and the upstream gradient in the layout the model's output
 * projection works on: out_bt and grad_out_bt are (batch, nq, heads_per_batch, d) arrays with
 * batch * heads_per_batch == bh, i.e. the reference's `o.transpose(1, 2)` (model.py:603) and its
 * inverse (the `.contiguous()` on the incoming gradient) are folded into the kernels that write
 * and read those tensors.  q, k, v, den and the gradients keep the (heads, n, d) layout.
 * Served by the tensor-core kernels only (bf16, d 64 or 128; the moment family when causal):
 * bt_layout_supported returns 1 when the problem qualifies, otherwise the calls return
 * FASTMAX_E_UNSUPPORTED and the caller swaps the axes itself (fastmax_b200_swap_middle_axes). */
int fastmax_b200_bt_layout_supported(const fastmax_problem* prob, int32_t heads_per_batch);
int fastmax_b200_forward_bt(const fastmax_problem* prob,
                            const void* q, const void* k, const void* v,
                            void* out_bt, float* den, void* stats, int32_t heads_per_batch,
                            void* workspace, size_t workspace_bytes, void* stream);
int fastmax_b200_backward_bt(const fastmax_problem* prob,
                             const void* q, const void* k, const void* v,
                             const void* out_bt, const float* den, const void* stats,
                             const void* grad_out_bt, int32_t heads_per_batch,
                             void* grad_q, void* grad_k, void* grad_v,
                             void* workspace, size_t workspace_bytes, void* stream);

/* Forward pass in the reference's packed layout: o is (bh, nq, d+1) float32
 * whose channels 0..d-1 hold the divided output and channel d the denominator
 * (reference fastmax_cuda_forward.cu:347, 199-210; the reference wrapper
 * slices o[:, :, :d], example.py:47).  stats may be NULL when normalize == 0. */
int fastmax_b200_forward_packed(const fastmax_problem* prob,
                                const void* q, const void* k, const void* v,
                                float* o_packed, void* stats,
                                void* workspace, size_t workspace_bytes,
                                void* stream);

/* Backward pass.  Replaces backward_cuda (reference fastmax_cuda_backward.cu:
 * 900-1006 and `old stuff/fastmax_cuda_backward_quad.cu`:26-479): given the
 * forward's out, den and stats and the upstream gradient, writes grad_q,
 * grad_k, grad_v (element type of the inputs).  Unlike the reference it does
 * not modify grad_out, and with normalize != 0 it includes the gradient of the
 * max-norm scaling, as autograd through the reference's PyTorch path does. */
int fastmax_b200_backward(const fastmax_problem* prob,
                          const void* q, const void* k, const void* v,
                          const void* out, const float* den, const void* stats,
                          const void* grad_out,
                          void* grad_q, void* grad_k, void* grad_v,
                          void* workspace, size_t workspace_bytes,
                          void* stream);

/* ---- sequence sharding ------------------------------------------------------
 * No counterpart in the reference, which has no multi-GPU code (its outputs are
 * hard-wired to cuda:0, fastmax_cuda_forward.cu:347).  A sequence is split
 * into contiguous shards, one per GPU, every shard holding all heads; `prob`
 * describes ONE shard (nq == nk == shard length, bh == bhkv); causal first.  The
 * moment states are additive over tokens, so a shard needs from the others only
 * the sum of their per-head totals: of all EARLIER shards' key/value states for
 * the forward pass and grad_q, of all LATER shards' query/gradient states for
 * grad_k and grad_v.  The caller moves those totals between GPUs (for instance an
 * NCCL all-gather followed by a local sum) between the calls below; the library
 * itself never communicates.  With normalize != 0 the caller also max-reduces the
 * stats words (as 64-bit integers) and sum-reduces the `dots` array over shards.
 *
 *   shard_rowmax      stats of this shard; recorded rows are row_offset + local row
 *   shard_kv_state    chunk states of (k, v) into kv_states, their sum into kv_total
 *   shard_forward     s_base = sum of earlier shards' kv_total (NULL on the first);
 *                     turns kv_states into running prefixes (keep them for backward)
 *   shard_qg_state    delta = grad_out.out per row, chunk states of (q, grad_out/den)
 *                     into qg_states, their sum into qg_total; takes the workspace that
 *                     shard_backward will be given (shard_backward_workspace_bytes)
 *   shard_backward    r_base = sum of later shards' qg_total (NULL on the last);
 *                     writes the gradients without the normalisation row and the
 *                     per-head dots (bh + bhkv floats, zeroed here); consumes qg_states
 *                     (their contents are undefined afterwards)
 *   shard_norm_fixup  after dots were summed over shards: corrects the max-norm row
 *                     on the shard that owns it
 * Unmasked shards (mask = 0): every token reads the totals of ALL shards, so the caller
 * sum-reduces kv_total and qg_total over the shards (an all-reduce) and passes
 *   shard_forward     s_base    = key/value total of all shards (kv_states may be NULL)
 *   shard_backward    kv_states = key/value total of all shards,
 *                     r_base    = query/gradient total of all shards (qg_states may be NULL)
 * Buffers: kv_states/qg_states fastmax_b200_moment_state_bytes, totals and bases
 * fastmax_b200_moment_total_bytes (float32), workspaces by the *_workspace_bytes
 * queries, delta bh*nq floats. */
size_t fastmax_b200_moment_state_bytes(const fastmax_problem* prob);
size_t fastmax_b200_moment_total_bytes(const fastmax_problem* prob);
size_t fastmax_b200_shard_forward_workspace_bytes(const fastmax_problem* prob);
size_t fastmax_b200_shard_backward_workspace_bytes(const fastmax_problem* prob);
int fastmax_b200_shard_rowmax(const fastmax_problem* prob, const void* q, const void* k,
                              int32_t row_offset, void* stats, void* stream);
int fastmax_b200_shard_kv_state(const fastmax_problem* prob, const void* k, const void* v,
                                float* kv_states, float* kv_total, void* stream);
int fastmax_b200_shard_forward(const fastmax_problem* prob, const void* q, const void* k,
                               const void* v, const void* stats, float* kv_states,
                               const float* s_base, void* out, float* den, void* workspace,
                               size_t workspace_bytes, void* stream);
int fastmax_b200_shard_qg_state(const fastmax_problem* prob, const void* q, const void* out,
                                const float* den, const void* grad_out, float* delta,
                                float* qg_states, float* qg_total, void* workspace,
                                size_t workspace_bytes, void* stream);
int fastmax_b200_shard_backward(const fastmax_problem* prob, const void* q, const void* k,
                                const void* v, const void* out, const float* den,
                                const void* stats, const void* grad_out, const float* delta,
                                const float* kv_states, float* qg_states, const float* r_base,
                                float* dots, void* grad_q, void* grad_k, void* grad_v,
                                int32_t dq_far_done, void* workspace, size_t workspace_bytes, void* stream);
/* Optional split of shard_backward for causal shards, so that the exchange of the query/gradient
 * totals can overlap compute: shard_dq_far evaluates the part of grad_q that reads the key/value
 * prefixes -- it needs nothing from later shards -- into the workspace.  Call it after
 * shard_qg_state on the same workspace (whose gs / dvec it uses) while the exchange is in flight,
 * then pass dq_far_done = 1 to shard_backward, again with the same, untouched workspace. */
int fastmax_b200_shard_dq_far(const fastmax_problem* prob, const void* q, const float* den, const void* stats,
                              const void* grad_out, const float* delta, const float* kv_states,
                              void* workspace, size_t workspace_bytes, void* stream);
/* After an all-gather of every shard's total into gathered (world, floats_per_shard): out = sum of
 * the totals of the shards before `rank` (after it when reverse != 0).  With no such shard out is
 * zero-filled; pass NULL as s_base / r_base instead of calling this. */
int fastmax_b200_shard_sum_totals(const float* gathered, int32_t world, int32_t rank, int32_t reverse,
                                  size_t floats_per_shard, float* out, void* stream);
int fastmax_b200_shard_norm_fixup(const fastmax_problem* prob, const void* q, const void* k,
                                  const void* stats, const float* dots, int32_t row_offset,
                                  void* grad_q, void* grad_k, void* stream);

/* Backward pass for callers that cannot supply or allocate scratch memory.  It
 * has no counterpart in the reference, whose backward_cuda allocates its outputs
 * and temporaries itself with torch::zeros (fastmax_cuda_backward.cu:951-959).
 *
 * Meant for programs in which device memory is not the library's to take: a
 * server or framework that has claimed the whole GPU for its own arena, or a
 * latency-critical loop that must not hit the device-wide synchronisation inside
 * cudaMalloc/cudaFree.  The scratch is a fixed array inside the library image,
 * fastmax_b200_static_scratch_bytes() bytes (8 MiB) on every GPU that loads the
 * library, held until the process exits.  The call allocates nothing, by any
 * route, and takes the same tensors as fastmax_b200_backward minus the workspace.
 *
 *  - Runs the CUDA-core score family (prob->impl AUTO or DENSE_FFMA), any
 *    supported dtype and head dimension.
 *  - Problems whose scratch does not fit -- roughly bh*nq above 2 million --
 *    return FASTMAX_E_WORKSPACE; use fastmax_b200_backward for those.
 *  - The first call on each GPU looks up the array's device address (with that
 *    GPU current); under CUDA's lazy module loading that is also when the driver
 *    reserves the 8 MiB there.  Make that first call before starting any stream
 *    capture and before your own allocator takes what is left of the GPU: a call
 *    with an empty problem (bh == 0, every pointer NULL) does just this set-up.
 *  - All calls on a GPU share the one array: calls that overlap on the GPU race,
 *    so keep them on one stream or order them yourself.  Nothing is assumed
 *    about the array's contents between calls; what must start at zero is
 *    cleared on the stream at the start of each call. */
size_t fastmax_b200_static_scratch_bytes(void);
int fastmax_b200_backward_static(const fastmax_problem* prob,
                                 const void* q, const void* k, const void* v,
                                 const void* out, const float* den, const void* stats,
                                 const void* grad_out,
                                 void* grad_q, void* grad_k, void* grad_v,
                                 void* stream);

/* ---- the transformer call site around the attention --------------------------
 * Replaces the elementwise passes of the reference's caller, model.py:472-499
 * and 557-603: the permute / split / expand of the packed projection, apply_rope
 * (model.py:812-825), the three `.contiguous()` copies (model.py:572-574) and the
 * transpose of the result (model.py:603).  Arrays are contiguous, 16-byte aligned,
 * of type `dtype`; the head size d is a multiple of 8; cos_table and sin_table are
 * float32 (n, rope_n) (NULL when rope_n == 0); rope_n is a multiple of 8, at most d.
 *
 * qkv_split_rope: qkv (batch, n, groups, q_per_group + 2, d) ->
 *   q (batch * groups * q_per_group, n, d), k and v (batch * groups, n, d), with the
 *   first rope_n features of q and k rotated:  y = x * cos + (-x2, x1) * sin, x1 / x2
 *   the two halves of those features.  k and v are NOT expanded to the query head
 *   count: pass bh = batch * groups * q_per_group and bhkv = batch * groups to the
 *   attention calls.
 * qkv_merge_rope_grad: the gradient of qkv from grad_q, grad_k, grad_v (same shapes),
 *   i.e. the transposed rotation and the inverse placement.
 * swap_middle_axes: src (batch, x, y, d) -> dst (batch, y, x, d); src != dst.
 * scale_by_noise: y[i] = x[i] * (1 + dropout * noise[i]) over `count` elements, the
 *   reference's output dropout (fastmax_cuda_forward.cu:271-280, applied at :396-399);
 *   y may be x. */
int fastmax_b200_qkv_split_rope(const void* qkv, const float* cos_table, const float* sin_table,
                                void* q, void* k, void* v,
                                long long batch, long long n, int groups, int q_per_group, int d,
                                int rope_n, int dtype, void* stream);
int fastmax_b200_qkv_merge_rope_grad(const void* grad_q, const void* grad_k, const void* grad_v,
                                     const float* cos_table, const float* sin_table, void* grad_qkv,
                                     long long batch, long long n, int groups, int q_per_group, int d,
                                     int rope_n, int dtype, void* stream);
int fastmax_b200_swap_middle_axes(const void* src, void* dst, long long batch, long long x, long long y,
                                  int d, int dtype, void* stream);
int fastmax_b200_scale_by_noise(const void* x, const void* noise, void* y, float dropout, size_t count,
                                int dtype, void* stream);
/* The same output dropout on the packed forward result of forward_packed: o_packed is
 * (rows, d + 1) float32, noise (rows, d) of type noise_dtype; channels 0..d-1 of every row
 * are scaled in place, the denominator channel is not (reference apply_dropout,
 * fastmax_cuda_forward.cu:271-280, which runs over the first d channels of o). */
int fastmax_b200_scale_packed_by_noise(float* o_packed, const void* noise, float dropout, long long rows,
                                       int d, int noise_dtype, void* stream);

/* ---- decoding against a persistent moment state --------------------------------
 * Replaces the key/value cache of the reference's model (model.py:501-504, 828-852)
 * for causal Fastmax attention: instead of all earlier keys and values, a fixed-size
 * fp32 state per key/value head (decode_state_bytes: 1 + d (+ d*d when p = 2) rows
 * of d + 1 floats and a small header) is updated by each new token and read by its
 * query, so a step costs the same at every length.  Only dtype, bh, bhkv, d, p,
 * normalize, a0, a1, a2 and lim of the problem are used; d is 32, 64 or 128.
 *
 * decode_append: adds n_new tokens, k and v (bhkv, n_new, d), to the state (prompt
 *   processing).  The state must be zero-filled (cudaMemsetAsync) before its first use.
 * decode_step: adds one token, k and v (bhkv, 1, d), then evaluates the attention row
 *   of q (bh, 1, d) over every token added so far into out (bh, 1, d).  The result
 *   equals fastmax_b200_forward with nq = 1, nk = the number of tokens, mask = 1:
 *   keys scaled by lim / max |k| over all of them, the query by lim / |q|.
 *   scratch: decode_scratch_bytes, any contents. */
size_t fastmax_b200_decode_state_bytes(const fastmax_problem* prob);
size_t fastmax_b200_decode_scratch_bytes(const fastmax_problem* prob);
int fastmax_b200_decode_append(const fastmax_problem* prob, const void* k, const void* v, long long n_new,
                               void* state, void* stream);
int fastmax_b200_decode_step(const fastmax_problem* prob, const void* q, const void* k, const void* v,
                             void* state, void* scratch, void* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FASTMAX_B200_H */
