/*
 * fields_read.h - C ABI of the B200 (sm_100a) Field-recurrence library.
 *
 * The library replaces one operator of Multisymboliccore/fields-lm: the fused
 * Field read, `fused_field_read(raw, transition_r, transition_i, gamma,
 * block_c, chunk_t)` (src/fields_official/reference/
 * field_only_v4_chunked_triton_wiki100.py:1108-1123), forward and backward.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer to memory owned by the caller; the
 *     library allocates nothing, frees nothing and keeps no state between calls
 *     (one exception: the built-in scratch of fields_read_forward_noalloc);
 *   - all tensors are contiguous float32 with the reference's layouts, channel
 *     fastest:  raw [B, L, 3C] = z_r | z_i | z_v,   read [B, L, 4C] =
 *     Re s | Im s | Re d | Im d,   states [B, 2C] = Re s | Im s;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it and the
 *     call returns without synchronising;
 *   - the return value is a status code (0 = success); nothing aborts, traps or
 *     asserts on the device;
 *   - `workspace` must hold at least fields_read_workspace_bytes(...) bytes and
 *     be 256-byte aligned; its contents are scratch.
 *   - 128-bit accesses are used when C is a multiple of 4 and every tensor
 *     pointer is 16-byte aligned; otherwise a scalar path with the same arithmetic
 *     (equal up to the last bit or two) runs.
 */
#ifndef FIELDS_READ_H_
#define FIELDS_READ_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum fields_status {
    FIELDS_OK = 0,
    FIELDS_ERR_ARGUMENT = 1,  /* null pointer or negative / zero extent */
    FIELDS_ERR_WORKSPACE = 2, /* workspace missing, too small or misaligned */
    FIELDS_ERR_LAUNCH = 3,    /* the CUDA runtime refused a launch (see fields_last_cuda_error) */
    FIELDS_ERR_TIMEOUT = 4,   /* a bounded device-side wait ran out */
    FIELDS_ERR_UNSUPPORTED = 5,
    FIELDS_ERR_SCRATCH_LIMIT = 6 /* fields_read_forward_noalloc: extents exceed the built-in scratch */
};

/* which pass a workspace is sized for */
enum fields_pass {
    FIELDS_PASS_FORWARD = 0,
    FIELDS_PASS_BACKWARD = 1
};

/* Human-readable text for a status code. Never null. */
const char *fields_status_string(int status);

/* Library version as major * 10000 + minor * 100 + patch. */
int fields_read_version(void);

/* Bytes of scratch the given pass needs for these extents (0 for empty inputs). */
size_t fields_read_workspace_bytes(int B, int L, int C, int pass);

/*
 * Forward of the fused Field read. Replaces _ChunkedFieldReadFunction.forward
 * (field_only_v4_chunked_triton_wiki100.py:912-1018): gates, independent
 * vacancy, complex diagonal recurrence and displaced readout.
 *   raw        [B, L, 3C]
 *   tr, ti, gamma [C]      lambda = tr + i ti
 *   state_in   [B, 2C] or NULL  (NULL = zero state, the reference's contract,
 *                                 same file :535-536)
 *   read       [B, L, 4C]  output
 *   state_out  [B, 2C] or NULL  state after the last step (extension)
 */
int fields_read_forward(const float *raw, const float *tr, const float *ti,
                        const float *gamma, const float *state_in, float *read,
                        float *state_out, void *workspace, size_t workspace_bytes,
                        int B, int L, int C, void *stream);

/*
 * Backward of the fused Field read. Replaces _ChunkedFieldReadFunction.backward
 * (field_only_v4_chunked_triton_wiki100.py:1020-1105) including the three
 * sums over (batch, chunk) that follow it (:1098-1105).
 *   read            saved forward output [B, L, 4C] (source of s_{t-1})
 *   grad_read       [B, L, 4C]
 *   grad_state_out  [B, 2C] or NULL  gradient flowing into state_out (extension)
 *   grad_raw        [B, L, 3C] output
 *   grad_tr, grad_ti, grad_gamma  [C] outputs (overwritten, not accumulated)
 *   grad_state_in   [B, 2C] or NULL  output (extension)
 */
int fields_read_backward(const float *raw, const float *tr, const float *ti,
                         const float *gamma, const float *state_in,
                         const float *read, const float *grad_read,
                         const float *grad_state_out, float *grad_raw,
                         float *grad_tr, float *grad_ti, float *grad_gamma,
                         float *grad_state_in, void *workspace,
                         size_t workspace_bytes, int B, int L, int C, void *stream);

/*
 * Backward pass without the saved forward output (no counterpart in the reference, whose
 * backward reads s_{t-1} of every step from the saved `read`,
 * field_only_v4_chunked_triton_wiki100.py:1008-1014 and :840-853).
 *
 * The kernel re-runs the state recurrence inside its first sweep and needs only the state at
 * every eighth step: states [B, fields_read_state_rows(L), 2C] fp32, row j = Re s | Im s
 * after step 8 (j + 1) - 1, i.e. read[:, 8 (j + 1) - 1, 0:2C]. A caller keeps those rows
 * (1/16 of `read`) and may free `read` itself. Other arguments, workspace and results as
 * fields_read_backward. Needs C % 4 == 0 and 16-byte aligned tensors
 * (FIELDS_ERR_UNSUPPORTED otherwise); states may be NULL when L <= 8.
 */
int fields_read_state_rows(int L);
int fields_read_backward_from_states(const float *raw, const float *tr, const float *ti,
                                     const float *gamma, const float *state_in,
                                     const float *states, const float *grad_read,
                                     const float *grad_state_out, float *grad_raw,
                                     float *grad_tr, float *grad_ti, float *grad_gamma,
                                     float *grad_state_in, void *workspace,
                                     size_t workspace_bytes, int B, int L, int C, void *stream);

/*
 * bfloat16 I/O twins of the two passes: raw, read, grad_read and grad_raw are bfloat16 (same
 * layouts, half the bytes); parameters, states, parameter gradients and all arithmetic stay
 * fp32. They serve a mixer that keeps the write projection's bf16 output instead of widening
 * it as field_only_v4_chunked_triton_wiki100.py:1168 does (`.float()`), which is where the
 * reference pays for "bf16 activations" with fp32 traffic. Need C % 4 == 0 and 8-byte aligned
 * tensors (FIELDS_ERR_UNSUPPORTED otherwise). Same workspace sizes as the fp32 passes.
 */
int fields_read_forward_bf16(const void *raw, const float *tr, const float *ti,
                             const float *gamma, const float *state_in, void *read,
                             float *state_out, void *workspace, size_t workspace_bytes,
                             int B, int L, int C, void *stream);
/*
 * fields_read_forward_bf16 that also returns what the RMS norm after the recurrence
 * (read_norm, field_only_v4_chunked_triton_wiki100.py:1177 and :300-309) needs from `read`:
 * sumsq [B, L, G] fp32, G = ceil(C / 128), the sum over the four output planes of the squares
 * of the 128 channels of group g at token t, taken from the fp32 values before they are
 * rounded to bfloat16. mean(read^2) over the 4C features of a token is the sum over g divided
 * by 4C, so the norm's reduction pass over `read` is not needed; a caller can apply
 * rsqrt(mean + eps) after the output projection instead of before it. B, L > 0.
 */
int fields_read_forward_bf16_stats(const void *raw, const float *tr, const float *ti,
                                   const float *gamma, const float *state_in, void *read,
                                   float *sumsq, float *state_out, void *workspace,
                                   size_t workspace_bytes, int B, int L, int C, void *stream);
int fields_read_backward_bf16(const void *raw, const float *tr, const float *ti,
                              const float *gamma, const float *state_in, const void *read,
                              const void *grad_read, const float *grad_state_out,
                              void *grad_raw, float *grad_tr, float *grad_ti,
                              float *grad_gamma, float *grad_state_in, void *workspace,
                              size_t workspace_bytes, int B, int L, int C, void *stream);

/*
 * EXPERIMENT, not the production path: the forward of fields_read_forward_bf16 with the
 * intra-chunk part of the recurrence computed as a dense contraction on the tensor cores
 * (tcgen05.mma, bf16 operands from shared memory, fp32 accumulator in tensor memory). No
 * counterpart in the reference, whose kernels use no tensor-core instruction
 * (field_only_v4_chunked_triton_wiki100.py:443-909). Inside sub-chunks of 16 steps the state is
 * s_t = P_t (s_in + sum_{j<=t} b_j / P_j) with P the prefix product of the per-step complex
 * decays; the sum over j is a product with a lower-triangular all-ones matrix shared by every
 * channel. The quotients are rounded to bfloat16, so the result meets the bfloat16 tolerance
 * (2e-2 relative) only. One CTA walks a (batch row, 32 channels) chain in tiles of 128 steps;
 * its elementwise work equals the scan's, so it is no faster - it exists to put a measured
 * tensor-pipe utilisation beside the scan kernels. Same tensors as fields_read_forward_bf16;
 * no workspace. error_word: a device word the caller zeroed, set to 1 if a bounded wait for the
 * tensor cores ran out. C % 4 == 0, 8-byte aligned raw / read (FIELDS_ERR_UNSUPPORTED otherwise).
 */
int fields_read_forward_bf16_tensor(const void *raw, const float *tr, const float *ti,
                                    const float *gamma, const float *state_in, void *read,
                                    float *state_out, unsigned *error_word, int B, int L, int C,
                                    void *stream);

/*
 * Sequence sharding (no counterpart in the reference, which runs a sequence on one GPU;
 * the arithmetic is the chunk-summary composition of
 * field_only_v4_chunked_triton_wiki100.py:503-509 and :539-550 applied to a whole span).
 *
 * fields_read_span_summary: the affine map  s_out = A s_in + Bv  of a span of L steps per
 * (batch, channel), as summary [B, 4, C] = Re A | Im A | Re Bv | Im Bv. Workspace as for
 * the forward pass.
 *
 * fields_read_fold_summaries: given the summaries of all P spans, [P, B, 4, C] in span
 * order, and the state before the first span (state0 [B, 2C] or NULL = zero), writes the
 * state entering span `rank` into state [B, 2C]. That state is the state_in of
 * fields_read_forward for that span.
 */
int fields_read_span_summary(const float *raw, const float *tr, const float *ti,
                             const float *gamma, float *summary, void *workspace,
                             size_t workspace_bytes, int B, int L, int C, void *stream);
int fields_read_fold_summaries(const float *summaries, const float *state0, float *state,
                               int rank, int P, int B, int C, void *stream);

/*
 * The same for the backward pass of a sharded sequence (the reverse-order composition of
 * field_only_v4_chunked_triton_wiki100.py:655-705 and :725-745 applied to a whole span).
 *
 * fields_read_span_summary_backward: the dual map  carry_in = P carry_out + Q  of a span per
 * (batch, channel): carry_out is the gradient carry arriving from the steps after the span,
 * carry_in the one leaving towards the steps before it. summary [B, 4, C] = Re P | Im P |
 * Re Q | Im Q. Reads z_v of raw and grad_read. Workspace as for the backward pass.
 *
 * fields_read_fold_summaries_backward: given the dual summaries of all P spans, [P, B, 4, C]
 * in span order, and the carry after the last span (carry_end [B, 2C] or NULL = zero), writes
 * the carry arriving at the end of span `rank` into carry [B, 2C] (the spans after `rank` are
 * applied last first). That carry is the grad_state_out of fields_read_backward for the span;
 * its state_in is the state fields_read_fold_summaries gave the forward pass. The three
 * parameter gradients of the spans add up (an all-reduce the caller owns).
 */
int fields_read_span_summary_backward(const float *raw, const float *tr, const float *ti,
                                      const float *grad_read, float *summary, void *workspace,
                                      size_t workspace_bytes, int B, int L, int C, void *stream);
int fields_read_fold_summaries_backward(const float *summaries, const float *carry_end,
                                        float *carry, int rank, int P, int B, int C,
                                        void *stream);

/*
 * One recurrent step for incremental decoding (no counterpart in the reference, whose
 * inference is always a full-sequence pass; the arithmetic is one iteration of
 * field_only_v4_chunked_triton_wiki100.py:599-622).
 *   raw    [B, 3C]  the new token's z_r | z_i | z_v for every sequence
 *   state  [B, 2C]  fp32, read and overwritten in place
 *   read   [B, 4C]  output row
 * fields_read_step_bf16 takes raw and writes read as bfloat16; the state stays fp32.
 */
int fields_read_step(const float *raw, const float *tr, const float *ti, const float *gamma,
                     float *state, float *read, int B, int C, void *stream);
int fields_read_step_bf16(const void *raw, const float *tr, const float *ti, const float *gamma,
                          float *state, void *read, int B, int C, void *stream);

/*
 * Real-valued first-order scan  s_t = a_t s_{t-1} + drive_t  over [B, L, C] fp32: the second call
 * site of the reference's scan primitive, hierarchical_scan(a, drive, block=32)
 * (field_only_v4_chunked_triton_wiki100.py:347-391) as the softpatch mixer calls it on a rank-64
 * state (official_source/field_hybrid_speed_optimization_v6.py:333-335).
 *   a            element (b, t, c) at a[b * a_batch + t * a_step + c * a_chan], strides in floats,
 *                a_chan 0 or 1: the reference passes one decay per token expanded over the channels
 *                (a_batch = L, a_step = 1, a_chan = 0); a dense tensor is (L * C, C, 1)
 *   drive        [B, L, C]
 *   state_in     [B, C] or NULL (zero, the reference's contract)
 *   states       [B, L, C] out: s_t for every step
 *   state_out    [B, C] or NULL
 *   workspace    fields_scan_workspace_bytes(B, L, C) bytes, 16-byte aligned
 * Backward: grad_a is written densely [B, L, C] also for a broadcast `a` (the caller sums over
 * the broadcast dimension, as autograd does for an expanded tensor); states is the forward output.
 * Three launches each way (chunk maps, carries, states); results are bitwise reproducible.
 */
size_t fields_scan_workspace_bytes(int B, int L, int C);
int fields_scan_forward(const float *a, long long a_batch, long long a_step, int a_chan,
                        const float *drive, const float *state_in, float *states,
                        float *state_out, void *workspace, size_t workspace_bytes, int B, int L,
                        int C, void *stream);
int fields_scan_backward(const float *a, long long a_batch, long long a_step, int a_chan,
                         const float *states, const float *state_in, const float *grad_states,
                         const float *grad_state_out, float *grad_a, float *grad_drive,
                         float *grad_state_in, void *workspace, size_t workspace_bytes, int B,
                         int L, int C, void *stream);

/*
 * The same exchange without a collective library: span summaries travel between the GPUs of a
 * node through peer-writable memory (NVLink / NVSwitch). No counterpart in the reference.
 *
 * Every rank owns a mailbox of fields_read_mailbox_bytes(P, B, C) bytes, zeroed once when it is
 * created, in memory its peers can write (peer access, IPC or symmetric memory); mailboxes[r] is
 * rank r's mailbox as seen from the calling GPU (a HOST array of P device pointers, P <= 16).
 * (The size includes a board behind the slots that only the owner's own kernels use.)
 *
 * fields_read_span_summary_put: computes this rank's span summary and stores it, tagged with
 * `epoch`, into its slot of every rank's mailbox (plain 8-byte peer stores; no TMA, no
 * multicast). Also writes the summary to `summary` [B, 4, C] if that is not NULL.
 *
 * fields_read_fold_mailbox: waits, with a bound, until the calling rank's own mailbox holds the
 * summaries of all P ranks for `epoch`, then writes the state entering the rank's span to
 * `state` [B, 2C] (state0 as in fields_read_fold_summaries). If a summary does not arrive in
 * time it sets *error_word (a device word the caller zeroed) to 1 and fills `state` with NaN.
 * `max_polls` bounds the wait for the whole call (a poll is well under a microsecond; 0 = the
 * library's default of 2^21, about a second of skew between the ranks): once one slot has run
 * out, the slots after it are not waited for.
 *
 * `epoch` is a per-call counter kept by the caller: the same on all ranks, never 0, increased
 * by one for every exchange on a mailbox. Two parities alternate inside the mailbox and every
 * rank waits for all ranks, so nothing is ever cleared and no rank can run more than one
 * exchange ahead. The epoch is a kernel argument: a captured CUDA graph would repeat it, so
 * these two calls must not be replayed from a graph.
 */
size_t fields_read_mailbox_bytes(int P, int B, int C);
int fields_read_span_summary_put(const float *raw, const float *tr, const float *ti,
                                 const float *gamma, void *const *mailboxes, float *summary,
                                 int rank, int P, unsigned epoch, void *workspace,
                                 size_t workspace_bytes, int B, int L, int C, void *stream);
int fields_read_fold_mailbox(const void *mailbox, const float *state0, float *state,
                             unsigned *error_word, int rank, int P, unsigned epoch,
                             unsigned max_polls, int B, int C, void *stream);

/*
 * The sequence-sharded forward of one rank in ONE launch (no counterpart in the reference, which
 * runs a sequence on one GPU; its serial chunk-carry kernel,
 * field_only_v4_chunked_triton_wiki100.py:519-550, is what the in-kernel scan replaces).
 *
 * Does what fields_read_span_summary_put + fields_read_fold_mailbox + fields_read_forward do,
 * with one read of the span from HBM when its raw fits the L2 cache: persistent blocks sweep
 * the span once to compose its map, the last block of every (batch row, 128 channels) chain
 * scans the maps and stores the span's map into every rank's mailbox, every block waits (with
 * a bound) for the P summaries of `epoch`, folds the earlier ranks onto state0 and sweeps its
 * part of the span again, now from L2, writing `read`.
 *
 *   raw [B, L, 3C], read [B, L, 4C]   this rank's span
 *   state0    [B, 2C] or NULL   state before the FIRST span (the same on every rank)
 *   state_out [B, 2C] or NULL   state after this rank's span
 *   summary   [B, 4, C] or NULL this span's own map, as fields_read_span_summary gives it
 *   mailboxes, rank, P, epoch   as fields_read_span_summary_put; each mailbox 256-byte aligned,
 *                               fields_read_mailbox_bytes(P, B, C) bytes, zeroed once
 *   error_word  device word the caller zeroed; set to 1 if a wait ran out (`read` and
 *               state_out then hold NaN from that point on)
 *   max_polls   bound of every wait in polls (a poll is well under a microsecond);
 *               0 = the library's default of 2^21, about a second
 *
 * No workspace: the kernel keeps its run maps on a board behind the slots of the rank's own
 * mailbox (part of fields_read_mailbox_bytes), tagged with the epoch like the slots, so
 * nothing is ever cleared. The launch is cooperative: all blocks are resident together,
 * because they wait for one another and for the peers. With P = 1 nothing is exchanged (the
 * mailbox only lends its board). Needs C % 4 == 0 and 16-byte aligned tensors
 * (FIELDS_ERR_UNSUPPORTED otherwise). Peer memory is written with plain 8-byte stores only.
 *
 * epoch > 0: the caller's per-call counter, as for the other mailbox calls; such a call must
 * not be replayed from a captured CUDA graph (the graph would repeat the epoch).
 * epoch == 0: the epoch lives on the rank's board; the kernel reads it when it starts and its
 * last block advances it, so the call carries no per-call value and a captured graph can
 * replay it. Every rank must then make the same sequence of calls on these mailboxes, and the
 * mailboxes must not be shared with calls that pass their own epochs.
 */
int fields_read_forward_sharded(const float *raw, const float *tr, const float *ti,
                                const float *gamma, const float *state0, float *read,
                                float *state_out, float *summary, void *const *mailboxes,
                                unsigned *error_word, int rank, int P, unsigned epoch,
                                unsigned max_polls, int B, int L, int C, void *stream);

/*
 * Sum of a short fp32 vector over the ranks through the same mailboxes, in one launch and without
 * a collective library: the 3 C parameter-gradient sums of a sequence-sharded backward pass (and
 * the ranks' status words beside them). No counterpart in the reference, which sums its
 * partials on one GPU (field_only_v4_chunked_triton_wiki100.py:1098-1105).
 *   values  [n] this rank's addends, out [n] the sum over the ranks, n <= 3 C + 64
 *   mailboxes, rank, P, epoch, max_polls   as for fields_read_fold_mailbox; the call takes the
 *            next epoch of the shared sequence; B and C are those the mailboxes were sized with
 * Every rank stores its values, tagged with the epoch, into every rank's reduction region
 * (part of fields_read_mailbox_bytes, behind the board) with plain 8-byte peer stores, waits
 * with a bound until its own region holds all P contributions and adds them in rank order:
 * every rank gets the same bits. A contribution that never arrives sets the error word and
 * leaves NaN in out.
 */
int fields_read_sum_over_ranks(const float *values, float *out, int n, void *const *mailboxes,
                               unsigned *error_word, int rank, int P, unsigned epoch,
                               unsigned max_polls, int B, int C, void *stream);

/*
 * The backward exchange through the same mailboxes (they and the epoch sequence are shared
 * with the forward exchange: every exchange, in either direction, takes the next epoch).
 * fields_read_span_summary_backward_put stores the span's dual summary (see
 * fields_read_span_summary_backward) into every rank's mailbox;
 * fields_read_fold_mailbox_backward waits, with the same bound, for all P dual summaries of
 * `epoch` and writes the gradient carry arriving at the end of the rank's span (carry_end as
 * in fields_read_fold_summaries_backward).
 */
int fields_read_span_summary_backward_put(const float *raw, const float *tr, const float *ti,
                                          const float *grad_read, void *const *mailboxes,
                                          float *summary, int rank, int P, unsigned epoch,
                                          void *workspace, size_t workspace_bytes, int B, int L,
                                          int C, void *stream);
int fields_read_fold_mailbox_backward(const void *mailbox, const float *carry_end, float *carry,
                                      unsigned *error_word, int rank, int P, unsigned epoch,
                                      unsigned max_polls, int B, int C, void *stream);

/* Text of the last CUDA runtime error seen by the calling thread inside this library. */
const char *fields_last_cuda_error(void);

/*
 * Reads back the error word that the single-pass kernels keep in the workspace they
 * were given, after waiting for `stream`. Returns FIELDS_OK, or FIELDS_ERR_TIMEOUT if a
 * block gave up a bounded wait for an earlier tile (its outputs then hold NaN). Only
 * meaningful directly after fields_read_forward / fields_read_backward on that
 * workspace. The reference has no counterpart (its kernels never wait on each other).
 */
int fields_read_device_status(const void *workspace, void *stream);

/*
 * Self-test of the bounded device-side wait: runs one block that waits for a publication
 * nothing ever makes, with the wait limited to max_polls polls, waits for the stream and
 * returns the resulting status - FIELDS_ERR_TIMEOUT when the wait gave up cleanly, as it
 * must. Nothing hangs, traps or faults; the context stays usable. workspace: at least
 * 8 KB, 256-byte aligned. (No counterpart in the reference.)
 */
int fields_read_selftest_wait(void *workspace, size_t workspace_bytes, unsigned max_polls,
                              void *stream);

/*
 * Forward of the fused Field read for callers that have no memory to give.
 * (No counterpart in the reference, whose operator allocates its work buffers
 * with torch.empty on every call.)
 *
 * Some hosts of this library cannot hand over a workspace: an operator running
 * inside an inference runtime's execution hook, a plug-in of a serving engine
 * whose memory plan was fixed at start-up, or a real-time loop that must not
 * stall - cudaMalloc synchronises the device and may fail under a full pool,
 * and such callers often have no allocator they are allowed to call at that
 * point. For them the library carries its own scratch: a fixed
 * FIELDS_STATIC_SCRATCH_BYTES buffer in device memory that every GPU which
 * loads the library holds until the process exits. This entry point runs the
 * same kernels as fields_read_forward on that buffer and calls no cudaMalloc,
 * cudaFree or other allocating routine. Inputs and outputs are still the
 * caller's, with the meanings given at fields_read_forward.
 *
 *   - Limit: extents whose fields_read_workspace_bytes(B, L, C,
 *     FIELDS_PASS_FORWARD) exceeds FIELDS_STATIC_SCRATCH_BYTES are refused with
 *     FIELDS_ERR_SCRATCH_LIMIT and nothing is launched. 16 MiB covers the
 *     training shape, 8 x 2,048 tokens at C = 512 (12 MiB), and 1 x 8,192.
 *   - The first call on each device looks the buffer's device address up
 *     (once, cached, with that device current); make that first call before
 *     any stream capture begins.
 *   - All calls on a device share the one buffer, which keeps whatever the last
 *     call left in it. The kernels overwrite what they later read, so no
 *     clearing is needed, but two calls that overlap on the GPU (different
 *     streams without an ordering between them, or host threads launching at
 *     the same time) race on it: serialise them.
 */
#define FIELDS_STATIC_SCRATCH_BYTES ((size_t)16 << 20)
size_t fields_read_static_scratch_bytes(void);
int fields_read_forward_noalloc(const float *raw, const float *tr, const float *ti,
                                const float *gamma, const float *state_in,
                                float *read, float *state_out, int B, int L, int C,
                                void *stream);

/*
 * Readout epilogue of the Field mixer with the RMS norm moved behind the output projection
 * (the reference computes, field_only_v4_chunked_triton_wiki100.py:1177-1179,
 *   y = x + out_proj(read_norm(read)) * sigmoid(gate_proj(x)) ).
 * Given acc = read @ (W diag(w))^T and gate = gate_proj(x), both [N, D] bfloat16, x [N, D] and
 * bias [D] fp32, and sumsq [N] = the sum of squares of each token's `features` read values
 * (fields_read_forward_bf16_stats, summed over the groups):
 *   y = x + (acc * rsqrt(sumsq / features + eps) + bias) * sigmoid(gate + gate_bias)   [N, D]
 * in one pass (gate_bias [D] may be NULL: then `gate` already contains it); the backward entry
 * returns, in one pass, grad_acc and grad_gate (bfloat16), grad_sumsq [N], and the gradients of
 * bias and, if given, gate_bias as fields_mixer_epilogue_bias_rows(N) partial rows [rows, D]
 * each for the caller to add up (grad_x is grad_y itself). D % 4 == 0, D <= 4096 for the
 * backward, 16-byte aligned fp32 and 8-byte aligned bfloat16 tensors
 * (FIELDS_ERR_UNSUPPORTED otherwise).
 *
 * fields_read_norm_grad_combine: the gradient that fields_read_backward_bf16 must receive when
 * sumsq of fields_read_forward_bf16_stats has a gradient of its own:
 *   total = grad_read + 2 * grad_sumsq[token] * read        ([N, F] bfloat16, F = 4C, F % 4 == 0)
 * in one pass; grad_read may be NULL.
 */
int fields_read_norm_grad_combine(const void *grad_read, const void *read,
                                  const float *grad_sumsq, void *total, long long N, int F,
                                  void *stream);
size_t fields_mixer_epilogue_bias_rows(long long N);
int fields_mixer_epilogue_forward(const float *x, const void *acc, const void *gate,
                                  const float *sumsq, const float *bias, const float *gate_bias,
                                  float *y, float eps, int features, long long N, int D,
                                  void *stream);
int fields_mixer_epilogue_backward(const float *grad_y, const void *acc, const void *gate,
                                   const float *sumsq, const float *bias, const float *gate_bias,
                                   void *grad_acc, void *grad_gate, float *grad_sumsq,
                                   float *grad_bias_rows, float *grad_gate_bias_rows, float eps,
                                   int features, long long N, int D, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* FIELDS_READ_H_ */
