/*
 * molla_sample.h - C ABI of the B200 token-sampling library.
 *
 * The library replaces one stage of the tamnd/molla inference server: the step
 * that turns a [batch x vocab] block of fp32 logits into next-token ids. In the
 * reference that stage is the host-side `Sampler` of
 * src/molla/engine/sample.mojo, called once per answered row from the decode
 * loop (src/molla/engine/batch.mojo:503-519) after the whole logit block has
 * been copied device -> host. Here the logits are consumed where the forward
 * pass left them, on the device, and only the token ids (and, when asked for,
 * logprobs) come back.
 *
 * Conventions (they follow how molla calls C, src/molla/tls/openssl.mojo:53-139
 * and src/molla/sys/clock.mojo:37-58): plain `extern "C"` functions, scalars and
 * raw pointers only, per-row parameters as parallel arrays (no struct layout to
 * agree on), no callbacks, no C++ types, nothing thrown across the boundary.
 * Every function that can fail returns an int32 status: 0 is success, negative
 * is an argument error found before anything was launched, positive is an error
 * the CUDA runtime or the device reported. `molla_sample_last_error()` gives
 * the text. Nothing here creates a CUDA context or a stream: work is enqueued
 * on the stream the caller passes (0 = the default stream) in the caller's
 * current context, and is asynchronous unless stated otherwise.
 *
 * There is no CPU fallback. Built for sm_100a only.
 */
#ifndef MOLLA_SAMPLE_H
#define MOLLA_SAMPLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOLLA_SAMPLE_ABI_VERSION 1

/* status codes */
#define MOLLA_OK 0
#define MOLLA_ERR_ARGUMENT (-1)   /* null pointer, negative size, bad alignment */
#define MOLLA_ERR_VOCAB (-2)      /* vocabulary too wide for the on-chip row buffer */
#define MOLLA_ERR_WORKSPACE (-3)  /* workspace missing or too small */
#define MOLLA_ERR_CONFIG (-4)     /* a sampler setting outside SamplerConfig.check's rules */
#define MOLLA_ERR_CUDA 1          /* a CUDA runtime call failed */
#define MOLLA_ERR_DEVICE 2        /* the kernel reported an error (see row status) */

/* Per-row status bits written to `d_row_status` (0 = clean row). The TIE bits
 * are not errors: they mark rows whose answer in the reference depends on the
 * unstable order its heapsort leaves equal probabilities in
 * (src/molla/engine/sample.mojo:440-483); the library then orders equal
 * probabilities by token id and says so. */
#define MOLLA_ROW_INVALID_CONFIG 0x001u /* row skipped, token = -1 (rules of sample.mojo:140-154) */
#define MOLLA_ROW_UNSUPPORTED 0x002u    /* token = -1: typical_p on a row no top_k / top_p sorted or whose kept set reaches past the
                                         * sorted head (1024 candidates); a min_p floor under 2.2e-8; more than 1024 window + bias entries */
#define MOLLA_ROW_TOPK_TIE 0x004u       /* the top-k boundary splits a run of equal probabilities */
#define MOLLA_ROW_TOPP_TIE 0x008u       /* the top-p cut splits a run of equal probabilities */
#define MOLLA_ROW_CHOSEN_TIE 0x010u     /* the chosen token shares its probability with another kept one */
#define MOLLA_ROW_LOAD_TIMEOUT 0x020u   /* a bounded wait on the row load ran out; result invalid */
#define MOLLA_ROW_SLOW_PATH 0x040u      /* informational: a sequential fallback ran for this row */
#define MOLLA_ROW_DEGENERATE 0x080u     /* more equal values than the candidate buffer holds; token = -1 */
#define MOLLA_ROW_SHARD_OVERFLOW 0x100u /* vocab-sharded form: a shard's list outgrew the exchange buffer */
#define MOLLA_ROW_EMPTY 0x200u          /* the grammar mask left no candidate; token = -1 (the reference raises, sample.mojo:578-579) */

/* Replaces nothing in the reference; lets a binding check what it loaded. */
int32_t molla_sample_abi_version(void);

/* Text of the last error on this host thread ("" if none). */
const char *molla_sample_last_error(void);

/* draw(seed, counter): the reference's counter-based uniform in [0,1), bit for
 * bit. Replaces `draw` at src/molla/engine/sample.mojo:62-71 (and `_mix`,
 * :49-59). Host function, no device work. */
float molla_sample_draw(uint64_t seed, uint64_t counter);

/* Bytes of device workspace `molla_sample_batch` needs for a block of this
 * shape (never zero; 256-byte aligned sizes). Negative status on bad
 * arguments. The reference keeps the equivalent scratch inside each Sampler
 * (`ids`/`vals`, src/molla/engine/sample.mojo:173-177). */
int64_t molla_sample_workspace_bytes(int32_t B, int32_t V, int32_t top_n);

/*
 * Sample one token for every row of a device-resident logit block.
 *
 * Replaces, for all B answered rows at once, the loop
 *     for r in range(len(answered)): streams[i].sampler.pick(self.logits, r)
 * at src/molla/engine/batch.mojo:509-511 together with the device->host copy
 * before it (:504-508), i.e. `Sampler.pick` (src/molla/engine/sample.mojo:
 * 295-359) with every stage it calls (:365-594) and `argmax`
 * (src/molla/nn/kernel.mojo:571-585).
 *
 * d_logits      [B x V] fp32, row r at d_logits + r*row_stride (floats); read only.
 * Per-row arrays, all device pointers of length B (the fields of SamplerConfig,
 * src/molla/engine/sample.mojo:74-126, plus the sampler's counter):
 *   d_temperature (<= 0 is greedy), d_top_k (0 = off), d_top_p (1 = off),
 *   d_min_p (0 = off), d_typical_p (1 = off), d_repeat_penalty (1 = off),
 *   d_frequency_penalty, d_presence_penalty (0 = off),
 *   d_window_on (uint8: repeat_last_n > 0), d_seed, d_drawn (draw number).
 *   Any of d_min_p, d_typical_p, d_window_on may be NULL (= off / off / on).
 * d_hist, d_hist_off   the filled part of each row's penalty window
 *   (Sampler.recent[0..filled), sample.mojo:167-171,260-266): row r's ids are
 *   d_hist[d_hist_off[r] .. d_hist_off[r+1]), int64 like Mojo's Int. NULL = none.
 * d_bias_ids, d_bias_vals, d_bias_off   each row's logit-bias list in the order
 *   `bias()` appended it (sample.mojo:217-234,381-396). NULL = none.
 * top_n         number of top logprobs per row (0..20); logprobs are of the raw
 *   logits as in `Sampler.logprobs` (sample.mojo:268-293).
 * d_workspace   device scratch of at least molla_sample_workspace_bytes().
 * stream        cudaStream_t as a pointer (NULL = default stream).
 * Outputs (device): d_tokens [B] int32 (required); d_chosen_logprob [B] or
 *   NULL; d_top_ids / d_top_logprobs [B x top_n] or NULL when top_n == 0;
 *   d_row_status [B] uint32 (required); d_diag [B x 4] floats or NULL
 *   (softmax denominator, kept-mass sum, draw target, chosen probability:
 *   testing aid).
 */
int32_t molla_sample_batch(
    const float *d_logits, int64_t row_stride, int32_t B, int32_t V,
    const float *d_temperature, const int32_t *d_top_k, const float *d_top_p,
    const float *d_min_p, const float *d_typical_p, const float *d_repeat_penalty,
    const float *d_frequency_penalty, const float *d_presence_penalty,
    const uint8_t *d_window_on, const uint64_t *d_seed, const uint64_t *d_drawn,
    const int64_t *d_hist, const int32_t *d_hist_off, const int64_t *d_bias_ids,
    const float *d_bias_vals, const int32_t *d_bias_off, int32_t top_n, void *d_workspace,
    int64_t workspace_bytes, void *stream, int32_t *d_tokens, float *d_chosen_logprob,
    int32_t *d_top_ids, float *d_top_logprobs, uint32_t *d_row_status, float *d_diag);

/*
 * The decode-step form: what `DeviceBatch.step` would call once the sampler state lives on the
 * device (src/molla/engine/batch.mojo:421-520), so that a step needs no host round trip before
 * the next forward pass. Compared with molla_sample_batch:
 *
 *   - batch row r reads logit row d_rows[r] of the block the forward pass left on the device
 *     (`DeviceScratch.logits`, rows picked by `rows[]`, src/molla/nn/gpu_block.mojo:1676-1680);
 *     d_rows NULL = row r;
 *   - final_softcap > 0 applies `cap * tanh(x / cap)` to every logit as it is read, i.e. the
 *     separate in-place pass of gpu_block.mojo:1568-1571 / gpu_ops.mojo:302-317 is fused into
 *     the first read (the block itself is not written); logprobs are of the capped logits, as
 *     they would be after that pass;
 *   - settings and state are stored per sampler slot (one per live sequence, n_slots of them)
 *     and batch row r uses slot d_slots[r] (NULL = r): every d_* settings array, d_seed,
 *     d_bias_off (n_slots + 1 offsets) and the state arrays are indexed by slot. No slot may
 *     appear twice in one call;
 *   - the state is `Sampler`'s (sample.mojo:157-212): d_ring [n_slots x ring_cap] int64 token
 *     windows with d_ring_head, d_ring_filled and d_ring_len (repeat_last_n of the slot, at most
 *     ring_cap <= 1024; 0 turns the penalties off), and d_drawn, the draw counters. After a
 *     successful pick the kernel does what `_took` does (sample.mojo:361-363, 246-258): the
 *     token enters the window, the counter advances. A row that fails leaves its slot as it was;
 *   - d_stopped [B] (optional) is set where the pick equals d_stop_token[slot] (the end-of-
 *     sequence test of batch.mojo:512-519); d_stop_token NULL or -1 = no stop token.
 *
 * A new sequence takes a slot by writing its settings and zeroing head, filled and drawn
 * (`reset`, sample.mojo:239-244). Everything else is as in molla_sample_batch.
 */
int32_t molla_sample_decode_step(
    const float *d_logits, int64_t row_stride, int32_t n_logit_rows, int32_t V,
    const int32_t *d_rows, const int32_t *d_slots, int32_t B, int32_t n_slots, float final_softcap,
    const float *d_temperature, const int32_t *d_top_k, const float *d_top_p, const float *d_min_p,
    const float *d_typical_p, const float *d_repeat_penalty, const float *d_frequency_penalty,
    const float *d_presence_penalty, const uint64_t *d_seed, uint64_t *d_drawn, int64_t *d_ring,
    int32_t ring_cap, int32_t *d_ring_head, int32_t *d_ring_filled, const int32_t *d_ring_len,
    const int64_t *d_stop_token, const int64_t *d_bias_ids, const float *d_bias_vals,
    const int32_t *d_bias_off, int32_t top_n, void *d_workspace, int64_t workspace_bytes, void *stream,
    int32_t *d_tokens, uint8_t *d_stopped, float *d_chosen_logprob, int32_t *d_top_ids,
    float *d_top_logprobs, uint32_t *d_row_status);

/*
 * Vocab-sharded form, for a tensor-parallel LM head: GPU g holds columns
 * [col0, col0 + V_local) of every row of a vocabulary of V_global. The reference has no
 * multi-GPU mode (docs/roadmap.md:74,80); the result is defined as `Sampler.pick`
 * (src/molla/engine/sample.mojo:295-359) on the unsharded row, and is reproduced bit for
 * bit because the list of logits that can matter to any of the reference's sums, kept in
 * vocabulary order, is a sufficient statistic of a row.
 *
 *   stage_a   per shard: maximum, first index, ties, region maxima and the largest
 *             per-thread maxima of the slice -> d_summary [B x summary_words] floats
 *   (all-gather the summaries: [world][B][summary_words])
 *   merge     per shard: folds them into d_global [B x 4] (global maximum, head threshold,
 *             a bound on the softmax sum before this shard's columns, global argmax) and
 *             answers greedy and top-k = 1 rows straight into d_tokens / d_row_status
 *   stage_b   per shard: the slice's list of (exp bits << 32 | ~token id) entries with
 *             global token ids -> d_list [B x list_cap], d_count [B] (-1 = outgrew list_cap)
 *   (all-gather lists and counts: [world][B][list_cap], [world][B], shards in column order)
 *   stage_c   on every GPU alike: penalties are already in the lists; exact softmax sum,
 *             top-k, top-p and the draw on the concatenated list -> d_tokens, d_row_status
 *
 * The collectives are the caller's (NCCL all-gather over NVLink); at most 16 shards.
 * Per-row arrays are the full batch's on every shard, windows and bias lists with global
 * token ids. Workspaces: molla_sample_workspace_bytes(B, V_local, 0) for stages a and b,
 * molla_sample_workspace_bytes(B, V_global, 0) for stage c.
 */
int32_t molla_sample_shard_summary_words(void);
int32_t molla_sample_shard_stage_a(
    const float *d_logits, int64_t row_stride, int32_t B, int32_t V_local, int32_t col0,
    int32_t V_global, const float *d_temperature, const int32_t *d_top_k, const float *d_top_p,
    const float *d_min_p, const float *d_typical_p, const float *d_repeat_penalty,
    const float *d_frequency_penalty, const float *d_presence_penalty,
    const uint8_t *d_window_on, const int64_t *d_hist, const int32_t *d_hist_off,
    const int64_t *d_bias_ids, const float *d_bias_vals, const int32_t *d_bias_off,
    void *d_workspace, int64_t workspace_bytes, void *stream, float *d_summary);
int32_t molla_sample_shard_merge(
    int32_t B, int32_t V_global, int32_t world, int32_t rank, const float *d_temperature,
    const int32_t *d_top_k, const float *d_gathered_summaries, void *stream, float *d_global,
    int32_t *d_tokens, uint32_t *d_row_status);
int32_t molla_sample_shard_stage_b(
    const float *d_logits, int64_t row_stride, int32_t B, int32_t V_local, int32_t col0,
    int32_t V_global, const float *d_temperature, const int32_t *d_top_k, const float *d_top_p,
    const float *d_min_p, const float *d_typical_p, const float *d_repeat_penalty,
    const float *d_frequency_penalty, const float *d_presence_penalty,
    const uint8_t *d_window_on, const int64_t *d_hist, const int32_t *d_hist_off,
    const int64_t *d_bias_ids, const float *d_bias_vals, const int32_t *d_bias_off,
    const float *d_global, int32_t list_cap, void *d_workspace, int64_t workspace_bytes,
    void *stream, uint64_t *d_list, int32_t *d_count);
int32_t molla_sample_shard_stage_c(
    int32_t B, int32_t V_global, const float *d_temperature, const int32_t *d_top_k,
    const float *d_top_p, const float *d_min_p, const float *d_typical_p,
    const uint64_t *d_seed, const uint64_t *d_drawn, const float *d_global, int32_t world,
    int32_t list_cap, const uint64_t *d_lists, const int32_t *d_counts, void *d_workspace,
    int64_t workspace_bytes, void *stream, int32_t *d_tokens, uint32_t *d_row_status,
    float *d_diag);

/*
 * The same sampling call for callers that must not allocate device memory. It has no
 * counterpart in the reference.
 *
 * Some hosts of this library cannot call cudaMalloc where they sample: a decode loop whose
 * memory was carved up once at start-up and handed out from a fixed arena, a plugin that
 * runs inside another runtime's allocator and may not go round it, a step that has to keep
 * the device heap untouched between two points. molla_sample_batch asks such a caller for a
 * workspace it has no way to obtain. This entry point brings its own: a fixed array of
 * MOLLA_NOALLOC_SCRATCH_BYTES bytes that is part of the library's device image, so every GPU
 * that loads the library gives up that much memory until the process ends, whether or not
 * this function is ever called. Inputs and outputs are still the caller's buffers, with
 * the meaning they have in molla_sample_batch (there is no d_diag).
 *
 * Limits: V <= MOLLA_NOALLOC_MAX_VOCAB and B <= MOLLA_NOALLOC_MAX_ROWS, otherwise
 * MOLLA_ERR_WORKSPACE and nothing is launched. The array holds the working lists of only a
 * few thread blocks at large vocabularies (about 13 at V = 151936), so the call is slower
 * than molla_sample_batch; results are the same.
 *
 * The first call on each device looks up the array's device address (with that device
 * current); make that first call before starting any stream capture. Every call on a device
 * uses the same array and leaves its contents behind; what has to start at zero is cleared
 * on the stream at the start of each call. Two calls that overlap on one GPU (different
 * streams, or different host threads) race on the array: run them one after the other.
 * The function calls no cudaMalloc, cudaFree or allocating library routine.
 */
#define MOLLA_NOALLOC_SCRATCH_BYTES (32u << 20)
#define MOLLA_NOALLOC_MAX_VOCAB 262144
#define MOLLA_NOALLOC_MAX_ROWS 4096
int32_t molla_sample_batch_noalloc(
    const float *d_logits, int64_t row_stride, int32_t B, int32_t V,
    const float *d_temperature, const int32_t *d_top_k, const float *d_top_p,
    const float *d_min_p, const float *d_typical_p, const float *d_repeat_penalty,
    const float *d_frequency_penalty, const float *d_presence_penalty,
    const uint8_t *d_window_on, const uint64_t *d_seed, const uint64_t *d_drawn,
    const int64_t *d_hist, const int32_t *d_hist_off, const int64_t *d_bias_ids,
    const float *d_bias_vals, const int32_t *d_bias_off, int32_t top_n, void *stream,
    int32_t *d_tokens, float *d_chosen_logprob, int32_t *d_top_ids, float *d_top_logprobs,
    uint32_t *d_row_status);

/*
 * The same call for a caller whose logits are in host memory, which is where the
 * reference's decode loop has them after `copy_out` (src/molla/engine/batch.mojo:
 * 504-508, `Buffer` of src/molla/nn/tensor.mojo:270-296): every argument that is a
 * device pointer above is a host pointer here (pinned memory makes the copies
 * asynchronous), the block and the parameters are copied into `d_workspace`, the
 * rows are sampled, the results are copied back and the stream is synchronised
 * before returning. Settings are validated on the host first with the rules and
 * messages of `SamplerConfig.check` (sample.mojo:140-154) and `Sampler.bias`
 * (:225-232): MOLLA_ERR_CONFIG, nothing launched. `temperature` is required;
 * the other per-row arrays may be NULL as above. A block of 32 MB and more goes up in
 * eight pieces on a copy stream the library makes for itself (one per device and
 * calling thread, on first use) while the pieces that have arrived are sampled on
 * `stream`; a row the library did not answer fails the call (MOLLA_ERR_DEVICE).
 */
int64_t molla_sample_host_workspace_bytes(int32_t B, int32_t V, int64_t n_hist, int64_t n_bias,
                                          int32_t top_n);
int32_t molla_sample_batch_host(
    const float *h_logits, int64_t row_stride, int32_t B, int32_t V, const float *temperature,
    const int32_t *top_k, const float *top_p, const float *min_p, const float *typical_p,
    const float *repeat_penalty, const float *frequency_penalty, const float *presence_penalty,
    const uint8_t *window_on, const uint64_t *seed, const uint64_t *drawn, const int64_t *hist,
    const int32_t *hist_off, const int64_t *bias_ids, const float *bias_vals,
    const int32_t *bias_off, int32_t top_n, void *d_workspace, int64_t workspace_bytes,
    void *stream, int32_t *h_tokens, float *h_chosen_logprob, int32_t *h_top_ids,
    float *h_top_logprobs, uint32_t *h_row_status);

/* The rows after logit bias and penalties, before temperature: what
 * `_bias` and `_penalise` (sample.mojo:381-417) leave in `vals`. Same arguments
 * as above where they share a name; d_out is [B x V] fp32, dense. For parity
 * checks of the penalty arithmetic. */
int32_t molla_sample_penalised(
    const float *d_logits, int64_t row_stride, int32_t B, int32_t V,
    const float *d_repeat_penalty, const float *d_frequency_penalty,
    const float *d_presence_penalty, const uint8_t *d_window_on, const int64_t *d_hist,
    const int32_t *d_hist_off, const int64_t *d_bias_ids, const float *d_bias_vals,
    const int32_t *d_bias_off, void *d_workspace, int64_t workspace_bytes, void *stream,
    float *d_out);

/* Full-row logprobs of the raw logits: `Sampler.logprobs`
 * (src/molla/engine/sample.mojo:268-293) for every row. d_out is [B x V]. */
int32_t molla_sample_logprobs(const float *d_logits, int64_t row_stride, int32_t B, int32_t V,
                              void *stream, float *d_out);

/* exp(x) exactly as the kernels evaluate it, element-wise on the device:
 * the one arithmetic dependency the reference takes from outside its tree
 * (`exp` of the Mojo standard library, imported at sample.mojo:40). For tests. */
int32_t molla_sample_expf(const float *d_x, int64_t n, void *stream, float *d_out);

/* log(x) exactly as the typical-p filter evaluates it (`log` of the Mojo standard
 * library at sample.mojo:541,550), element-wise on the device. For tests. */
int32_t molla_sample_logf(const float *d_x, int64_t n, void *stream, float *d_out);

/* molla_sample_batch with a grammar mask: `_mask` (sample.mojo:371-379) is the place where a
 * grammar drops the tokens it forbids, ahead of every other filter; the reference ships it
 * empty. Row r may only choose among the tokens t whose bit is set in
 * d_mask[r * mask_stride_words + t / 32] (bit t % 32); dropped tokens are no candidates at all:
 * they take no bias, no penalty, and no place in the softmax or the top-k count. A row whose
 * mask allows nothing comes back with MOLLA_ROW_EMPTY and token -1. d_mask = NULL is
 * molla_sample_batch. Logprobs stay those of the unmasked logits (sample.mojo:268-293 reads the
 * raw block). Vocabularies of more than 307200 logits are refused with MOLLA_ERR_VOCAB. */
int32_t molla_sample_batch_masked(const uint32_t *d_mask, int64_t mask_stride_words,
                                  const float *d_logits, int64_t row_stride, int32_t B, int32_t V,
                                  const float *d_temperature, const int32_t *d_top_k, const float *d_top_p,
                                  const float *d_min_p, const float *d_typical_p, const float *d_repeat_penalty,
                                  const float *d_frequency_penalty, const float *d_presence_penalty,
                                  const uint8_t *d_window_on, const uint64_t *d_seed, const uint64_t *d_drawn,
                                  const int64_t *d_hist, const int32_t *d_hist_off, const int64_t *d_bias_ids,
                                  const float *d_bias_vals, const int32_t *d_bias_off, int32_t top_n,
                                  void *d_workspace, int64_t workspace_bytes, void *stream, int32_t *d_tokens,
                                  float *d_chosen_logprob, int32_t *d_top_ids, float *d_top_logprobs,
                                  uint32_t *d_row_status, float *d_diag);

/* ---- the vocab-sharded step as one call that owns its collectives ----------------------------
 * No counterpart in the reference (tensor parallelism is on its roadmap, docs/roadmap.md:72-80);
 * the call shape follows how the reference binds C (src/molla/tls/openssl.mojo:53-139): opaque
 * handles as pointers, no callbacks. NCCL is loaded at run time (libnccl.so.2, or the path in
 * MOLLA_LIBNCCL); a host without an NCCL binding creates its communicator through the three
 * functions below: rank 0 asks for an id, hands the 128 bytes to the other ranks by any means it
 * has, and every rank creates its communicator from them with its GPU current. */
int32_t molla_sample_nccl_unique_id(uint8_t *out128);
int32_t molla_sample_nccl_comm_create(const uint8_t *id128, int32_t rank, int32_t world, void **comm_out);
int32_t molla_sample_nccl_comm_destroy(void *comm);
const char *molla_sample_sharded_last_error(void);

/* Device bytes molla_sample_sharded_step needs for B rows of V_local of V_global columns over
 * `world` shards when a shard's list may hold list_cap entries per row (V_local never overflows). */
int64_t molla_sample_sharded_workspace_bytes(int32_t B, int32_t V_local, int32_t V_global, int32_t world, int32_t list_cap);

/* One sampling step on this rank's columns [col0, col0 + V_local) of every row: stage a, an
 * all-gather of the slices' summaries, the merge, stage b, an all-gather of the list lengths
 * and then of only as many list entries per row as the longest list anywhere holds, stage c.
 * All on `stream`; the call waits once in the middle (for the list lengths). Every rank ends
 * with the same tokens, equal to the unsharded call's. Arguments as molla_sample_batch's
 * (per-row arrays replicated on every rank; window and bias ids are global token ids).
 * `wire_bytes` (host, optional): [0] bytes this rank put into the all-gathers, [1] bytes it
 * received, [2] list entries per row that travelled. */
int32_t molla_sample_sharded_step(void *comm, int32_t rank, int32_t world, const float *d_logits, int64_t row_stride,
                                  int32_t B, int32_t V_local, int32_t col0, int32_t V_global,
                                  const float *d_temperature, const int32_t *d_top_k, const float *d_top_p,
                                  const float *d_min_p, const float *d_typical_p, const float *d_repeat_penalty,
                                  const float *d_frequency_penalty, const float *d_presence_penalty,
                                  const uint8_t *d_window_on, const int64_t *d_hist, const int32_t *d_hist_off,
                                  const int64_t *d_bias_ids, const float *d_bias_vals, const int32_t *d_bias_off,
                                  const uint64_t *d_seed, const uint64_t *d_drawn, int32_t list_cap,
                                  void *d_workspace, int64_t workspace_bytes, void *stream, int32_t *d_tokens,
                                  uint32_t *d_row_status, float *d_diag, int64_t *wire_bytes);

/* cudaStreamSynchronize on `stream`, returning a status; then, if
 * `d_row_status` is given, nothing else is implied: rows report for themselves. */
int32_t molla_sample_sync(void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MOLLA_SAMPLE_H */
