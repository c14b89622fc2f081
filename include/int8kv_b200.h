/*
 * int8kv_b200 — C ABI of the B200 (sm_100a) INT8 paged-KV decode kernels.
 *
 * Every entry point takes plain device pointers, sizes and element strides; no framework
 * types cross this boundary.  All calls are asynchronous on `stream` (a cudaStream_t passed
 * as void*), never synchronise the device, never allocate device memory and never throw:
 * they return 0 or a negative INT8KV_E_* code.  The caller owns every buffer, including the
 * split-KV workspace (int8kv_paged_attn_int8_static_ws, which brings its own, is the one
 * exception and says so).  The library keeps no mutable state apart from per-device "set up
 * once" flags, so it may be called from several host threads and streams.
 *
 * Tensor conventions (the reference prototype cjsmt/Int8-kvcache uses the same ones):
 *   key/value (new tokens)  [T, Hkv, D]                bf16 / fp16 / fp32, any strides
 *   key_cache/value_cache   [num_blocks, BS, Hkv, D]   int8 (or bf16/fp16 for the baseline)
 *   slot_mapping            [T]        int32/int64, slot = block*BS + offset, slot < 0 = skip
 *   query / out             [B, Hq, D]                 bf16 / fp16 / fp32
 *   block_tables            [B, width] int32/int64, logical block -> physical block
 *   seq_lens                [B]        int32/int64
 *   k_scale / v_scale       [Hkv]      fp32
 * Query head h reads KV head h / (Hq/Hkv).  Strides are in ELEMENTS of the tensor's dtype.
 */
#ifndef INT8KV_B200_H
#define INT8KV_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define INT8KV_ABI_VERSION 2

/* status codes */
#define INT8KV_OK 0
#define INT8KV_E_NULLPTR (-1)     /* a required pointer is NULL */
#define INT8KV_E_BAD_SHAPE (-2)   /* sizes/strides inconsistent (Hq % Hkv, negative sizes, ...) */
#define INT8KV_E_BAD_DTYPE (-3)   /* dtype code out of range */
#define INT8KV_E_UNSUPPORTED (-4) /* valid request that no kernel here covers */
#define INT8KV_E_LAUNCH (-5)      /* CUDA reported an error at launch / attribute set-up */
#define INT8KV_E_WORKSPACE (-6)   /* workspace missing or smaller than int8kv_workspace_bytes() */

/* dtype codes for float tensors */
#define INT8KV_BF16 0
#define INT8KV_FP16 1
#define INT8KV_FP32 2

/* Bits set by a kernel in the workspace's trailing status word (see int8kv_workspace_status_offset). */
#define INT8KV_DEV_WAIT_TIMEOUT 1u /* a bounded wait for a staged page ran out; result invalid */
#define INT8KV_DEV_SLOT_MISMATCH 2u /* int8kv_decode_step: a slot was not the slot of its sequence's last token */

/* num_splits values with a special meaning (attention entry points) */
#define INT8KV_SPLITS_AUTO 0      /* choose from the shape; large calls may plan their parts on the device */
#define INT8KV_SPLITS_PLANNED (-1) /* always plan on the device; INT8KV_E_UNSUPPORTED for shapes outside the tiled
                                      kernels, more than 512 sequences or more (sequence, head) pairs than resident
                                      warps; INT8KV_E_WORKSPACE below int8kv_workspace_bytes_auto() bytes */

/*
 * `flags` of the attention entry points (a bit set; 0 = none).
 *   INT8KV_FLAG_QUANTIZE_Q    quantise each query head to INT8 (absmax/127, round half away from zero) before the
 *                             dot product, the reference's QUANTIZE_Q option (src/triton_ops/int8_paged_attention.py
 *                             :137-146).  INT8 caches with static scales only.
 *   INT8KV_FLAG_INPUTS_READY  a promise by the caller: nothing this call READS (query, new K/V rows, slot mapping,
 *                             block tables, sequence lengths, caches, scales) is written by the kernel that
 *                             precedes the call on `stream`.  The tiled kernels then start streaming pages while
 *                             that kernel (typically the previous layer's split-KV merge) is still running, and
 *                             order themselves behind it only before their first write.  Results are identical;
 *                             a call of about 10 us gets 2-3 us shorter in a chain of such calls.  Breaking the
 *                             promise gives stale reads, not a fault.  Shapes outside the tiled kernels ignore it.
 *                             No counterpart in the reference (one Triton launch per call, fully ordered).
 */
#define INT8KV_FLAG_QUANTIZE_Q 1
#define INT8KV_FLAG_INPUTS_READY 2

int int8kv_abi_version(void);
const char* int8kv_status_str(int status);

/*
 * INT8 KV cache write.  Replaces int8_kv_cache_write and its Triton kernel
 * (reference src/triton_ops/int8_cache_write.py:7-149): q = clamp(rint(x / max(scale,1e-6)), -127, 127)
 * with an IEEE fp32 quotient and round-half-to-even (the rounding of the reference's own oracle,
 * src/quant.py:37-40), stored at cache[slot / BS, slot % BS, head, :]; rows with slot < 0 are skipped and
 * every other cache byte is left untouched.  Slots >= num_blocks*BS are skipped as well.
 */
int int8kv_cache_write(const void* key, const void* value, int in_dtype,
                       int64_t num_tokens, int num_kv_heads, int head_dim,
                       const int64_t key_strides[3], const int64_t value_strides[3],
                       int8_t* key_cache, int8_t* value_cache,
                       const int64_t key_cache_strides[4], const int64_t value_cache_strides[4],
                       int64_t num_blocks, int block_size,
                       const void* slot_mapping, int slot_is_i64,
                       const float* k_scale, const float* v_scale,
                       void* stream);

/*
 * INT8 paged decode attention.  Replaces int8_paged_attention with its V3/V4 kernels and the split-KV
 * merge (reference src/triton_ops/int8_paged_attention.py:68-769).  out[b,h,:] = softmax(q.K^T * k_scale/sqrt(D)) .
 * V * v_scale over the first seq_lens[b] tokens of sequence b.  A sequence with seq_len <= 0 yields zeros.
 *   num_splits  0 = choose from the shape (int8kv_choose_splits; for large calls of up to 512 sequences the
 *               kernel itself reads seq_lens and cuts every sequence into parts of one common length, chosen so
 *               that all parts together fill a whole number of resident waves of warps, if the workspace has
 *               int8kv_workspace_bytes_auto() bytes), -1 = always plan on the device, >= 1 = exactly that many
 *   max_seq_len_hint  upper bound of seq_lens used only to size the grid; <= 0 means width*BS
 *   workspace   required when the effective split count is > 1: int8kv_workspace_bytes() bytes
 *   flags       INT8KV_FLAG_* bits (INT8KV_FLAG_QUANTIZE_Q = 1, so a plain 0/1 "quantize_q" still means the same)
 */
int int8kv_paged_attn_int8(const void* query, int q_dtype, const int64_t q_strides[3],
                           int batch, int num_q_heads, int num_kv_heads, int head_dim,
                           const int8_t* key_cache, const int8_t* value_cache,
                           const int64_t key_cache_strides[4], const int64_t value_cache_strides[4],
                           int64_t num_blocks, int block_size,
                           const void* block_tables, int bt_is_i64, const int64_t bt_strides[2], int64_t bt_width,
                           const void* seq_lens, int sl_is_i64, int64_t max_seq_len_hint,
                           const float* k_scale, const float* v_scale,
                           void* out, int out_dtype, const int64_t out_strides[3],
                           int num_splits, void* workspace, int64_t workspace_bytes,
                           int flags, void* stream);

/*
 * BF16/FP16 paged decode attention, the same-run baseline.  Replaces bf16_paged_attention
 * (reference src/triton_ops/bf16_paged_attention.py:9-165).  `cache_dtype` is INT8KV_BF16 or INT8KV_FP16.
 * flags: INT8KV_FLAG_INPUTS_READY only.
 */
int int8kv_paged_attn_bf16(const void* query, int q_dtype, const int64_t q_strides[3],
                           int batch, int num_q_heads, int num_kv_heads, int head_dim,
                           const void* key_cache, const void* value_cache, int cache_dtype,
                           const int64_t key_cache_strides[4], const int64_t value_cache_strides[4],
                           int64_t num_blocks, int block_size,
                           const void* block_tables, int bt_is_i64, const int64_t bt_strides[2], int64_t bt_width,
                           const void* seq_lens, int sl_is_i64, int64_t max_seq_len_hint,
                           void* out, int out_dtype, const int64_t out_strides[3],
                           int num_splits, void* workspace, int64_t workspace_bytes,
                           int flags, void* stream);

/*
 * Variants that return unmerged partial attention for a sequence-parallel split: every rank attends to its own
 * tokens and writes rows of int8kv_partial_row_floats(D) fp32 = [out (D floats, normalised) | lse | padding] into
 * `partial` ([B, Hq, row]); lse is the natural-log sum-exp of the scaled scores, -inf for an empty range.  The rows
 * of all ranks, gathered into local memory, are combined by int8kv_merge_partials.  This is the split-KV step of
 * the reference (:293-318) exposed across devices; the reference itself has no multi-GPU path.
 */
int int8kv_paged_attn_int8_partial(const void* query, int q_dtype, const int64_t q_strides[3],
                           int batch, int num_q_heads, int num_kv_heads, int head_dim,
                           const int8_t* key_cache, const int8_t* value_cache,
                           const int64_t key_cache_strides[4], const int64_t value_cache_strides[4],
                           int64_t num_blocks, int block_size,
                           const void* block_tables, int bt_is_i64, const int64_t bt_strides[2], int64_t bt_width,
                           const void* seq_lens, int sl_is_i64, int64_t max_seq_len_hint,
                           const float* k_scale, const float* v_scale,
                           float* partial,
                           int num_splits, void* workspace, int64_t workspace_bytes,
                           int flags, void* stream);

/*
 * Dynamic per-(token, head) INT8 cache write.  Replaces reshape_and_cache_int8 and its Triton kernel (reference
 * vllm_int8/vllm_int8_cache_ops.py:13-210), the reference's alternative quantisation scheme: for every token and
 * KV head, scale = max(absmax / 127, 1e-6) over the D elements, q = clamp(x / scale, +-127) rounded half away from
 * zero; the INT8 row goes to cache[slot / BS, slot % BS, head, :] and the fp32 scale to scale_cache[slot / BS,
 * slot % BS, head] ([num_blocks, BS, Hkv], strides in elements).  slot < 0 skips the token.
 */
int int8kv_cache_write_dynamic(const void* key, const void* value, int in_dtype,
                               int64_t num_tokens, int num_kv_heads, int head_dim,
                               const int64_t key_strides[3], const int64_t value_strides[3],
                               int8_t* key_cache, int8_t* value_cache,
                               const int64_t key_cache_strides[4], const int64_t value_cache_strides[4],
                               float* k_scale_cache, float* v_scale_cache,
                               const int64_t k_scale_strides[3], const int64_t v_scale_strides[3],
                               int64_t num_blocks, int block_size,
                               const void* slot_mapping, int slot_is_i64, void* stream);

/*
 * INT8 paged decode attention over a cache written by int8kv_cache_write_dynamic: the K and V bytes of token t,
 * head h dequantise with k_scale_cache / v_scale_cache [num_blocks, BS, Hkv] (fp32, any strides) instead of one
 * static scale per head.  out = softmax(q . (K8 * ks)^T / sqrt(D)) . (V8 * vs), the attention of the cache that
 * dequantize_int8_cache (vllm_int8/vllm_int8_cache_ops.py:250-277) reconstructs.  The reference stops at that
 * write/dequantise pair and has no attention kernel for this scheme; this entry point is the reader that pairs
 * with its writer.  Other arguments as int8kv_paged_attn_int8 (flags: INT8KV_FLAG_INPUTS_READY only).
 */
int int8kv_paged_attn_int8_dynamic(const void* query, int q_dtype, const int64_t q_strides[3],
                                   int batch, int num_q_heads, int num_kv_heads, int head_dim,
                                   const int8_t* key_cache, const int8_t* value_cache,
                                   const int64_t key_cache_strides[4], const int64_t value_cache_strides[4],
                                   const float* k_scale_cache, const float* v_scale_cache,
                                   const int64_t k_scale_strides[3], const int64_t v_scale_strides[3],
                                   int64_t num_blocks, int block_size,
                                   const void* block_tables, int bt_is_i64, const int64_t bt_strides[2], int64_t bt_width,
                                   const void* seq_lens, int sl_is_i64, int64_t max_seq_len_hint,
                                   void* out, int out_dtype, const int64_t out_strides[3],
                                   int num_splits, void* workspace, int64_t workspace_bytes, int flags, void* stream);

/*
 * One decode step of one layer in a single call: the step's `batch` new K/V rows (one per sequence) are quantised
 * and written at slot_mapping, and query attends over the updated cache.  This is the pair of calls that the
 * reference's vLLM hooks make back to back for every layer (do_kv_cache_update then forward,
 * vllm_int8/vllm_shadow_cache_patch.py:154-166 and vllm_int8/vllm_int8_attention_patch.py:117-137).
 * Contract: seq_lens already count the new token and slot_mapping[b] is the slot of token seq_lens[b] - 1 of
 * sequence b (what a decode step produces), or negative for a padding row.  For the shapes the tiled kernel
 * covers the write happens inside the attention kernel (no separate launch): the warp that owns a sequence's
 * last tile quantises the row, stores it to the cache and patches its staged copy.  A slot that is not the last
 * token's is still written, but attention may not see it and INT8KV_DEV_SLOT_MISMATCH is set in the status word.
 * Other shapes run int8kv_cache_write followed by int8kv_paged_attn_int8.  flags: INT8KV_FLAG_INPUTS_READY (the new
 * rows and the slot mapping count as inputs of the call).
 */
int int8kv_decode_step(const void* key, const void* value, int kv_dtype,
                       const int64_t key_strides[3], const int64_t value_strides[3],
                       const void* slot_mapping, int slot_is_i64,
                       const void* query, int q_dtype, const int64_t q_strides[3],
                       int batch, int num_q_heads, int num_kv_heads, int head_dim,
                       int8_t* key_cache, int8_t* value_cache,
                       const int64_t key_cache_strides[4], const int64_t value_cache_strides[4],
                       int64_t num_blocks, int block_size,
                       const void* block_tables, int bt_is_i64, const int64_t bt_strides[2], int64_t bt_width,
                       const void* seq_lens, int sl_is_i64, int64_t max_seq_len_hint,
                       const float* k_scale, const float* v_scale,
                       void* out, int out_dtype, const int64_t out_strides[3],
                       int num_splits, void* workspace, int64_t workspace_bytes, int flags, void* stream);

/*
 * The decode step of `num_layers` layers in one call: int8kv_decode_step once per entry of `layers`, in order, on
 * `stream`, sharing every shape, stride, table and the workspace.  It exists to pay the host cost of a call
 * (argument marshalling of the binding, validation) once per model step instead of once per layer: the reference's
 * microbenchmark and its vLLM hooks make 28 such calls per step for Qwen2.5-7B.  Per layer: query, output, the
 * layer's cache pair and scales, and the step's new K/V rows (key == NULL: attention only, nothing is written, and
 * slot_mapping may be NULL).  Stops at the first layer that fails and returns its status; *failed_layer (optional)
 * then holds its index, else -1.
 * flags: with INT8KV_FLAG_INPUTS_READY the promise is about the layers of this call: no layer reads what an earlier
 * layer of the call writes (all queries and new rows were produced before the call, every layer has its own cache
 * and output).  The first layer orders itself behind whatever precedes the call in the ordinary way; the layers
 * after it are CHAINED when the workspace holds at least twice what one layer needs (and starts on a 256-byte
 * boundary): layer l works in half l % 2 of the workspace, and its split-KV merge is not a launch of its own but
 * rides, as extra thread blocks, on the launch of layer l + 1, whose page stream starts while layer l is still
 * draining.  A step is then one launch per layer plus one closing merge; layer l's output is complete when layer
 * l + 1's launch is (all outputs when the call's work on the stream is).  Results are identical to unchained calls.
 * With a smaller workspace the layers still overlap their predecessor's merge, as single calls with the flag do.
 */
typedef struct int8kv_layer_args {
  const void* query;      /* [batch, Hq, D] */
  void* out;              /* [batch, Hq, D] */
  const void* key;        /* [batch, Hkv, D] new rows of this step, or NULL */
  const void* value;
  int8_t* key_cache;      /* [num_blocks, BS, Hkv, D] */
  int8_t* value_cache;
  const float* k_scale;   /* [Hkv] */
  const float* v_scale;
} int8kv_layer_args;

int int8kv_decode_step_layers(const int8kv_layer_args* layers, int num_layers, int* failed_layer,
                              int kv_dtype, const int64_t key_strides[3], const int64_t value_strides[3],
                              const void* slot_mapping, int slot_is_i64,
                              int q_dtype, const int64_t q_strides[3],
                              int batch, int num_q_heads, int num_kv_heads, int head_dim,
                              const int64_t key_cache_strides[4], const int64_t value_cache_strides[4],
                              int64_t num_blocks, int block_size,
                              const void* block_tables, int bt_is_i64, const int64_t bt_strides[2], int64_t bt_width,
                              const void* seq_lens, int sl_is_i64, int64_t max_seq_len_hint,
                              int out_dtype, const int64_t out_strides[3],
                              int num_splits, void* workspace, int64_t workspace_bytes, int flags, void* stream);

/*
 * The BF16/FP16 baseline for `num_layers` layers in one call: int8kv_paged_attn_bf16 once per entry of `layers`
 * (query, out, key_cache, value_cache; key, value and the scales must be NULL), sharing shapes, tables and the
 * workspace, with the same chaining under INT8KV_FLAG_INPUTS_READY as int8kv_decode_step_layers, so that the
 * baseline can be timed under the conditions of the INT8 path.  The reference's baseline is one call per layer
 * (src/triton_ops/bf16_paged_attention.py:118-165).
 */
int int8kv_paged_attn_bf16_layers(const int8kv_layer_args* layers, int num_layers, int* failed_layer,
                              int cache_dtype, int q_dtype, const int64_t q_strides[3],
                              int batch, int num_q_heads, int num_kv_heads, int head_dim,
                              const int64_t key_cache_strides[4], const int64_t value_cache_strides[4],
                              int64_t num_blocks, int block_size,
                              const void* block_tables, int bt_is_i64, const int64_t bt_strides[2], int64_t bt_width,
                              const void* seq_lens, int sl_is_i64, int64_t max_seq_len_hint,
                              int out_dtype, const int64_t out_strides[3],
                              int num_splits, void* workspace, int64_t workspace_bytes, int flags, void* stream);

/*
 * INT8 paged decode attention for callers that must not allocate device memory.  No counterpart in the
 * reference: there every call allocates its split-KV buffers with torch.empty.
 *
 * Who needs it: a serving engine that has already handed every free byte of HBM to its KV-cache pool (a late
 * cudaMalloc can fail, or fragment the pool), and request loops that may not call cudaMalloc at all because it
 * synchronises the whole device at an unpredictable moment.  Such a caller passes only inputs and the output;
 * the split-KV partial rows go to a buffer that is part of the library image itself: INT8KV_STATIC_WS_BYTES
 * bytes of device memory, held by every GPU that loads the library until the process exits.
 *
 * Limits and rules:
 *   - num_splits means what it means for int8kv_paged_attn_int8 called with a workspace of INT8KV_STATIC_WS_BYTES
 *     bytes: 0 picks the count from the shape (the rule of the tiled kernels or of the kernels for other shapes,
 *     or parts planned on the device where those fit the buffer), -1 insists on the device plan, n >= 1 is taken
 *     as given.  The call is rejected with INT8KV_E_WORKSPACE, before anything is launched, when the split-KV rows
 *     of the chosen count (int8kv_workspace_bytes) do not fit in INT8KV_STATIC_WS_BYTES; pass a smaller num_splits
 *     (1 needs almost nothing) or use int8kv_paged_attn_int8 with a workspace of your own;
 *   - the first call on each device looks up the device address of the buffer (with that device current);
 *     make that first call outside any stream capture;
 *   - all calls on a device share the one buffer, which keeps whatever the previous call left in it.  Nothing in
 *     it has to start at zero (every row is written before it is read), but two calls of one process whose
 *     kernels overlap on the GPU (different streams or host threads) race on it: serialise them;
 *   - the device status word (INT8KV_DEV_* bits, set when a bounded wait ran out: the result is then invalid)
 *     lives at the end of that buffer; int8kv_static_ws_status copies it out, again without allocating;
 *   - it never calls cudaMalloc, cudaFree or any allocating library routine.
 * Arguments and result are those of int8kv_paged_attn_int8 without the workspace pair.
 */
#define INT8KV_STATIC_WS_BYTES (8 * 1024 * 1024)
int int8kv_paged_attn_int8_static_ws(const void* query, int q_dtype, const int64_t q_strides[3],
                           int batch, int num_q_heads, int num_kv_heads, int head_dim,
                           const int8_t* key_cache, const int8_t* value_cache,
                           const int64_t key_cache_strides[4], const int64_t value_cache_strides[4],
                           int64_t num_blocks, int block_size,
                           const void* block_tables, int bt_is_i64, const int64_t bt_strides[2], int64_t bt_width,
                           const void* seq_lens, int sl_is_i64, int64_t max_seq_len_hint,
                           const float* k_scale, const float* v_scale,
                           void* out, int out_dtype, const int64_t out_strides[3],
                           int num_splits, int flags, void* stream);

/*
 * Status word of the library's own workspace, for callers of int8kv_paged_attn_int8_static_ws (no counterpart in
 * the reference, which has no failure detection).  Enqueues on `stream` an asynchronous 4-byte copy of the word to
 * `dst` (device memory or pinned host memory of the caller; read it after synchronising the stream) and, with
 * `clear` non-zero, a reset of the word to 0 behind it.  The bits are only ever OR-ed by the kernels, so without a
 * clear they stay set across later calls.  Allocates nothing.
 */
int int8kv_static_ws_status(void* dst, int clear, void* stream);

/*
 * Device address of the library's own workspace (INT8KV_STATIC_WS_BYTES bytes) on the current device, for tools
 * that want to hand it to an entry point taking a workspace, such as int8kv_selftest_bounded_wait.  The first call
 * on a device looks the address up; make it outside any stream capture.
 */
int int8kv_static_ws_address(void** device_ptr);

/*
 * Merge `num_parts` partial results.  Replaces _merge_split_kv_kernel (reference
 * src/triton_ops/int8_paged_attention.py:330-388): out = sum_r w_r * out_r / sum_r w_r, w_r = exp(lse_r - max lse);
 * parts with lse = -inf are ignored; all-empty rows give zeros.  `parts` is [num_parts, rows, row_floats] fp32 with
 * rows = B*Hq and row_floats = int8kv_partial_row_floats(D).
 */
int int8kv_merge_partials(const float* parts, int num_parts, int batch, int num_q_heads, int head_dim,
                          void* out, int out_dtype, const int64_t out_strides[3], void* stream);

/*
 * Sequence-parallel exchange over peer memory (NVLink / NVSwitch), for the split of one long sequence across GPUs
 * with one process per GPU.  The reference has no multi-GPU path; the math is its split-KV merge (:330-388) across
 * devices, as with int8kv_paged_attn_int8_partial + int8kv_merge_partials, but the partial rows travel by plain
 * 16-byte stores into the other ranks' memory instead of through a collective library, every fp32 value paired with
 * the step's number so that the receiver recognises a value of the current step by itself (no flag behind the data,
 * no fence on the sender):
 *   - every rank owns one exchange buffer of int8kv_exchange_bytes() bytes, 256-byte aligned, ZEROED before first
 *     use, and mapped into every other rank's address space (CUDA IPC or a symmetric-memory allocator; the library
 *     allocates and maps nothing).  `peer_buffers[r]` is rank r's buffer as seen from THIS process; entry `rank`
 *     is the local one.  All ranks must agree on world, batch, num_q_heads, head_dim;
 *   - int8kv_paged_attn_int8_partial_push computes this rank's partial rows (arguments of
 *     int8kv_paged_attn_int8_partial) and stores them into every rank's buffer; it never waits for another GPU;
 *   - int8kv_merge_exchanged, enqueued behind it on the same stream, waits until every rank's rows of the current
 *     step have arrived and merges them from LOCAL memory.  The wait is bounded (about a second); if it runs out,
 *     INT8KV_DEV_WAIT_TIMEOUT is set in the status word of `workspace` (optional) and the output is left unwritten.
 *     (With 4 ranks or more the rows are scattered to owner ranks and the merged rows gathered from them instead
 *     of every row going to every rank; see int8kv_merge_exchanged_phase.  The calls stay the same.)
 * Both keep their step count on the device, so the pair can be captured in a CUDA graph and replayed.  Every rank must
 * make the same sequence of push / merge pairs; buffers alternate between two slabs so that a fast rank's next step
 * does not overwrite what a slow rank is still merging.
 */
typedef struct int8kv_exchange {
  int world;                 /* ranks, 1..16 */
  int rank;                  /* this process's rank */
  void* peer_buffers[16];    /* [world] device addresses valid in this process */
  int64_t buffer_bytes;      /* size of each buffer */
} int8kv_exchange;

int64_t int8kv_exchange_bytes(int world, int batch, int num_q_heads, int head_dim);

int int8kv_paged_attn_int8_partial_push(const void* query, int q_dtype, const int64_t q_strides[3],
                           int batch, int num_q_heads, int num_kv_heads, int head_dim,
                           const int8_t* key_cache, const int8_t* value_cache,
                           const int64_t key_cache_strides[4], const int64_t value_cache_strides[4],
                           int64_t num_blocks, int block_size,
                           const void* block_tables, int bt_is_i64, const int64_t bt_strides[2], int64_t bt_width,
                           const void* seq_lens, int sl_is_i64, int64_t max_seq_len_hint,
                           const float* k_scale, const float* v_scale,
                           const int8kv_exchange* exchange,
                           int num_splits, void* workspace, int64_t workspace_bytes,
                           int flags, void* stream);

int int8kv_merge_exchanged(const int8kv_exchange* exchange, int batch, int num_q_heads, int head_dim,
                           void* out, int out_dtype, const int64_t out_strides[3],
                           void* workspace, int64_t workspace_bytes, void* stream);

/*
 * The two halves of int8kv_merge_exchanged, for hosts that put other work between them.  With 4 ranks or more (and a
 * row count B * Hq that divides by them) the exchange does not send every row to every rank: a push sends a row to one
 * owner rank, the owner merges its rows (INT8KV_EXCHANGE_MERGE_PHASE) and stores the merged fp32 rows into every
 * rank's buffer, and every rank then writes `out` from what the owners sent (INT8KV_EXCHANGE_GATHER_PHASE) — a
 * quarter of the bytes on eight GPUs.  With fewer ranks the merge phase is the whole step and the gather phase does
 * nothing.  INT8KV_EXCHANGE_BOTH_PHASES is int8kv_merge_exchanged.  Every rank must run both phases, in this order,
 * with the same arguments.
 */
#define INT8KV_EXCHANGE_BOTH_PHASES 0
#define INT8KV_EXCHANGE_MERGE_PHASE 1
#define INT8KV_EXCHANGE_GATHER_PHASE 2
int int8kv_merge_exchanged_phase(const int8kv_exchange* exchange, int batch, int num_q_heads, int head_dim,
                                 void* out, int out_dtype, const int64_t out_strides[3],
                                 void* workspace, int64_t workspace_bytes, int phase, void* stream);

/*
 * Self-test of the failure path.  Every wait for staged data inside the kernels is bounded; when one runs out the
 * kernel sets INT8KV_DEV_WAIT_TIMEOUT in the workspace's status word and returns.  This entry point launches one warp
 * that waits, with at most `attempts` (1..65536) attempts of about a microsecond, for data that nothing sends, so a
 * caller can check that the timeout is reported and the context stays usable.  No counterpart in the reference,
 * which has no failure detection.
 */
int int8kv_selftest_bounded_wait(void* workspace, int64_t workspace_bytes, int attempts, void* stream);

/* Floats per partial row: D for the output, one for the lse, padded to a multiple of 4. */
int int8kv_partial_row_floats(int head_dim);

/* Bytes of split-KV workspace for `num_splits` splits (includes the trailing status word). */
int64_t int8kv_workspace_bytes(int batch, int num_q_heads, int head_dim, int num_splits);

/* Bytes of workspace with which every automatic path (num_splits 0 or -1) of the attention entry points is
 * available for this shape, the device-planned one included: partial rows of the items and the per-sequence
 * table.  Never smaller than int8kv_workspace_bytes() for the split count int8kv_choose_splits() picks.
 * A planned call leaves {items, part length in 16-token tiles, waves aimed for, INT8KV_PLAN_HEADER_TAG} as four
 * int32 in the 16 bytes before the status word (other calls may use those bytes for partial rows). */
#define INT8KV_PLAN_HEADER_TAG 0x504c414e
int64_t int8kv_workspace_bytes_auto(int batch, int num_q_heads, int num_kv_heads, int head_dim, int64_t max_seq_len,
                                    int block_size, int sm_count);

/* Byte offset of the 32-bit device status word inside a workspace of `workspace_bytes` bytes. */
int64_t int8kv_workspace_status_offset(int64_t workspace_bytes);

/* Split count the library would pick for this shape on a device with `sm_count` SMs
 * (re-derivation of _choose_num_splits, reference :39-49, for 148 SMs). */
int int8kv_choose_splits(int batch, int num_kv_heads, int64_t max_seq_len, int block_size, int sm_count);

/* Largest split count any entry point accepts. */
int int8kv_max_splits(void);

#ifdef __cplusplus
}
#endif
#endif /* INT8KV_B200_H */
