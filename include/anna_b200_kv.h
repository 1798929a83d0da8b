/*
 * anna_b200_kv.h - C ABI of libanna_b200_kv.so: the quantized paged KV-cache path of Anna for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes, element strides and a CUDA stream, enqueues its kernels on
 * that stream without synchronising, and returns an int status (0 = ok).  A non-zero status comes with a message
 * from anna_kv_last_error().  Nothing here allocates or frees device memory; scratch is passed in by the caller.  No entry point ever traps or aborts the device: bad page ids are skipped and recorded in the
 * optional device status word.
 *
 * Citations name the interface of the reference (funkpopo/Anna) that each entry point stands in for.
 */
#ifndef ANNA_B200_KV_H_
#define ANNA_B200_KV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of q / K / V / metadata tensors */
#define ANNA_DTYPE_F32 0
#define ANNA_DTYPE_F16 1
#define ANNA_DTYPE_BF16 2

/* status codes */
#define ANNA_OK 0
#define ANNA_ERR_INVALID 1     /* bad argument (shape, stride, null pointer) */
#define ANNA_ERR_UNSUPPORTED 2 /* combination not compiled in (head_dim, dtype, group size) */
#define ANNA_ERR_CUDA 3        /* a CUDA runtime call failed */
#define ANNA_ERR_WORKSPACE 4   /* caller-provided scratch is too small */

/* bits of the device status word written by kernels (OR-ed in, never cleared by the library) */
#define ANNA_DEV_BAD_PAGE 1u   /* a block-table entry needed by a write was < 0 or >= num_pages */
#define ANNA_DEV_PEER_TIMEOUT 2u /* anna_peer_signal_wait gave up waiting for another rank's arrival flag */

typedef void* anna_stream_t; /* cudaStream_t */

/* Message of the last non-zero status returned on the calling thread. */
const char* anna_kv_last_error(void);
int anna_kv_abi_version(void);

/*
 * Health counter: how many bounded waits inside the kernels expired on the current device since the library was
 * loaded (every wait on an asynchronous copy has an iteration limit; a kernel whose wait expires still terminates,
 * but its output is not valid).  0 in a healthy run.  Synchronises the device.  No counterpart in the reference.
 */
int anna_kv_device_faults(int* count);

/*
 * Self-test of that mechanism: one warp waits on a barrier that nothing completes; *expired = 1 when the bounded wait
 * gave up as designed (after its whole budget, about a second).  Synchronises the stream; the context stays usable.
 * No counterpart in the reference.
 */
int anna_kv_selftest_wait_expiry(int* expired, anna_stream_t stream);

/*
 * Self-test of the tensor-memory matrix multiply (tcgen05) in the two operand arrangements of the packed decode:
 *   d1 float [128][16] = a1 . b1^T   a1 uint8 [128][128], b1 uint8 [16][128]: e4m3 bytes, K contiguous
 *   d2 float [128][16] = a2^T . b2   a2 f16 [128 (K)][128 (rows)], b2 f16 [128 (K)][16 (columns)]
 * The kernel re-tiles the row-major inputs into the shared-memory layouts of the real kernel, multiplies with fp32
 * accumulation in tensor memory and returns the accumulators.  *status = 1 when the tensor core did not report back
 * within the bounded wait.  Synchronises the stream.  No counterpart in the reference.
 */
int anna_kv_selftest_umma(const void* a1, const void* b1, const void* a2, const void* b2, float* d1, float* d2,
                          int* status, anna_stream_t stream);

/*
 * Second self-test of the tensor-memory primitives: bf16 operands a, b1, b2 [128][128] (row-major, 16-byte aligned)
 * travel to shared memory by tiled TMA loads with the 128-byte swizzle and are read through swizzled descriptors;
 * d1 = a . b1^T (both K-major), d2 = a . b2 (b2 MN-major: its rows are K indices), float [128][128].  *status = 1 when a
 * bounded wait ran out, 2 when the driver's tensor-map encoder is unavailable.  Synchronises the stream.  No counterpart
 * in the reference.
 */
int anna_kv_selftest_umma_tma(const void* a, const void* b1, const void* b2, float* d1, float* d2, int* status,
                              anna_stream_t stream);

/*
 * Third self-test: d = a . b (bf16 [128][128] operands, float [128][128] result) with a packed into tensor memory by the
 * threads (the A operand of the instruction read from there) and b brought in by TMA, MN-major.  *status as above.
 * Synchronises the stream.  No counterpart in the reference.
 */
int anna_kv_selftest_umma_ts(const void* a, const void* b, float* d, int* status, anna_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------------
 * Split-K scratch shared by all decode entry points.  The context is cut into chunks of `chunk_tokens` tokens; every
 * (row, query head, chunk) leaves a partial in caller-owned float32 buffers
 *   partial_stats  [B, Hq, chunk_capacity, 2]   (running max, denominator)
 *   partial_values [B, Hq, chunk_capacity, D]
 * which a second pass merges: the workspace contract of gqa_decode_splitkv_fused_out
 * (src/anna/model/custom_ops/gated_delta_fused_op.sycl:4634-4706, :1521-1556; capacity may exceed the need).
 * chunk_tokens > 0 is used as given (the reference's `block_size`, src/anna/model/turboquant.py:22);
 * chunk_tokens == 0 asks the library to choose.  Context lengths are only known on the device, so the choice is
 * made from the host-visible upper bound: anna_decode_plan(batch, kv_heads, max_len) returns the chunk length the
 * library will use and the number of chunks the scratch must hold.
 *
 * split_counters (optional, may be NULL): int32 [2, B, Hkv * ceil(G / 8)] that is all-zero on entry (arrival counters,
 * then tile cursors).  When given (and the plan has at most 512 chunks) the 16-bit tensor-core path merges the
 * partials inside the split kernel: whoever finishes a (row, kv-head group) last does the merge and puts the counters
 * back to zero, so the buffer can be reused by the next call on the same stream without clearing.  Without it a second
 * small kernel does the merge.
 */
int anna_decode_plan(int batch, int kv_heads, int64_t max_len, int* chunk_tokens, int* num_chunks);

/* ---------------------------------------------------------------------------------------------------------------
 * Unquantized paged cache.
 */

/*
 * Write T new tokens per row into paged K/V: token (past_lengths[b] + t) of row b goes to
 * pages[page_table[b][pos / S], h, pos % S, :].  Batched form of Qwen3DynamicCache._write_pages
 * (src/anna/model/ops.py:748-777).
 *   k_new, v_new   [B, Hkv, T, D] with element strides (kn_stride_b, kn_stride_h, kn_stride_t); last dim contiguous
 *   key_pages, value_pages  [P, Hkv, S, D] contiguous
 *   page_table     int32 [B, table_stride >= blocks];   past_lengths  int64 [B]
 *   new_lengths    optional int64 [B] (may be NULL, must not alias past_lengths): receives past_lengths[b] + T, so a
 *                  decode loop can keep its lengths on the device instead of uploading them every step
 *   status         optional device int32 (may be NULL): ANNA_DEV_BAD_PAGE is OR-ed in when a page id is invalid
 */
int anna_paged_kv_write(const void* k_new, const void* v_new, int64_t kn_stride_b, int64_t kn_stride_h,
                        int64_t kn_stride_t, void* key_pages, void* value_pages, const int32_t* page_table,
                        int64_t table_stride, const int64_t* past_lengths, int64_t* new_lengths, int batch,
                        int kv_heads, int new_tokens, int head_dim, int block_size, int64_t num_pages,
                        int64_t max_blocks, int dtype, int32_t* status, anna_stream_t stream);

/*
 * Patch a device block table in place: entry i of `entries` is the int32 triple (row, column, page id); triples outside
 * [0, rows) x [0, cols) are ignored.  Replaces the per-row rebuild-and-upload of the table in
 * Qwen3DynamicCache._sync_page_table_layer_buffer (src/anna/model/ops.py:532-588) for the rows that took pages.
 */
int anna_block_table_patch(int32_t* table, int64_t table_stride, int64_t rows, int64_t cols, const int32_t* entries,
                           int count, anna_stream_t stream);

/*
 * Dense view of un-quantized paged K/V: key_out / value_out [B, Hkv, max_len, D] (element strides out_stride_b / _h /
 * _t, last dim contiguous) from the pages named by the block table; positions at or past a row's length and tokens
 * of unmapped blocks come out as zeros.  Stands in for Qwen3DynamicCache._gather_layer_cache
 * (src/anna/model/ops.py:931-1006).
 */
int anna_paged_kv_gather(const void* key_pages, const void* value_pages, const int32_t* page_table,
                         int64_t table_stride, const int64_t* lengths, void* key_out, void* value_out,
                         int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_t, int batch, int kv_heads,
                         int head_dim, int block_size, int64_t num_pages, int64_t max_blocks, int64_t max_len, int dtype,
                         anna_stream_t stream);

/*
 * Single-token GQA decode over paged K/V.  Stands in for torch.ops.anna.paged_gqa_decode_fused
 * (gated_delta_fused_op.sycl:5206-5360, schema :7670-7679): same masking (entries < 0 or >= P are skipped,
 * visible length clamped to [0, max_blocks * S]), fp32 online softmax, optional sigmoid(gate) epilogue, rows with
 * no visible key give zeros.  Split-K over the context with a second combine pass.
 *   q, out         [B, Hq, D] with element strides (stride_b, stride_h); last dim contiguous
 *   gate           NULL or [B, Hq, D] with element strides (gate_stride_b, gate_stride_h)
 *   visible_lengths int64 [B]
 *   partial_stats, partial_values, chunk_capacity, chunk_tokens: split-K scratch (see above); the plan bound is
 *                  max_blocks * block_size tokens
 */
int anna_paged_gqa_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* key_pages,
                          const void* value_pages, const int32_t* page_table, int64_t table_stride,
                          const int64_t* visible_lengths, const void* gate, int64_t gate_stride_b,
                          int64_t gate_stride_h, void* out, int64_t out_stride_b, int64_t out_stride_h,
                          float* partial_stats, float* partial_values, int chunk_capacity, int chunk_tokens,
                          int32_t* split_counters, int batch, int q_heads, int kv_heads, int head_dim,
                          int block_size, int64_t num_pages, int64_t max_blocks, float scaling, int dtype,
                          anna_stream_t stream);

/*
 * Paged decode without caller scratch (no counterpart in the reference).  Same inputs, outputs and result as
 * anna_paged_gqa_decode, for hosts that cannot allocate device memory themselves (a plugin working inside another
 * engine's memory pool, a caller whose allocator is locked): the split-K partials and arrival counters live in a
 * fixed 16 MiB array that is part of the library's device image, so every GPU that loads the library holds those
 * 16 MiB until the process exits.  The entry point calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - Problems whose plan needs more than the array (anna_noalloc_scratch_bytes()) are rejected with
 *     ANNA_ERR_WORKSPACE; batch * kv_heads * ceil(G / 8) must also stay within 8192 (64 KiB of the array hold two
 *     32-bit merge counters per (row, head-group) pair), which is reported with a message of its own.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current); make that first call outside of any stream capture.  Host threads whose first calls on one device
 *     coincide may each do that look-up; they store the same address, so no lock is taken.
 *   - All calls share the one array.  Calls that can overlap on the GPU (different streams, no ordering between
 *     them) race on it; order them or use anna_paged_gqa_decode with separate scratch.
 */
size_t anna_noalloc_scratch_bytes(void);
int anna_paged_gqa_decode_noalloc(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* key_pages,
                                  const void* value_pages, const int32_t* page_table, int64_t table_stride,
                                  const int64_t* visible_lengths, const void* gate, int64_t gate_stride_b,
                                  int64_t gate_stride_h, void* out, int64_t out_stride_b, int64_t out_stride_h,
                                  int batch, int q_heads, int kv_heads, int head_dim, int block_size,
                                  int64_t num_pages, int64_t max_blocks, float scaling, int dtype,
                                  anna_stream_t stream);

/*
 * Single-token GQA decode over dense K/V [B, Hkv, L, D] (arbitrary batch/head/token strides, last dim contiguous)
 * with per-row visible lengths.  Stands in for torch.ops.anna.gqa_decode_fused (gated_delta_fused_op.sycl:4339-4479)
 * and, with visible_lengths == NULL (all L keys visible), for gqa_decode_splitkv_fused / _out (:4494-4769).
 */
int anna_gqa_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* key, const void* value,
                    int64_t kv_stride_b, int64_t kv_stride_h, int64_t kv_stride_t, const int64_t* visible_lengths,
                    const void* gate, int64_t gate_stride_b, int64_t gate_stride_h, void* out, int64_t out_stride_b,
                    int64_t out_stride_h, float* partial_stats, float* partial_values, int chunk_capacity,
                    int chunk_tokens, int32_t* split_counters, int batch, int q_heads, int kv_heads, int64_t key_len,
                    int head_dim, float scaling, int dtype, anna_stream_t stream);

/*
 * Multi-token (prefill / chunked prefill) GQA over dense K/V: q [B, Hq, T, D], key / value [B, Hkv, L, D], out
 * [B, Hq, T, D], element strides for batch / head / token, last dim contiguous.  Replaces grouped_query_attention
 * (src/anna/model/ops.py:1552-1574) for the masks the model builds (ops.py:1840-1852, :2008-2016):
 *   key_lengths int64 [B] (or NULL = L): row r sees its first key_lengths[r] keys (visible_mask / key_padding_mask in
 *   prefix form); causal != 0: query t sits at position key_lengths[r] - T + t and sees keys up to its own position.
 * softmax in fp32; a query without any visible key gives zeros.  16-bit dtypes, head_dim 64 / 128 / 256 (else
 * ANNA_ERR_UNSUPPORTED); q / k / v 16-byte aligned with strides that are multiples of 8 elements.
 */
int anna_gqa_prefill(const void* q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_t, const void* key,
                     const void* value, int64_t kv_stride_b, int64_t kv_stride_h, int64_t kv_stride_t,
                     const int64_t* key_lengths, void* out, int64_t out_stride_b, int64_t out_stride_h,
                     int64_t out_stride_t, int batch, int q_heads, int kv_heads, int q_len, int64_t key_len,
                     int head_dim, float scaling, int causal, int dtype, anna_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------------
 * TurboQuant packed paged cache.
 *
 * Packed pool: uint8 [P, Hkv, chunk_bytes]; one chunk holds S tokens of one kv head:
 *   key codes  S x (D*bits/8)  | key norms S x f32 | key residual norms S x f32 |
 *   value codes S x (D*sb/8)   | value scales S x (D/group) x dtype | value zeros S x (D/group) x dtype
 * (sb = 2 for bits == 2 else 4, as in quantize_turboquant_values, src/anna/model/turboquant.py:214), every
 * sub-array starting on a 16-byte boundary and the chunk padded to 128 bytes; anna_tq_page_layout reports the
 * offsets.  Quantized token j of a row lives in block j / S of the row's table, slot j % S.
 * The newest `residual_len` tokens of a row stay un-quantized in a ring: window [slots, 2, Hkv, R, D] (index 0 =
 * keys, 1 = values), token position p in ring slot p % R.
 */
typedef struct anna_tq_layout {
  int32_t key_bytes;   /* packed key bytes per token */
  int32_t value_bytes; /* packed value bytes per token */
  int32_t groups;      /* value groups per token */
  int32_t off_kcodes, off_knorm, off_krnorm, off_vdata, off_vscale, off_vzero;
  int32_t chunk_bytes;
} anna_tq_layout;

int anna_tq_page_layout(int head_dim, int bits, int block_size, int dtype, int value_group, anna_tq_layout* out);

/*
 * Append T tokens per row: the batched, fused form of TurboQuantKVRow.append (src/anna/model/turboquant.py:1027-1140)
 * driven by Qwen3DynamicCache._update_turboquant_layer (src/anna/model/ops.py:618-660).  With L = old_lengths[b] and
 * L' = L + T, every token whose position falls below L' - R and that is not yet quantized is rotated, indexed,
 * sign-projected, value-quantized (turboquant.py:199-230, :255-272) and bit-packed straight into its page; tokens that
 * stay inside the window are written to the ring.  A ring slot is read before the same warp overwrites it.
 *   k_new, v_new  [B, Hkv, T, D] element strides (kn_stride_b, kn_stride_h, kn_stride_t)
 *   old_lengths   int64 [B] (lengths before this call);  window_slots int64 [B] (ring index of each row)
 *   new_lengths   optional int64 [B] (may be NULL, must not alias old_lengths): receives old_lengths[b] + T
 *   shared_blocks optional uint32 [B, mask_stride] bit mask (may be NULL): bit j of row b set = block j of that row is a
 *                 page mapped from another sequence with the same prompt prefix and already holds these tokens' codes,
 *                 so its tokens are not quantized again (extends the prefix sharing of ops.py:779-857 to packed pages)
 *   signs1, signs2  float32 [D] (+1 / -1): rotation and QJL sign vectors;  centroids float32 [2^(bits-1)];
 *   boundaries    float32 [2^(bits-1) - 1]
 */
int anna_tq_append(const void* k_new, const void* v_new, int64_t kn_stride_b, int64_t kn_stride_h,
                   int64_t kn_stride_t, uint8_t* packed_pages, const int32_t* block_table, int64_t table_stride,
                   const uint32_t* shared_blocks, int64_t mask_stride, void* window, const int64_t* window_slots, const int64_t* old_lengths, int64_t* new_lengths,
                   const float* signs1, const float* signs2, const float* centroids, const float* boundaries,
                   int batch, int kv_heads, int new_tokens, int head_dim, int block_size, int residual_len, int bits,
                   int value_group, int64_t num_pages, int64_t max_blocks, int dtype, int32_t* status,
                   anna_stream_t stream);

/*
 * Single-token GQA decode over [packed quantized prefix | un-quantized window].  Batched, paged form of
 * TurboQuantKVRow.decode_attention (src/anna/model/turboquant.py:1181-1293) /
 * Qwen3DynamicCache.turboquant_single_token_decode_attention (src/anna/model/ops.py:1024-1070) and of
 * torch.ops.anna.gqa_decode_splitkv_turboquant_fused_out (gated_delta_fused_op.sycl:4771-5094), except that keys are
 * scored from their packed codes in the rotated basis (the identity of turboquant_key_attention_scores,
 * turboquant.py:290-332) instead of from a dense de-quantized copy.
 *   lengths   int64 [B]: total tokens per row (quantized = max(0, L - R), window = min(L, R)); L == 0 gives zeros
 *   query_scratch: optional 16-byte aligned device scratch of at least anna_tq_query_scratch_bytes(B, Hq, Hkv, D)
 *   bytes; the tensor-core path stores the rotated queries there (as fp16 MMA fragments)
 *   before the split pass.  Without it, or for fp32 caches, head_dim 64, value groups other than 32 or page sizes that
 *   are not a multiple of 16, the CUDA-core path runs.
 *   split-K slots: anna_tq_decode_plan gives the chunk length and the slot count (window chunks first, then the
 *   chunks of the packed prefix); scratch and counters as for the other decode entry points
 */
int anna_tq_decode_plan(int batch, int kv_heads, int64_t max_blocks, int block_size, int residual_len,
                        int* chunk_tokens, int* num_chunks);
size_t anna_tq_query_scratch_bytes(int batch, int q_heads, int kv_heads, int head_dim);  /* 0 for invalid sizes */

int anna_tq_paged_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h, const uint8_t* packed_pages,
                         const int32_t* block_table, int64_t table_stride, const void* window,
                         const int64_t* window_slots, const int64_t* lengths, const float* signs1,
                         const float* signs2, const float* centroids, const void* gate, int64_t gate_stride_b,
                         int64_t gate_stride_h, void* out, int64_t out_stride_b, int64_t out_stride_h,
                         float* partial_stats, float* partial_values, int chunk_capacity, int chunk_tokens,
                         int32_t* split_counters, void* query_scratch, size_t query_scratch_bytes, int batch,
                         int q_heads, int kv_heads, int head_dim, int block_size, int residual_len, int bits,
                         int value_group, int64_t num_pages, int64_t max_blocks, float scaling, int dtype,
                         anna_stream_t stream);

/*
 * KV-head-sharded form of anna_tq_paged_decode for the GPUs of one box: this rank decodes its own KV heads and the
 * merge that finishes a (row, head group) stores the output row into `out` and, at the same element offset, into
 * num_peers (0..7) peer tensors -- the output tensors of the other ranks, mapped into this process -- so that no
 * all-gather follows.  `out` and the peer pointers address this rank's first query head inside [B, Hq_total, D]
 * tensors of equal strides.  Needs the tensor-core path with the fused merge (16-bit cache, head_dim 128 / 256,
 * split_counters given); otherwise ANNA_ERR_UNSUPPORTED.  The stores are plain peer stores over NVLink followed by a
 * system-scope fence; readers on the other ranks synchronise through anna_peer_signal_wait.
 * The reference is single-device and has no counterpart.
 */
int anna_tq_paged_decode_peers(const void* q, int64_t q_stride_b, int64_t q_stride_h, const uint8_t* packed_pages,
                               const int32_t* block_table, int64_t table_stride, const void* window,
                               const int64_t* window_slots, const int64_t* lengths, const float* signs1,
                               const float* signs2, const float* centroids, const void* gate, int64_t gate_stride_b,
                               int64_t gate_stride_h, void* out, int64_t out_stride_b, int64_t out_stride_h,
                               float* partial_stats, float* partial_values, int chunk_capacity, int chunk_tokens,
                               int32_t* split_counters, void* query_scratch, size_t query_scratch_bytes, int batch,
                               int q_heads, int kv_heads, int head_dim, int block_size, int residual_len, int bits,
                               int value_group, int64_t num_pages, int64_t max_blocks, float scaling, int dtype,
                               void* const* peer_outputs, int num_peers, anna_stream_t stream);

/*
 * Arrival flags between the ranks of one box.  flag_arrays[r] (host array of `world` device pointers, 8-byte aligned)
 * is rank r's array of `world` uint64 flags in memory every rank can write; entry [rank] is the caller's own.  One warp
 * stores `step` into flag `rank` of every other rank (release, system scope: everything this stream wrote to peer
 * memory before is visible first), then waits until the caller's own flags of all other ranks are >= step.  Steps
 * are positive and must grow from call to call; flags start at 0.  After timeout_ms (1..60000) without the flags the kernel ORs
 * ANNA_DEV_PEER_TIMEOUT into *status (optional device int32) and returns; the context stays usable.  world == 1
 * launches nothing.  No counterpart in the reference.
 */
int anna_peer_signal_wait(void* const* flag_arrays, int rank, int world, int64_t step, int64_t timeout_ms,
                          int32_t* status, anna_stream_t stream);

/*
 * De-quantize the packed prefix of each row to dense [B, Hkv, Lq_max, D] keys and values in the cache dtype (element
 * strides out_stride_b / _h / _t; rows shorter than max_quantized_len are left untouched beyond their length).
 * Stands in for TurboQuantKVRow._materialize_quantized_prefix (src/anna/model/turboquant.py:925-984), i.e.
 * dequantize_turboquant_keys (:275-287) + dequantize_turboquant_values (:233-252).
 */
int anna_tq_materialize(const uint8_t* packed_pages, const int32_t* block_table, int64_t table_stride,
                        const int64_t* quantized_lengths, const float* signs1, const float* signs2,
                        const float* centroids, void* key_out, void* value_out, int64_t out_stride_b,
                        int64_t out_stride_h, int64_t out_stride_t, int batch, int kv_heads, int head_dim,
                        int block_size, int bits, int value_group, int64_t num_pages, int64_t max_blocks,
                        int64_t max_quantized_len, int dtype, anna_stream_t stream);

/*
 * Single-token GQA decode over (dense de-quantized keys | packed values | un-quantized residual), the exact operand
 * set of torch.ops.anna.gqa_decode_splitkv_turboquant_fused_out (gated_delta_fused_op.sycl:4771-5094, schema
 * :7652-7669, validator :1447-1501).  All tensors carry element strides for batch / head / token; last dim contiguous.
 *   quantized_key [B, Hkv, Lq, D];  value_data uint8 [B, Hkv, Lq, D / per_byte] (per_byte = 4 for 2 bits, else 2);
 *   value_scales / value_zeros [B, Hkv, Lq, D / value_group] in the query dtype (shared strides);
 *   residual_key / residual_value [B, Hkv, Lr, D] (may be NULL when Lr == 0);  scratch as for the other decode calls
 */
int anna_gqa_decode_turboquant_values(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                      const void* quantized_key, int64_t qk_stride_b, int64_t qk_stride_h,
                                      int64_t qk_stride_t, const uint8_t* value_data, int64_t vd_stride_b,
                                      int64_t vd_stride_h, int64_t vd_stride_t, const void* value_scales,
                                      const void* value_zeros, int64_t vs_stride_b, int64_t vs_stride_h,
                                      int64_t vs_stride_t, const void* residual_key, const void* residual_value,
                                      int64_t r_stride_b, int64_t r_stride_h, int64_t r_stride_t, const void* gate,
                                      int64_t gate_stride_b, int64_t gate_stride_h, void* out, int64_t out_stride_b,
                                      int64_t out_stride_h, float* partial_stats, float* partial_values,
                                      int chunk_capacity, int chunk_tokens, int batch, int q_heads, int kv_heads,
                                      int64_t quantized_len, int64_t residual_len, int head_dim, int value_bits,
                                      int value_group, float scaling, int dtype, anna_stream_t stream);

/*
 * Dense view of a batch of TurboQuant rows in one launch: keys / values [B, Hkv, max_len, D] in the cache dtype with
 * the de-quantized prefix, then the un-quantized window tokens (read from the ring), then zeros up to max_len.
 * Batched form of Qwen3DynamicCache._gather_layer_cache for quantized layers (src/anna/model/ops.py:931-1006, which
 * calls TurboQuantKVRow.materialize row by row, turboquant.py:1142-1179, and pads).
 *   lengths int64 [B] (total tokens per row);  window_slots int64 [B];  other arguments as anna_tq_paged_decode
 */
int anna_tq_gather_dense(const uint8_t* packed_pages, const int32_t* block_table, int64_t table_stride,
                         const void* window, const int64_t* window_slots, const int64_t* lengths, const float* signs1,
                         const float* signs2, const float* centroids, void* key_out, void* value_out,
                         int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_t, int batch, int kv_heads,
                         int head_dim, int block_size, int residual_len, int bits, int value_group, int64_t num_pages,
                         int64_t max_blocks, int64_t max_len, int dtype, anna_stream_t stream);

/*
 * MSE-only TurboQuant codes for a plain tensor row: what TurboQuantTensorRow (src/anna/model/turboquant.py:335-477, the
 * K / V history rows of the Gemma4 runtime) asks of TurboQuantMSE(dim, bits, seed=42).quantize / .dequantize
 * (turboquant.py:392-395, :415-418).  Every [head_dim] vector becomes `bits`-bit Lloyd-Max indices of its normalised,
 * rotated coordinates plus its fp32 norm.  head_dim 64 / 128 / 256 / 512; bits 2 / 3 / 4.
 *   x / out   [heads, tokens, head_dim] with element strides (stride_h, stride_t), last dim contiguous
 *   idx       uint8 [heads, capacity, anna_tq_tensor_row_bytes(head_dim, bits)]: 2-bit fields for bits == 2, else 4-bit
 *             fields, low field first;   norms  float32 [heads, capacity]
 *   offset    position of token 0 of this call inside the code buffers (offset + tokens <= capacity)
 *   signs1 float32 [head_dim];  boundaries float32 [2^bits - 1];  centroids float32 [2^bits]
 */
int anna_tq_tensor_row_bytes(int head_dim, int bits);
int anna_tq_tensor_quantize(const void* x, int64_t stride_h, int64_t stride_t, uint8_t* idx, float* norms,
                            int64_t capacity, int64_t offset, int heads, int tokens, int head_dim, int bits,
                            const float* signs1, const float* boundaries, int dtype, anna_stream_t stream);
int anna_tq_tensor_dequantize(const uint8_t* idx, const float* norms, int64_t capacity, int64_t offset, void* out,
                              int64_t stride_h, int64_t stride_t, int heads, int tokens, int head_dim, int bits,
                              const float* signs1, const float* centroids, int dtype, anna_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* ANNA_B200_KV_H_ */
