/* b200_attn.h -- C ABI of the B200 (sm_100a) paged-KV attention library, libb200attn.so.
 *
 * The entry points are what a binding for nano-vllm's attention layer calls in place of the
 * reference's Triton kernel and flash_attn calls.  File:line citations are relative to the
 * nano-vllm project root.
 *
 * Conventions
 *  - Every pointer is a device pointer on the current CUDA device unless stated otherwise.
 *    The compute entry points never allocate, free or copy device memory and never synchronise;
 *    every launch goes to `stream` (a cudaStream_t passed as void*; NULL = legacy default stream),
 *    so calls can be captured into CUDA graphs.  The exceptions say so in their own comments: the
 *    two status queries synchronise the device, b200_ipc_open maps another process's buffer.
 *  - Activations and caches are bf16 for the attention entry points.  head_dim must be 128.
 *  - Strides are in ELEMENTS.  Pointers and row strides must be 16-byte aligned.
 *  - The paged cache has the reference's layout (nanovllm/engine/model_runner.py:107-117): one
 *    contiguous array (num_blocks, block_size, num_kv_heads, head_dim) for K and one for V;
 *    flat slot = block_id * block_size + offset.  block_size must be a multiple of 256
 *    (nanovllm/config.py:22).
 *  - Block tables are int32 (batch, bt_cols) with row stride bt_row_stride; entries at columns
 *    >= ceil(len / block_size) may hold -1 or stale ids (nanovllm/engine/model_runner.py:119-123,
 *    :203) and are never dereferenced.
 *  - Return value: 0 on success; negative = arguments rejected before any launch; positive = a
 *    cudaError_t from the launch.  b200_last_error() describes the last failure of the calling
 *    thread.  Nothing throws, aborts or traps.
 */
#ifndef B200_ATTN_H_
#define B200_ATTN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ATTN_VERSION 100

#define B200_OK 0
#define B200_ERR_NULL_POINTER (-1)
#define B200_ERR_BAD_SHAPE (-2)
#define B200_ERR_MISALIGNED (-3)
#define B200_ERR_WORKSPACE (-4)
#define B200_ERR_NO_DRIVER (-5)
#define B200_ERR_TENSOR_MAP (-6)
#define B200_ERR_DEVICE (-7)
#define B200_ERR_TIMEOUT (-8)

/* Library version (B200_ATTN_VERSION of the build). */
int b200_version(void);

/* Message for the last non-zero status returned to this thread ("" if none). Host pointer,
 * valid until the thread's next failing call. */
const char* b200_last_error(void);

/* Replaces store_kvcache_kernel + store_kvcache (nanovllm/layers/attention.py:10-40).
 * For token i in [0, n_tokens): slot = slot_mapping[i]; slot == -1 is skipped; otherwise the
 * row_elems elements of key row i (at key + i * key_row_stride) are copied to flat cache row
 * `slot` of k_cache, and likewise for value / v_cache.  Pure byte copy (any elem_bytes);
 * row_elems * elem_bytes and both row strides must be multiples of 16 bytes.  Offsets are
 * formed in 64 bits.  n_slots (= num_blocks * block_size) bounds the slot: an out-of-range
 * slot is skipped, never written.  n_tokens == 0 is a no-op. */
int b200_store_kvcache(const void* key, const void* value, int64_t key_row_stride, int64_t value_row_stride,
                       void* k_cache, void* v_cache, const int32_t* slot_mapping, int32_t n_tokens,
                       int32_t row_elems, int32_t elem_bytes, int64_t n_slots, void* stream);

/* Bytes of workspace b200_decode_attn needs for any batch up to `max_batch` with this head
 * geometry on the current device (depends on its multiprocessor count).  The caller allocates
 * it once, ZERO-FILLS it once, and passes it to every call; the kernels leave the parts that
 * must be zero as they found them.  Calls that share a workspace must not overlap on the GPU.
 * Returns a negative status on bad arguments. */
int64_t b200_decode_workspace_bytes(int32_t max_batch, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim);

/* Replaces flash_attn_with_kvcache as called for decode (nanovllm/layers/attention.py:71-74).
 * For sequence i: the single query token q[i] (num_heads x head_dim at q + i * q_row_stride)
 * attends the context_lens[i] cached tokens reached through block_tables[i, :]; GQA maps q head
 * h to kv head h / (num_heads / num_kv_heads); softmax(scale * q k^T) v with fp32 softmax and
 * accumulation; out[i] (num_heads x head_dim, contiguous rows of num_heads * head_dim) in bf16.
 * context_lens[i] <= 0 writes zeros and touches no cache.  The launch geometry depends only on
 * (batch, head geometry), never on device data.  The launch may begin while the previous kernel of
 * the stream is still running if that kernel lets it (programmatic dependent launch: of this library
 * b200_store_kvcache and b200_qk_norm_rope_store do); it reads context_lens and block_tables before it
 * waits for that kernel, so a kernel that triggers its dependents early must not be the writer of
 * those two arrays. */
int b200_decode_attn(const void* q, int64_t q_row_stride, const void* k_cache, const void* v_cache,
                     int64_t num_blocks, int32_t block_size, const int32_t* block_tables, int64_t bt_row_stride,
                     int32_t bt_cols, const int32_t* context_lens, void* out, void* workspace,
                     int64_t workspace_bytes, int32_t batch, int32_t num_heads, int32_t num_kv_heads,
                     int32_t head_dim, float scale, void* stream);

/* No counterpart in the reference: decode attention for callers that cannot allocate.
 *
 * b200_decode_attn needs a caller-owned workspace.  Some callers have no way to provide one: an
 * engine that has already given all free device memory to its KV cache (a later cudaMalloc may
 * fail), a plugin interface that forbids allocating inside the call, code that must stay away from
 * the framework's allocator.  This variant computes exactly what b200_decode_attn computes, with
 * the same arguments minus the workspace, and keeps its scratch inside the library: a __device__
 * array of b200_decode_static_scratch_bytes() (8 249 600 bytes, about 7.9 MiB) that every GPU which loads the
 * library holds until the process exits.  It calls no cudaMalloc/cudaFree and no allocating
 * library routine.
 *
 * Limits (rejected with B200_ERR_WORKSPACE and a message, nothing launched): (persistent CTAs of
 * the device = 2 per multiprocessor) x (num_heads / num_kv_heads) may be at most 1280 -- on a
 * 148-SM B200 that is up to 4 query heads per kv head -- and num_kv_heads at most 128.  Beyond
 * that use b200_decode_attn.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 * that device current); make that first call before any stream capture begins.  All calls on a
 * device share the one array: it keeps the previous call's contents (the entry point clears the
 * part that must start at zero, on `stream`, before launching), and two calls that overlap on
 * the GPU -- different streams, or different host threads -- race on it.  Serialise them. */
int64_t b200_decode_static_scratch_bytes(void);
int b200_decode_attn_static(const void* q, int64_t q_row_stride, const void* k_cache, const void* v_cache,
                            int64_t num_blocks, int32_t block_size, const int32_t* block_tables,
                            int64_t bt_row_stride, int32_t bt_cols, const int32_t* context_lens, void* out,
                            int32_t batch, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim, float scale,
                            void* stream);

/* Replaces flash_attn_varlen_func as called for prefill (nanovllm/layers/attention.py:64-70).
 * Sequence i owns query rows cu_seqlens_q[i] .. cu_seqlens_q[i+1] of q (total_q, num_heads, 128)
 * and keys 0 .. Lk_i - 1 with Lk_i = cu_seqlens_k[i+1] - cu_seqlens_k[i].  Causal mask aligned
 * bottom-right: query row r sees keys 0 .. Lk_i - Lq_i + r.
 *  - block_tables == NULL: dense K/V.  k, v are (total_k, num_kv_heads, 128) with row strides
 *    k_row_stride / v_row_stride, sequence i's keys at rows cu_seqlens_k[i] ...
 *  - block_tables != NULL (prefix cache): K/V for the whole key range come from k_cache/v_cache
 *    through block_tables[i, t / block_size]; k and v are ignored.
 * Sequences with Lq_i == 0 produce no rows.  out is (total_q, num_heads, 128) contiguous bf16.
 * max_seqlen_q / max_seqlen_k are the host-side bounds the caller already has
 * (nanovllm/utils/context.py:9-10).  kernel_variant: 0 = default (the persistent tcgen05 kernel
 * when 128 % (num_heads / num_kv_heads) == 0, else the mma.sync kernel), 1 = force the mma.sync
 * kernel, 2 = force the tcgen05 kernel (B200_ERR_BAD_SHAPE if it cannot take the shape).  Launches
 * of the tcgen05 kernel share one device-side ticket counter: do not overlap two of them on one
 * GPU.  The persistent kernel
 * writes `out` through TMA stores: out must be 16-byte aligned (as every tensor here). */
int b200_prefill_attn(const void* q, int64_t q_row_stride, const void* k, const void* v, int64_t k_row_stride,
                      int64_t v_row_stride, int64_t total_k, const void* k_cache, const void* v_cache,
                      int64_t num_blocks, int32_t block_size, const int32_t* block_tables, int64_t bt_row_stride,
                      int32_t bt_cols, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int32_t batch,
                      int32_t total_q, int32_t max_seqlen_q, int32_t max_seqlen_k, void* out, int32_t num_heads,
                      int32_t num_kv_heads, int32_t head_dim, float scale, int32_t kernel_variant, void* stream);

/* ---- producer side of the layer: QK-norm + rotary embedding + cache store in one launch -------------------
 * Replaces, for one decoder layer and one step, what the reference runs between its fused qkv projection
 * and its attention call (nanovllm/models/qwen3.py:75-79 and nanovllm/layers/attention.py:62-63):
 *   q_norm, k_norm   nanovllm/layers/layernorm.py:16-26       fp32 RMS normalisation over head_dim, cast to
 *                                                              bf16, times the bf16 weight
 *   rotary_emb       nanovllm/layers/rotary_embedding.py:6-14  rotate-half with cos/sin gathered by position
 *   store_kvcache    nanovllm/layers/attention.py:10-40        k (after norm and rotation) and v to their slots
 * qkv is the (n_tokens, (num_heads + 2 * num_kv_heads) * 128) bf16 output of the fused projection with row
 * stride qkv_row_stride (elements); positions are int64 as in the reference; cos_sin_cache is the reference's
 * (max_position, 1, 128) fp32 table (64 cos then 64 sin per position).  q_out (n_tokens, num_heads, 128) and
 * k_out (n_tokens, num_kv_heads, 128) are written contiguous (dense prefill reads k from there).  With
 * k_cache / v_cache given, token i's k and v rows also go to flat cache row slot_mapping[i] (-1 and slots
 * >= n_slots are skipped); both NULL = no store (the engine's warm-up pass).  v is never copied anywhere else:
 * the attention call keeps reading it as a view of qkv. */
int b200_qk_norm_rope_store(const void* qkv, int64_t qkv_row_stride, const int64_t* positions, const void* q_weight,
                            const void* k_weight, const float* cos_sin_cache, int32_t max_position, float eps,
                            void* q_out, void* k_out, void* k_cache, void* v_cache, const int32_t* slot_mapping,
                            int64_t n_slots, int32_t n_tokens, int32_t num_heads, int32_t num_kv_heads,
                            int32_t head_dim, void* stream);

/* ---- caller side of the decode path: a step's metadata into the graph's static buffers in one launch -----
 * Replaces, for one decode step, the seven device operations with which the reference's model runner moves
 * its freshly copied metadata into the buffers its CUDA graphs were captured on
 * (nanovllm/engine/model_runner.py:193-203), and lets its five host-to-device copies (:163-179, :119-123)
 * become one: the host packs the step into one record,
 *   int64 input_ids[batch] | int64 positions[batch] | int32 slot_mapping[batch] | int32 context_lens[batch] |
 *   int32 block_tables[batch][table_width]  (rows padded with -1)
 * copies it to the device (8-byte aligned), and this call scatters it with the reference's exact effect:
 * rows [0, batch) of input_ids and positions are written; slot_mapping is -1 and context_lens 0 on rows
 * [batch, buffer_rows); block_tables (row stride buffer_table_cols) gets columns [0, table_width) of rows
 * [0, batch) and keeps the rest.  batch <= buffer_rows and table_width <= buffer_table_cols. */
int b200_unpack_decode_metadata(const void* packed, int32_t batch, int32_t table_width, int32_t buffer_rows,
                                int32_t buffer_table_cols, int64_t* input_ids, int64_t* positions,
                                int32_t* slot_mapping, int32_t* context_lens, int32_t* block_tables, void* stream);

/* ---- behind the path: the all-reduce after the output projection, for decode-sized messages ---------------
 * Replaces `dist.all_reduce(y)` in RowParallelLinear.forward (nanovllm/layers/linear.py:149-153) when y is at
 * most b200_small_allreduce_max_bytes() (512 KiB) of bf16: a one-shot sum over plain peer loads and stores.
 * Set-up is the caller's: every rank allocates an exchange buffer of b200_small_allreduce_buffer_bytes(),
 * zero-filled, shares it with the other ranks of the node (CUDA IPC) and passes the `world` device pointers under
 * which IT sees the ranks' buffers (own buffer at index `rank`; a HOST array of pointers), plus a private,
 * zero-filled device block of b200_small_allreduce_state_bytes().  All ranks must make the same sequence of calls
 * with the same sizes.  inout (n_elems bf16, a multiple of 8, 16-byte aligned) is replaced by the sum over ranks,
 * accumulated in fp32 in rank order (every rank gets identical bits).  Every wait is bounded
 * (wait_limit_seconds, default 1 s when <= 0): a rank whose peers do not show up leaves its message unchanged
 * and sets a status word, read with b200_small_allreduce_status(); after that the ranks must zero their buffers
 * and state blocks together before the next call.  The launch can be captured in a CUDA graph. */
int64_t b200_small_allreduce_buffer_bytes(void);
int64_t b200_small_allreduce_state_bytes(void);
int64_t b200_small_allreduce_max_bytes(void);
int b200_small_allreduce(void* const* peer_buffers, int32_t rank, int32_t world, void* local_state, void* inout,
                         int64_t n_elems, double wait_limit_seconds, void* stream);
/* Synchronises the current device and returns B200_ERR_TIMEOUT if a wait of b200_small_allreduce gave up since the
 * state block was zero-filled, else 0. */
int b200_small_allreduce_status(const void* local_state);
/* Set-up helpers for the exchange buffers (no counterpart in the reference, which leaves this to NCCL): export a
 * device buffer of this process as a 64-byte CUDA IPC handle plus the buffer's offset inside its allocation, and map
 * a buffer exported by another process into the current device's address space.  The mapping lasts until the process
 * exits.  Host pointers for handle, offset and result. */
int b200_ipc_export(const void* ptr, void* handle_out_64_bytes, int64_t* offset_out);
int b200_ipc_open(const void* handle_64_bytes, int64_t offset, void** ptr_out);

/* Number of kernels this library has launched from the calling process so far (all threads).
 * Benchmarks use the difference across a timed region. */
int64_t b200_launch_count(void);

/* Diagnostic, not for the hot path: synchronises the current device and returns
 * B200_ERR_TIMEOUT if any kernel of this library gave up on a bounded wait since the last call
 * that reported one (the output of that launch is undefined), a positive cudaError_t if the
 * device reports an error, else 0.  A call that reports a timeout also recovers: it clears the
 * status words and the prefill kernel's ticket counter, so later launches start clean and the
 * next call speaks about them only.  What the library cannot reach is the caller-owned decode
 * workspace: if the failed launch was a decode, zero-fill that workspace again. */
int b200_device_status(void);

/* Test hook for the recovery path above, never called by the product: synchronises the device and
 * leaves the library's device-side state as a prefill launch that gave up on a wait would have
 * left it (status word set, ticket counter stale).  Nothing is launched and no GPU fault is
 * involved.  The next b200_device_status() must report B200_ERR_TIMEOUT and repair the state. */
int b200_test_inject_timeout(void);

#ifdef __cplusplus
}
#endif
#endif /* B200_ATTN_H_ */
