/* C ABI of libdscuda_mla_bench.so and libdscuda_flash_attention_bench.so.
 *
 * Plain pointers and sizes only.  Every tensor argument is a DEVICE pointer the
 * caller owns; `stream` is a cudaStream_t passed as void*.  Functions returning
 * int give 0 on success and 1 on failure; the message of the last failure on the
 * calling thread is returned by the matching *_last_error().  No call
 * allocates, synchronises or reads device memory back, so all of them can be
 * captured in a CUDA graph.
 *
 * The symbols marked "reference:" replace the extern "C" function of the same
 * name in the reference's benchmarks/bindings/ and keep its signature, so the
 * reference's benchmarks/mla.py and benchmarks/flash_attention.py bind them
 * unchanged.
 */
#ifndef DSCUDA_C_API_H
#define DSCUDA_C_API_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* reference: benchmarks/bindings/mla_bridge.cu:12 */
const char* dscuda_mla_last_error(void);

/* reference: benchmarks/bindings/mla_bridge.cu:16-21 (ctypes [P]*6+[I]*5+[F,P],
 * benchmarks/mla.py:28).  Absorbed causal forward; bf16 tensors, fp32 lse. */
int dscuda_mla_forward(
    void* output, float* lse,
    const void* query, const void* query_rope, const void* latent, const void* key_rope,
    int batch, int sequence, int heads, int rank, int rope, float scale, void* stream);

/* reference: benchmarks/bindings/mla_bridge.cu:33-40 ([P]*11+[I]*5+[F,P],
 * benchmarks/mla.py:29). */
int dscuda_mla_backward(
    void* dquery, void* dquery_rope, void* dlatent, void* dkey_rope,
    const void* dout, const void* output, const float* lse,
    const void* query, const void* query_rope, const void* latent, const void* key_rope,
    int batch, int sequence, int heads, int rank, int rope, float scale, void* stream);

/* reference: benchmarks/bindings/mla_bridge.cu:53-56 (benchmarks/mla.py:31-32). */
size_t dscuda_mla_workspace_elements(int batch, int heads, int splits, int rank);

/* reference: benchmarks/bindings/mla_bridge.cu:58-63 ([P]*7+[I]*7+[F,P],
 * benchmarks/mla.py:30). */
int dscuda_mla_decode(
    void* output, float* lse,
    const void* query, const void* paged_cache,
    const int* block_table, const int* lengths, float* workspace,
    int batch, int heads, int rank, int rope, int page_size, int pages, int splits,
    float scale, void* stream);

/* No counterpart in the reference (include/mla.h, mla_decode_forward_checked_cuda):
 * dscuda_mla_decode plus the number of physical cache pages; a block-table entry
 * outside [0, cache_blocks) is read as page 0 and sets the device status to 3. */
int dscuda_mla_decode_checked(
    void* output, float* lse,
    const void* query, const void* paged_cache,
    const int* block_table, const int* lengths, float* workspace,
    int batch, int heads, int rank, int rope, int page_size, int pages, int cache_blocks, int splits,
    float scale, void* stream);

/* No counterpart in the reference: paged decode that takes no workspace and
 * allocates nothing.  For hosts that cannot allocate device memory where they
 * call from (fixed up-front memory pools, plugins inside a foreign allocator,
 * places where cudaMalloc would stall the device).  The split partials live in a
 * fixed 16.1 MiB array inside the library; batch*heads*splits may be at most
 * dscuda_mla_decode_static_capacity() (8192), else status 1.  The first call on
 * a device resolves the array's address and should happen outside stream
 * capture.  All calls on a device share the array: calls that overlap on the
 * GPU race, so keep them in one stream order. */
size_t dscuda_mla_decode_static_capacity(void);
int dscuda_mla_decode_static(
    void* output, float* lse,
    const void* query, const void* paged_cache,
    const int* block_table, const int* lengths,
    int batch, int heads, int rank, int rope, int page_size, int pages, int splits,
    float scale, void* stream);

/* No counterpart in the reference (include/mla.h, mla_cache_append_cuda): writes
 * the rows [latent | key_rope] of new tokens into the paged cache, in the layout
 * reference/python/mla.py:11-23 packs on the host.  start_positions and
 * token_counts may be NULL (0, and all `tokens` rows). */
int dscuda_mla_cache_append(
    void* paged_cache, const void* latent, const void* key_rope,
    const int* block_table, const int* start_positions, const int* token_counts,
    int batch, int tokens, int rank, int rope, int page_size, int pages, int cache_blocks,
    void* stream);

/* No counterpart in the reference (include/mla.h, mla_cache_append_fp8_cuda): dscuda_mla_cache_append
 * into the FP8 cache format (656 bytes per token: 512 e4m3, four fp32 group scales, 64 bf16 rotary). */
int dscuda_mla_cache_append_fp8(
    void* paged_fp8_cache, const void* latent, const void* key_rope,
    const int* block_table, const int* start_positions, const int* token_counts,
    int batch, int tokens, int rank, int rope, int page_size, int pages, int cache_blocks,
    void* stream);

/* No counterpart in the reference (mla_cache_dequantize_fp8_cuda): physical rows
 * [first_row, first_row + rows) of the FP8 cache rewritten in the bf16 layout dscuda_mla_decode reads. */
int dscuda_mla_cache_dequantize_fp8(
    void* paged_cache, const void* paged_fp8_cache, long long first_row, long long rows, void* stream);

/* No counterpart in the reference (include/mla.h, mla_rope_apply_cuda): rotary
 * embedding in place of q_pe [rows,heads,64] and k_pe [rows,1,64]; either pointer
 * may be NULL; positions may be NULL (position = row % sequence_length). */
int dscuda_mla_rope_apply(
    void* q_pe, void* k_pe, const int* positions,
    long long rows, int heads, int sequence_length, int rope, float theta, void* stream);

/* No counterpart in the reference: non-absorbed causal prefill forward
 * (include/mla.h, mla_prefill_forward_cuda).  cu_seqlens may be NULL (dense). */
int dscuda_mla_prefill_forward(
    void* output, float* lse,
    const void* q_nope, const void* q_pe, const void* k_nope, const void* k_pe, const void* v,
    const int* cu_seqlens, int batch, int max_sequence, int total_tokens, int heads,
    int nope, int rope, int value, float scale, void* stream);

/* No counterpart in the reference (mla_prefill_backward_scratch_limit): workspace the dense backward may
 * use for dS^T; returns the previous limit, a negative value only reads it. */
size_t dscuda_mla_prefill_backward_scratch_limit(long long bytes);

/* No counterpart in the reference (mla_prefill_backward_launches): kernels per backward call. */
int dscuda_mla_prefill_backward_launches(int batch, int max_sequence, int total_tokens, int heads, int packed);

/* No counterpart in the reference (mla_prefill_backward_workspace_bytes). */
size_t dscuda_mla_prefill_backward_workspace_bytes(
    int batch, int max_sequence, int total_tokens, int heads);

/* No counterpart in the reference (mla_prefill_backward_cuda). */
int dscuda_mla_prefill_backward(
    void* dq, void* dk_nope, void* dk_pe, void* dv,
    const void* dout, const void* output, const float* lse,
    const void* q_nope, const void* q_pe, const void* k_nope, const void* k_pe, const void* v,
    const int* cu_seqlens, void* workspace,
    int batch, int max_sequence, int total_tokens, int heads,
    int nope, int rope, int value, float scale, void* stream);

/* No counterpart in the reference (include/mla.h, mla_up_project_cuda): k_nope [rows,H,128] =
 * kv_latent [rows,512] W_UK^T and v = kv_latent W_UV^T, weights [H*128,512]; k_nope or v may be NULL. */
int dscuda_mla_up_project(
    void* k_nope, void* v, const void* kv_latent, const void* w_uk, const void* w_uv,
    long long rows, int heads, void* stream);

/* No counterpart in the reference (mla_absorb_query_cuda): q_latent [rows,H,512] = q_nope [rows,H,128] W_UK[h]. */
int dscuda_mla_absorb_query(
    void* q_latent, const void* q_nope, const void* w_uk, long long rows, int heads, void* stream);

/* No counterpart in the reference (mla_unabsorb_output_cuda): out [rows,H,128] = o_latent [rows,H,512] W_UV[h]^T. */
int dscuda_mla_unabsorb_output(
    void* output, const void* output_latent, const void* w_uv, long long rows, int heads, void* stream);

/* No counterpart in the reference: sticky device status of the MLA kernels
 * (0 fine, 1 a bounded in-kernel wait ran out, 2 misaligned shared memory, 3 a
 * cache append skipped, or a checked decode replaced, an index outside the cache).  Synchronises the device. */
int dscuda_mla_device_status(int reset);

/* reference: benchmarks/bindings/flash_attention_bridge.cu:13 */
const char* dscuda_flash_last_error(void);

/* reference: benchmarks/bindings/flash_attention_bridge.cu:17-20 ([P]*5+[I]*5+[F,P],
 * benchmarks/flash_attention.py:37). */
int dscuda_flash_forward(
    void* output, float* lse, const void* query, const void* key, const void* value,
    int batch, int sequence, int query_heads, int key_value_heads, int dimension,
    float scale, void* stream);

/* No counterpart in the reference: device status of the flash kernel. */
int dscuda_flash_device_status(int reset);

#ifdef __cplusplus
}
#endif

#endif /* DSCUDA_C_API_H */
