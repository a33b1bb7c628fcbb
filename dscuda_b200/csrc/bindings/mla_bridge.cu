// extern "C" surface of libdscuda_mla_bench.so.  Same symbols and signatures as
// the reference's benchmarks/bindings/mla_bridge.cu:12-73, plus the prefill
// entry points.  C++ exceptions stop here: they become status 1 and a
// thread-local message.
#include "mla.h"

#include <exception>
#include <string>

namespace {
thread_local std::string last_error;

template <class Call>
int guarded(Call&& call) {
    try {
        call();
        return 0;
    } catch (const std::exception& error) {
        last_error = error.what();
        return 1;
    } catch (...) {
        last_error = "unknown failure";
        return 1;
    }
}
}  // namespace

using bf16 = __nv_bfloat16;

extern "C" const char* dscuda_mla_last_error() {
    return last_error.c_str();
}

extern "C" int dscuda_mla_forward(bf16* output, float* lse, const bf16* query, const bf16* query_rope, const bf16* latent,
                                  const bf16* key_rope, int batch, int sequence, int heads, int rank, int rope, float scale,
                                  cudaStream_t stream) {
    return guarded([&] {
        dscuda::mla_compressed_attention_forward_cuda(output, lse, query, query_rope, latent, key_rope, batch, sequence, heads,
                                                      rank, rope, scale, stream);
    });
}

extern "C" int dscuda_mla_backward(bf16* dquery, bf16* dquery_rope, bf16* dlatent, bf16* dkey_rope, const bf16* dout,
                                   const bf16* output, const float* lse, const bf16* query, const bf16* query_rope,
                                   const bf16* latent, const bf16* key_rope, int batch, int sequence, int heads, int rank,
                                   int rope, float scale, cudaStream_t stream) {
    return guarded([&] {
        dscuda::mla_compressed_attention_backward_cuda(dquery, dquery_rope, dlatent, dkey_rope, dout, output, lse, query,
                                                       query_rope, latent, key_rope, batch, sequence, heads, rank, rope, scale,
                                                       stream);
    });
}

extern "C" std::size_t dscuda_mla_workspace_elements(int batch, int heads, int splits, int rank) {
    return dscuda::mla_decode_workspace_elements(batch, heads, splits, rank);
}

extern "C" int dscuda_mla_decode(bf16* output, float* lse, const bf16* query, const bf16* paged_cache, const int* block_table,
                                 const int* lengths, float* workspace, int batch, int heads, int rank, int rope, int page_size,
                                 int pages, int splits, float scale, cudaStream_t stream) {
    return guarded([&] {
        dscuda::mla_decode_forward_cuda(output, lse, query, paged_cache, block_table, lengths, workspace, batch, heads, rank, rope,
                                        page_size, pages, splits, scale, stream);
    });
}

extern "C" int dscuda_mla_decode_checked(bf16* output, float* lse, const bf16* query, const bf16* paged_cache, const int* block_table,
                                         const int* lengths, float* workspace, int batch, int heads, int rank, int rope, int page_size,
                                         int pages, int cache_blocks, int splits, float scale, cudaStream_t stream) {
    return guarded([&] {
        dscuda::mla_decode_forward_checked_cuda(output, lse, query, paged_cache, block_table, lengths, workspace, batch, heads, rank,
                                                rope, page_size, pages, cache_blocks, splits, scale, stream);
    });
}

extern "C" std::size_t dscuda_mla_decode_static_capacity() {
    return dscuda::mla_decode_static_capacity();
}

extern "C" int dscuda_mla_decode_static(bf16* output, float* lse, const bf16* query, const bf16* paged_cache, const int* block_table,
                                        const int* lengths, int batch, int heads, int rank, int rope, int page_size, int pages,
                                        int splits, float scale, cudaStream_t stream) {
    return guarded([&] {
        dscuda::mla_decode_forward_static_cuda(output, lse, query, paged_cache, block_table, lengths, batch, heads, rank, rope,
                                               page_size, pages, splits, scale, stream);
    });
}

extern "C" int dscuda_mla_cache_append(bf16* paged_cache, const bf16* latent, const bf16* key_rope, const int* block_table,
                                       const int* start_positions, const int* token_counts, int batch, int tokens, int rank, int rope,
                                       int page_size, int pages, int cache_blocks, cudaStream_t stream) {
    return guarded([&] {
        dscuda::mla_cache_append_cuda(paged_cache, latent, key_rope, block_table, start_positions, token_counts, batch, tokens, rank, rope,
                                      page_size, pages, cache_blocks, stream);
    });
}

extern "C" int dscuda_mla_cache_append_fp8(void* paged_fp8_cache, const bf16* latent, const bf16* key_rope, const int* block_table,
                                           const int* start_positions, const int* token_counts, int batch, int tokens, int rank, int rope,
                                           int page_size, int pages, int cache_blocks, cudaStream_t stream) {
    return guarded([&] {
        dscuda::mla_cache_append_fp8_cuda(paged_fp8_cache, latent, key_rope, block_table, start_positions, token_counts, batch, tokens, rank, rope,
                                          page_size, pages, cache_blocks, stream);
    });
}

extern "C" int dscuda_mla_cache_dequantize_fp8(bf16* paged_cache, const void* paged_fp8_cache, long long first_row, long long rows,
                                               cudaStream_t stream) {
    return guarded([&] { dscuda::mla_cache_dequantize_fp8_cuda(paged_cache, paged_fp8_cache, first_row, rows, stream); });
}

extern "C" int dscuda_mla_rope_apply(bf16* q_pe, bf16* k_pe, const int* positions, long long rows, int heads, int sequence_length, int rope,
                                     float theta, cudaStream_t stream) {
    return guarded([&] { dscuda::mla_rope_apply_cuda(q_pe, k_pe, positions, rows, heads, sequence_length, rope, theta, stream); });
}

extern "C" int dscuda_mla_prefill_forward(bf16* output, float* lse, const bf16* q_nope, const bf16* q_pe, const bf16* k_nope,
                                          const bf16* k_pe, const bf16* v, const int* cu_seqlens, int batch, int max_sequence,
                                          int total_tokens, int heads, int nope, int rope, int value, float scale,
                                          cudaStream_t stream) {
    return guarded([&] {
        dscuda::mla_prefill_forward_cuda(output, lse, q_nope, q_pe, k_nope, k_pe, v, cu_seqlens, batch, max_sequence, total_tokens,
                                         heads, nope, rope, value, scale, stream);
    });
}

extern "C" std::size_t dscuda_mla_prefill_backward_scratch_limit(long long bytes) {
    return dscuda::mla_prefill_backward_scratch_limit(bytes);
}

extern "C" int dscuda_mla_prefill_backward_launches(int batch, int max_sequence, int total_tokens, int heads, int packed) {
    return dscuda::mla_prefill_backward_launches(batch, max_sequence, total_tokens, heads, packed != 0);
}

extern "C" std::size_t dscuda_mla_prefill_backward_workspace_bytes(int batch, int max_sequence, int total_tokens, int heads) {
    return dscuda::mla_prefill_backward_workspace_bytes(batch, max_sequence, total_tokens, heads);
}

extern "C" int dscuda_mla_prefill_backward(bf16* dq, bf16* dk_nope, bf16* dk_pe, bf16* dv, const bf16* dout, const bf16* output,
                                           const float* lse, const bf16* q_nope, const bf16* q_pe, const bf16* k_nope,
                                           const bf16* k_pe, const bf16* v, const int* cu_seqlens, void* workspace, int batch,
                                           int max_sequence, int total_tokens, int heads, int nope, int rope, int value,
                                           float scale, cudaStream_t stream) {
    return guarded([&] {
        dscuda::mla_prefill_backward_cuda(dq, dk_nope, dk_pe, dv, dout, output, lse, q_nope, q_pe, k_nope, k_pe, v, cu_seqlens,
                                          workspace, batch, max_sequence, total_tokens, heads, nope, rope, value, scale, stream);
    });
}

extern "C" int dscuda_mla_up_project(bf16* k_nope, bf16* v, const bf16* kv_latent, const bf16* w_uk, const bf16* w_uv, long long rows, int heads,
                                     cudaStream_t stream) {
    return guarded([&] { dscuda::mla_up_project_cuda(k_nope, v, kv_latent, w_uk, w_uv, rows, heads, stream); });
}

extern "C" int dscuda_mla_absorb_query(bf16* q_latent, const bf16* q_nope, const bf16* w_uk, long long rows, int heads, cudaStream_t stream) {
    return guarded([&] { dscuda::mla_absorb_query_cuda(q_latent, q_nope, w_uk, rows, heads, stream); });
}

extern "C" int dscuda_mla_unabsorb_output(bf16* output, const bf16* output_latent, const bf16* w_uv, long long rows, int heads,
                                          cudaStream_t stream) {
    return guarded([&] { dscuda::mla_unabsorb_output_cuda(output, output_latent, w_uv, rows, heads, stream); });
}

extern "C" int dscuda_mla_device_status(int reset) {
    int status = -1;
    if (guarded([&] { status = dscuda::mla_device_status(reset != 0); }) != 0) {
        return -1;
    }
    return status;
}

