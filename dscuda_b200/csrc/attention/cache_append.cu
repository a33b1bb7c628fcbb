// Appends new tokens to the paged latent cache the decode kernel reads.
//
// The cache layout is the one reference/python/mla.py:11-23 (pack_cache) builds:
// [blocks, page_size, 1, 576] bf16, a token's row being its 512 latent values
// followed by its 64 rotary key values, and a block table [B, pages] of physical
// page numbers.  The reference only ever packs a whole tensor on the host; a
// serving loop writes the rows of the tokens it has just computed, which is what
// this kernel does: token t of sequence b goes to position start[b] + t, i.e.
// page block_table[b][position / page_size], slot position % page_size.
//
// One warp per token: 72 16-byte units are read from the two sources and written
// as one contiguous 1152-byte row.  The kernel is bound by HBM (1152 bytes read
// and 1152 written per token).  A page number or position outside the cache is
// never written; it raises the sticky status word instead.
#include "mla.h"
#include "cuda_common.h"
#include "attention_internal.h"
#include "sm100_primitives.cuh"

#include <cstdint>
#include <stdexcept>

namespace dscuda {
namespace {

constexpr int ROW_UNITS = (MLA_KV_RANK + MLA_ROPE_SIZE) * 2 / 16;      // 72
constexpr int LATENT_UNITS = MLA_KV_RANK * 2 / 16;                     // 64
constexpr int ROPE_UNITS = MLA_ROPE_SIZE * 2 / 16;                     // 8
constexpr int APPEND_THREADS = 256;

__device__ int append_status = 0;

__global__ void __launch_bounds__(APPEND_THREADS) cache_append_kernel(uint4* cache, const uint4* latent, const uint4* rope, const int* block_table,
                                                                      const int* start_positions, const int* token_counts, int batch,
                                                                      int tokens, int page_size, int pages, int cache_blocks) {
    const int lane = threadIdx.x % 32;
    const long long warps = static_cast<long long>(gridDim.x) * (APPEND_THREADS / 32);
    const long long total = static_cast<long long>(batch) * tokens;
    for (long long item = static_cast<long long>(blockIdx.x) * (APPEND_THREADS / 32) + threadIdx.x / 32; item < total; item += warps) {
        const int b = static_cast<int>(item / tokens);
        const int t = static_cast<int>(item % tokens);
        if (token_counts != nullptr && t >= token_counts[b]) {
            continue;
        }
        const long long position = (start_positions != nullptr ? start_positions[b] : 0) + static_cast<long long>(t);
        const long long logical_page = position / page_size;
        if (position < 0 || logical_page >= pages) {
            if (lane == 0) {
                atomicExch(&append_status, sm100::STATUS_BAD_INDEX);
            }
            continue;
        }
        const int physical_page = block_table[static_cast<long long>(b) * pages + logical_page];
        if (physical_page < 0 || physical_page >= cache_blocks) {
            if (lane == 0) {
                atomicExch(&append_status, sm100::STATUS_BAD_INDEX);
            }
            continue;
        }
        uint4* dst = cache + (static_cast<long long>(physical_page) * page_size + position % page_size) * ROW_UNITS;
        const uint4* src_latent = latent + item * LATENT_UNITS;
        const uint4* src_rope = rope + item * ROPE_UNITS;
        const uint4 first = __ldg(src_latent + lane);
        const uint4 second = __ldg(src_latent + 32 + lane);
        uint4 third = make_uint4(0, 0, 0, 0);
        if (lane < ROPE_UNITS) {
            third = __ldg(src_rope + lane);
        }
        dst[lane] = first;
        dst[32 + lane] = second;
        if (lane < ROPE_UNITS) {
            dst[64 + lane] = third;
        }
    }
}

}  // namespace

namespace internal {

int append_device_status(bool reset) {
    int status = 0;
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemcpyFromSymbol(&status, append_status, sizeof(int)));
    if (reset && status != 0) {
        const int zero = 0;
        CUDA_CHECK(cudaMemcpyToSymbol(append_status, &zero, sizeof(int)));
    }
    return status;
}

}  // namespace internal

void mla_cache_append_cuda(__nv_bfloat16* paged_kv_cache, const __nv_bfloat16* kv_latent, const __nv_bfloat16* key_rope, const int* block_table,
                           const int* start_positions, const int* token_counts, int batch_size, int tokens, int kv_rank, int rope_size,
                           int page_size, int pages_per_sequence, int cache_blocks, cudaStream_t stream) {
    if (kv_rank != MLA_KV_RANK || rope_size != MLA_ROPE_SIZE) {
        throw std::invalid_argument("MLA requires KV rank 512 and RoPE size 64");
    }
    if (batch_size <= 0 || tokens <= 0 || page_size <= 0 || pages_per_sequence <= 0 || cache_blocks <= 0) {
        throw std::invalid_argument("MLA cache append requires positive batch, tokens, page size, pages per sequence and cache blocks");
    }
    for (const void* pointer : {static_cast<const void*>(paged_kv_cache), static_cast<const void*>(kv_latent), static_cast<const void*>(key_rope),
                                static_cast<const void*>(block_table)}) {
        if (pointer == nullptr) {
            throw std::invalid_argument("null tensor pointer");
        }
    }
    for (const void* pointer : {static_cast<const void*>(paged_kv_cache), static_cast<const void*>(kv_latent), static_cast<const void*>(key_rope)}) {
        if ((reinterpret_cast<std::uintptr_t>(pointer) & 15U) != 0) {
            throw std::invalid_argument("tensor pointers must be 16-byte aligned");
        }
    }
    const long long total = static_cast<long long>(batch_size) * tokens;
    const long long wanted = (total + APPEND_THREADS / 32 - 1) / (APPEND_THREADS / 32);
    const unsigned blocks = static_cast<unsigned>(wanted < 148LL * 8 ? wanted : 148LL * 8);      // 8 resident CTAs on each of 148 SMs
    cache_append_kernel<<<blocks, APPEND_THREADS, 0, stream>>>(reinterpret_cast<uint4*>(paged_kv_cache), reinterpret_cast<const uint4*>(kv_latent),
                                                               reinterpret_cast<const uint4*>(key_rope), block_table, start_positions, token_counts,
                                                               batch_size, tokens, page_size, pages_per_sequence, cache_blocks);
    CUDA_CHECK(cudaGetLastError());
}

}  // namespace dscuda
