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

#include <cuda_fp8.h>

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

// ---------------------------------------------------------------------------
// FP8 variant of the cache.  The reference is unquantised (reference/python/sources.json:2 names
// FP8 as what the official decode library adds); this is the storage format and the two kernels
// around it.  A token's row is 656 bytes: the 512 latent values as e4m3, one fp32 scale per 128
// columns (value = e4m3 * scale, scale = max|x| of the group / 448, or 1 for an all-zero group), and
// the 64 rotary values unchanged in bf16: 57 % of the bf16 row.
//
//   cache_append_fp8_kernel      quantises and writes new tokens' rows (same addressing as above);
//   cache_dequantize_fp8_kernel  rewrites a range of physical rows in the bf16 layout the decode
//                                kernel reads.
// One warp per token in both: a lane owns 16 latent columns (one 16-byte unit of e4m3), eight lanes
// own a scale group.
// ---------------------------------------------------------------------------
constexpr int FP8_ROW_BYTES = MLA_FP8_CACHE_ROW_BYTES;                  // 656
constexpr int FP8_SCALES_OFFSET = MLA_KV_RANK;                          // 512: four fp32 scales
constexpr int FP8_ROPE_OFFSET = MLA_KV_RANK + 16;                       // 528: 64 bf16
static_assert(FP8_ROW_BYTES == FP8_ROPE_OFFSET + MLA_ROPE_SIZE * 2 && FP8_ROW_BYTES % 16 == 0, "FP8 cache row layout");

__global__ void __launch_bounds__(APPEND_THREADS) cache_append_fp8_kernel(uint8_t* cache, const uint4* latent, const uint4* rope, const int* block_table,
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
        uint8_t* dst = cache + (static_cast<long long>(physical_page) * page_size + position % page_size) * FP8_ROW_BYTES;
        // 16 latent columns per lane: two 16-byte units of bf16
        const uint4 raw[2] = {__ldg(latent + item * LATENT_UNITS + 2 * lane), __ldg(latent + item * LATENT_UNITS + 2 * lane + 1)};
        float values[16];
        const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(raw);
        float amax = 0.0F;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float2 x = __bfloat1622float2(pairs[e]);
            values[2 * e] = x.x;
            values[2 * e + 1] = x.y;
            amax = fmaxf(amax, fmaxf(fabsf(x.x), fabsf(x.y)));
        }
#pragma unroll
        for (int offset = 4; offset > 0; offset >>= 1) {          // the eight lanes of a 128-column group
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffU, amax, offset));
        }
        const float scale = amax > 0.0F ? amax / 448.0F : 1.0F;
        uint32_t packed[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(values[4 * e] / scale, values[4 * e + 1] / scale), __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(values[4 * e + 2] / scale, values[4 * e + 3] / scale), __NV_SATFINITE, __NV_E4M3);
            packed[e] = lo | (hi << 16);
        }
        reinterpret_cast<uint4*>(dst)[lane] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        if ((lane & 7) == 0) {
            reinterpret_cast<float*>(dst + FP8_SCALES_OFFSET)[lane >> 3] = scale;
        }
        if (lane < ROPE_UNITS) {
            reinterpret_cast<uint4*>(dst + FP8_ROPE_OFFSET)[lane] = __ldg(rope + item * ROPE_UNITS + lane);
        }
    }
}

__global__ void __launch_bounds__(APPEND_THREADS) cache_dequantize_fp8_kernel(uint4* bf16_cache, const uint8_t* fp8_cache, long long rows) {
    const int lane = threadIdx.x % 32;
    const long long warps = static_cast<long long>(gridDim.x) * (APPEND_THREADS / 32);
    for (long long row = static_cast<long long>(blockIdx.x) * (APPEND_THREADS / 32) + threadIdx.x / 32; row < rows; row += warps) {
        const uint8_t* src = fp8_cache + row * FP8_ROW_BYTES;
        uint4* dst = bf16_cache + row * ROW_UNITS;
        const uint4 quantised = __ldg(reinterpret_cast<const uint4*>(src) + lane);
        const float scale = __ldg(reinterpret_cast<const float*>(src + FP8_SCALES_OFFSET) + (lane >> 3));
        const uint32_t words[4] = {quantised.x, quantised.y, quantised.z, quantised.w};
        uint32_t out[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>((words[e] >> (16 * half)) & 0xffffU), __NV_E4M3);
                const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&h));
                out[2 * e + half] = sm100::pack_bf16x2(x.x * scale, x.y * scale);
            }
        }
        dst[2 * lane] = make_uint4(out[0], out[1], out[2], out[3]);
        dst[2 * lane + 1] = make_uint4(out[4], out[5], out[6], out[7]);
        if (lane < ROPE_UNITS) {
            dst[LATENT_UNITS + lane] = __ldg(reinterpret_cast<const uint4*>(src + FP8_ROPE_OFFSET) + lane);
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

void mla_cache_append_fp8_cuda(void* paged_fp8_cache, const __nv_bfloat16* kv_latent, const __nv_bfloat16* key_rope, const int* block_table,
                               const int* start_positions, const int* token_counts, int batch_size, int tokens, int kv_rank, int rope_size,
                               int page_size, int pages_per_sequence, int cache_blocks, cudaStream_t stream) {
    if (kv_rank != MLA_KV_RANK || rope_size != MLA_ROPE_SIZE) {
        throw std::invalid_argument("MLA requires KV rank 512 and RoPE size 64");
    }
    if (batch_size <= 0 || tokens <= 0 || page_size <= 0 || pages_per_sequence <= 0 || cache_blocks <= 0) {
        throw std::invalid_argument("MLA cache append requires positive batch, tokens, page size, pages per sequence and cache blocks");
    }
    for (const void* pointer : {static_cast<const void*>(paged_fp8_cache), static_cast<const void*>(kv_latent), static_cast<const void*>(key_rope)}) {
        if (pointer == nullptr || (reinterpret_cast<std::uintptr_t>(pointer) & 15U) != 0) {
            throw std::invalid_argument("tensor pointers must be non-null and 16-byte aligned");
        }
    }
    if (block_table == nullptr) {
        throw std::invalid_argument("null tensor pointer");
    }
    const long long total = static_cast<long long>(batch_size) * tokens;
    const long long wanted = (total + APPEND_THREADS / 32 - 1) / (APPEND_THREADS / 32);
    const unsigned blocks = static_cast<unsigned>(wanted < 148LL * 8 ? wanted : 148LL * 8);
    cache_append_fp8_kernel<<<blocks, APPEND_THREADS, 0, stream>>>(static_cast<uint8_t*>(paged_fp8_cache), reinterpret_cast<const uint4*>(kv_latent),
                                                                   reinterpret_cast<const uint4*>(key_rope), block_table, start_positions,
                                                                   token_counts, batch_size, tokens, page_size, pages_per_sequence, cache_blocks);
    CUDA_CHECK(cudaGetLastError());
}

void mla_cache_dequantize_fp8_cuda(__nv_bfloat16* paged_kv_cache, const void* paged_fp8_cache, long long first_row, long long rows,
                                   cudaStream_t stream) {
    if (first_row < 0 || rows <= 0) {
        throw std::invalid_argument("MLA cache dequantisation requires a non-empty range of rows");
    }
    for (const void* pointer : {static_cast<const void*>(paged_kv_cache), paged_fp8_cache}) {
        if (pointer == nullptr || (reinterpret_cast<std::uintptr_t>(pointer) & 15U) != 0) {
            throw std::invalid_argument("tensor pointers must be non-null and 16-byte aligned");
        }
    }
    const long long wanted = (rows + APPEND_THREADS / 32 - 1) / (APPEND_THREADS / 32);
    const unsigned blocks = static_cast<unsigned>(wanted < 148LL * 8 ? wanted : 148LL * 8);
    cache_dequantize_fp8_kernel<<<blocks, APPEND_THREADS, 0, stream>>>(reinterpret_cast<uint4*>(paged_kv_cache) + first_row * ROW_UNITS,
                                                                       static_cast<const uint8_t*>(paged_fp8_cache) + first_row * FP8_ROW_BYTES, rows);
    CUDA_CHECK(cudaGetLastError());
}

}  // namespace dscuda
