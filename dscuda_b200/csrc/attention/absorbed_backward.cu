// Backward of the absorbed-latent causal MLA forward
// (mla_compressed_attention_backward_cuda).  The interface gives no scratch
// memory and the gradients of the shared latent / rotary key sum over every
// head and every later query, so the work is split the way the reference splits
// it (kernels/attention/mla/sm89.cu:295,356): one pass owns the query-side
// rows, one pass owns the key-side rows, and each recomputes P from the saved
// LSE.  Unlike the reference, a warp (not a CTA) owns a row, the opposite side
// streams through shared memory in tiles shared by the 8 warps of a CTA, and the
// row-sum delta = dO.O is computed once per row instead of once per pair.
//
// These are CUDA-core kernels (fp32 FMA, warp-shuffle reductions): the 576-wide
// output rows leave no room in tensor memory for a tcgen05 formulation without
// scratch, and the sizes this entry point sees in the reference's harness
// (T <= 512, H <= 8) are far from tensor-bound.
#include "mla.h"
#include "cuda_common.h"
#include "attention_internal.h"

#include <cstdint>
#include <stdexcept>

namespace dscuda {
namespace {

constexpr int RANK = MLA_KV_RANK;       // 512
constexpr int ROPE = MLA_ROPE_SIZE;     // 64
constexpr int WIDTH = RANK + ROPE;      // 576
constexpr int PAIRS = WIDTH / 64;       // 9 bf16 pairs per lane: pair i covers columns 64*i + 2*lane, +1
constexpr int LATENT_PAIRS = RANK / 64; // the first 8 pairs are latent (they double as V), the last is rotary
constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int KEY_TILE = 32;            // keys staged per step in the query-side kernel
constexpr int ROW_TILE = 16;            // (token, head) rows staged per step in the key-side kernel

__device__ __forceinline__ float warp_sum(float value) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        value += __shfl_xor_sync(0xffffffffU, value, offset);
    }
    return value;
}

__device__ __forceinline__ float2 load_pair(const __nv_bfloat16* base) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(base));
}

// Loads the 9 column pairs of one 576-wide row whose latent and rotary parts
// live in two tensors.
__device__ __forceinline__ void load_row(float2 (&dst)[PAIRS], const __nv_bfloat16* latent_row, const __nv_bfloat16* rope_row, int lane) {
#pragma unroll
    for (int i = 0; i < LATENT_PAIRS; ++i) {
        dst[i] = load_pair(latent_row + 64 * i + 2 * lane);
    }
    dst[LATENT_PAIRS] = load_pair(rope_row + 2 * lane);
}

// ---------------------------------------------------------------------------
// Query side: one warp per (token, head) row.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS) absorbed_backward_query_kernel(
    __nv_bfloat16* dq_latent, __nv_bfloat16* dq_rope, const __nv_bfloat16* dout, const __nv_bfloat16* out, const float* lse,
    const __nv_bfloat16* q_latent, const __nv_bfloat16* q_rope, const __nv_bfloat16* kv_latent, const __nv_bfloat16* k_rope,
    int sequence, int heads, float scale) {
    __shared__ __align__(16) __nv_bfloat16 keys[KEY_TILE][WIDTH];
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const int b = blockIdx.y;
    const int rows = sequence * heads;
    const int first_row = blockIdx.x * WARPS;
    const int row = first_row + warp;
    const bool active = row < rows;
    const int token = active ? row / heads : 0;
    const int head = active ? row % heads : 0;
    const int last_token = min(rows - 1, first_row + WARPS - 1) / heads;   // furthest key any warp of the CTA needs

    float2 q[PAIRS], grad[PAIRS], d_out[LATENT_PAIRS];
    float delta = 0.0F, row_lse = 0.0F;
#pragma unroll
    for (int i = 0; i < PAIRS; ++i) {
        q[i] = make_float2(0.0F, 0.0F);
        grad[i] = make_float2(0.0F, 0.0F);
    }
    if (active) {
        const size_t global_row = static_cast<size_t>(b) * rows + row;
        load_row(q, q_latent + global_row * RANK, q_rope + global_row * ROPE, lane);
        float partial = 0.0F;
#pragma unroll
        for (int i = 0; i < LATENT_PAIRS; ++i) {
            d_out[i] = load_pair(dout + global_row * RANK + 64 * i + 2 * lane);
            const float2 o = load_pair(out + global_row * RANK + 64 * i + 2 * lane);
            partial += d_out[i].x * o.x + d_out[i].y * o.y;
        }
        delta = warp_sum(partial);
        row_lse = lse[(static_cast<size_t>(b) * heads + head) * sequence + token];
    } else {
#pragma unroll
        for (int i = 0; i < LATENT_PAIRS; ++i) {
            d_out[i] = make_float2(0.0F, 0.0F);
        }
    }

    for (int key0 = 0; key0 <= last_token; key0 += KEY_TILE) {
        const int tile_keys = min(KEY_TILE, last_token + 1 - key0);
        __syncthreads();
        // stage [tile_keys x 576] as 16-byte vectors: 64 per latent row, 8 per rotary row
        for (int index = threadIdx.x; index < tile_keys * 72; index += THREADS) {
            const int k = index / 72;
            const int v = index % 72;
            const size_t key_row = static_cast<size_t>(b) * sequence + key0 + k;
            const uint4 value = v < 64 ? reinterpret_cast<const uint4*>(kv_latent + key_row * RANK)[v]
                                       : reinterpret_cast<const uint4*>(k_rope + key_row * ROPE)[v - 64];
            reinterpret_cast<uint4*>(&keys[k][0])[v] = value;
        }
        __syncthreads();
        const int visible = active ? min(tile_keys, token + 1 - key0) : 0;     // causal: key <= token
        for (int k = 0; k < visible; ++k) {
            float2 kv[PAIRS];
            float s = 0.0F, dp = 0.0F;
#pragma unroll
            for (int i = 0; i < PAIRS; ++i) {
                kv[i] = load_pair(&keys[k][64 * i + 2 * lane]);
                s += q[i].x * kv[i].x + q[i].y * kv[i].y;
            }
#pragma unroll
            for (int i = 0; i < LATENT_PAIRS; ++i) {
                dp += d_out[i].x * kv[i].x + d_out[i].y * kv[i].y;
            }
            s = warp_sum(s);
            dp = warp_sum(dp);
            const float probability = __expf(s * scale - row_lse);
            const float ds = probability * (dp - delta) * scale;
#pragma unroll
            for (int i = 0; i < PAIRS; ++i) {
                grad[i].x += ds * kv[i].x;
                grad[i].y += ds * kv[i].y;
            }
        }
    }
    if (active) {
        const size_t global_row = static_cast<size_t>(b) * rows + row;
#pragma unroll
        for (int i = 0; i < LATENT_PAIRS; ++i) {
            *reinterpret_cast<__nv_bfloat162*>(dq_latent + global_row * RANK + 64 * i + 2 * lane) = __float22bfloat162_rn(grad[i]);
        }
        *reinterpret_cast<__nv_bfloat162*>(dq_rope + global_row * ROPE + 2 * lane) = __float22bfloat162_rn(grad[LATENT_PAIRS]);
    }
}

// ---------------------------------------------------------------------------
// Key side: one warp per key; every (token >= key, head) row contributes.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS) absorbed_backward_key_kernel(
    __nv_bfloat16* dkv_latent, __nv_bfloat16* dk_rope, const __nv_bfloat16* dout, const __nv_bfloat16* out, const float* lse,
    const __nv_bfloat16* q_latent, const __nv_bfloat16* q_rope, const __nv_bfloat16* kv_latent, const __nv_bfloat16* k_rope,
    int sequence, int heads, float scale) {
    __shared__ __align__(16) __nv_bfloat16 queries[ROW_TILE][WIDTH];
    __shared__ __align__(16) __nv_bfloat16 gradients[ROW_TILE][RANK];
    __shared__ float row_lse[ROW_TILE];
    __shared__ float row_delta[ROW_TILE];
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const int b = blockIdx.y;
    const int rows = sequence * heads;
    const int first_key = blockIdx.x * WARPS;
    const int key = first_key + warp;
    const bool active = key < sequence;

    float2 kv[PAIRS], grad[PAIRS];
#pragma unroll
    for (int i = 0; i < PAIRS; ++i) {
        kv[i] = make_float2(0.0F, 0.0F);
        grad[i] = make_float2(0.0F, 0.0F);
    }
    if (active) {
        const size_t key_row = static_cast<size_t>(b) * sequence + key;
        load_row(kv, kv_latent + key_row * RANK, k_rope + key_row * ROPE, lane);
    }

    for (int row0 = first_key * heads; row0 < rows; row0 += ROW_TILE) {
        const int tile_rows = min(ROW_TILE, rows - row0);
        __syncthreads();
        // each warp stages two rows and computes their delta on the way
        for (int r = warp; r < tile_rows; r += WARPS) {
            const int row = row0 + r;
            const size_t global_row = static_cast<size_t>(b) * rows + row;
            float partial = 0.0F;
#pragma unroll
            for (int i = 0; i < LATENT_PAIRS; ++i) {
                const __nv_bfloat162 qv = *reinterpret_cast<const __nv_bfloat162*>(q_latent + global_row * RANK + 64 * i + 2 * lane);
                const __nv_bfloat162 gv = *reinterpret_cast<const __nv_bfloat162*>(dout + global_row * RANK + 64 * i + 2 * lane);
                const float2 o = load_pair(out + global_row * RANK + 64 * i + 2 * lane);
                const float2 g = __bfloat1622float2(gv);
                partial += g.x * o.x + g.y * o.y;
                *reinterpret_cast<__nv_bfloat162*>(&queries[r][64 * i + 2 * lane]) = qv;
                *reinterpret_cast<__nv_bfloat162*>(&gradients[r][64 * i + 2 * lane]) = gv;
            }
            *reinterpret_cast<__nv_bfloat162*>(&queries[r][RANK + 2 * lane]) =
                *reinterpret_cast<const __nv_bfloat162*>(q_rope + global_row * ROPE + 2 * lane);
            partial = warp_sum(partial);
            if (lane == 0) {
                row_delta[r] = partial;
                row_lse[r] = lse[(static_cast<size_t>(b) * heads + row % heads) * sequence + row / heads];
            }
        }
        __syncthreads();
        if (!active) {
            continue;
        }
        for (int r = 0; r < tile_rows; ++r) {
            const int token = (row0 + r) / heads;
            if (token < key) {          // causal: this query does not see the key
                continue;
            }
            float2 qv[PAIRS], gv[LATENT_PAIRS];
            float s = 0.0F, dp = 0.0F;
#pragma unroll
            for (int i = 0; i < PAIRS; ++i) {
                qv[i] = load_pair(&queries[r][64 * i + 2 * lane]);
                s += qv[i].x * kv[i].x + qv[i].y * kv[i].y;
            }
#pragma unroll
            for (int i = 0; i < LATENT_PAIRS; ++i) {
                gv[i] = load_pair(&gradients[r][64 * i + 2 * lane]);
                dp += gv[i].x * kv[i].x + gv[i].y * kv[i].y;
            }
            s = warp_sum(s);
            dp = warp_sum(dp);
            const float probability = __expf(s * scale - row_lse[r]);
            const float ds = probability * (dp - row_delta[r]) * scale;
#pragma unroll
            for (int i = 0; i < LATENT_PAIRS; ++i) {
                // score path plus value path (the latent is both K and V)
                grad[i].x += ds * qv[i].x + probability * gv[i].x;
                grad[i].y += ds * qv[i].y + probability * gv[i].y;
            }
            grad[LATENT_PAIRS].x += ds * qv[LATENT_PAIRS].x;
            grad[LATENT_PAIRS].y += ds * qv[LATENT_PAIRS].y;
        }
    }
    if (active) {
        const size_t key_row = static_cast<size_t>(b) * sequence + key;
#pragma unroll
        for (int i = 0; i < LATENT_PAIRS; ++i) {
            *reinterpret_cast<__nv_bfloat162*>(dkv_latent + key_row * RANK + 64 * i + 2 * lane) = __float22bfloat162_rn(grad[i]);
        }
        *reinterpret_cast<__nv_bfloat162*>(dk_rope + key_row * ROPE + 2 * lane) = __float22bfloat162_rn(grad[LATENT_PAIRS]);
    }
}

}  // namespace

void mla_compressed_attention_backward_cuda(__nv_bfloat16* query_latent_gradient, __nv_bfloat16* query_rope_gradient,
                                            __nv_bfloat16* kv_latent_gradient, __nv_bfloat16* key_rope_gradient,
                                            const __nv_bfloat16* output_gradient, const __nv_bfloat16* output, const float* logsumexp,
                                            const __nv_bfloat16* query_latent, const __nv_bfloat16* query_rope,
                                            const __nv_bfloat16* kv_latent, const __nv_bfloat16* key_rope, int batch_size,
                                            int sequence_length, int heads, int kv_rank, int rope_size, float scale, cudaStream_t stream) {
    // kernels/attention/mla/sm89.cu:20-24 of the reference: same condition, same message.
    if (kv_rank != MLA_KV_RANK || rope_size != MLA_ROPE_SIZE) {
        throw std::invalid_argument("MLA requires C=512 and RoPE=64");
    }
    if (batch_size <= 0 || sequence_length <= 0 || heads <= 0) {
        throw std::invalid_argument("MLA backward requires positive batch, sequence length and heads");
    }
    if (batch_size > 65535 || static_cast<long long>(sequence_length) * heads * batch_size > 0x7fffffffLL) {
        throw std::invalid_argument("MLA backward shape exceeds the supported index range");
    }
    for (const void* pointer : {static_cast<const void*>(query_latent_gradient), static_cast<const void*>(query_rope_gradient),
                                static_cast<const void*>(kv_latent_gradient), static_cast<const void*>(key_rope_gradient),
                                static_cast<const void*>(output_gradient), static_cast<const void*>(output),
                                static_cast<const void*>(logsumexp), static_cast<const void*>(query_latent),
                                static_cast<const void*>(query_rope), static_cast<const void*>(kv_latent),
                                static_cast<const void*>(key_rope)}) {
        if (pointer == nullptr) {
            throw std::invalid_argument("null tensor pointer");
        }
        if ((reinterpret_cast<std::uintptr_t>(pointer) & 15U) != 0) {
            throw std::invalid_argument("tensor pointers must be 16-byte aligned");
        }
    }
    const int rows = sequence_length * heads;
    absorbed_backward_query_kernel<<<dim3((rows + WARPS - 1) / WARPS, batch_size), THREADS, 0, stream>>>(
        query_latent_gradient, query_rope_gradient, output_gradient, output, logsumexp, query_latent, query_rope, kv_latent, key_rope,
        sequence_length, heads, scale);
    CUDA_CHECK(cudaGetLastError());
    absorbed_backward_key_kernel<<<dim3((sequence_length + WARPS - 1) / WARPS, batch_size), THREADS, 0, stream>>>(
        kv_latent_gradient, key_rope_gradient, output_gradient, output, logsumexp, query_latent, query_rope, kv_latent, key_rope,
        sequence_length, heads, scale);
    CUDA_CHECK(cudaGetLastError());
}

}  // namespace dscuda
