// Backward of the non-absorbed causal MLA attention for sm_100a.
//
// One call launches, on the caller's stream:
//   1. delta_kernel:          delta[q] = sum_d dO[q,d] * O[q,d]            (fp32, LSE layout);
//   then, for one group of heads after the other (as many heads as the dS scratch holds),
//   2. backward_dkdv_kernel:  per 128-key tile, over 64-query tiles
//                             S^T = K Q^T, dP^T = V dO^T (tcgen05, fp32 in tensor memory),
//                             P^T = exp(S^T*scale - LSE), dS^T = P^T (dP^T - delta) scale (one thread
//                             per key, bf16 back into tensor memory as the A operands),
//                             dV += P^T dO, dK += dS^T Q; the rotary 64 columns of dK go, per head
//                             and in fp32, to the workspace; dS^T goes to the scratch as well;
//   3. backward_dq_stream_kernel: per 256 query rows, dQ = dS K streamed from the scratch: nothing is
//                             recomputed, the kernel is bound by reading dS once from HBM;
//   and finally
//   4. sum_dk_pe_kernel:      the per-head dk_pe contributions added in head order -> the fp32 sums
//                             at the start of the workspace and bf16 dk_pe.
//
// A single fused kernel does not fit: dV (128) + dK (192) + the score tiles fill the 512 tensor-memory
// columns, so a dQ accumulator has no room, and adding dQ partials into global memory instead costs
// more than writing dS once and reading it back (measured; see build/probe_dq_reduction).  Every
// gradient is a plain single-writer store, so results are bit-identical from call to call.
//
// When the caller leaves no room for the scratch (mla_prefill_backward_scratch_limit), step 2 runs
// without the dS output and backward_dq_kernel takes the place of step 3: per 128-row query tile it
// recomputes S = Q K^T and dP = dO V^T over 128-key tiles and accumulates dQ += dS K.
//
// Key-side and recomputing kernels: warps 0-7 are the softmax threads (all 256 on the same tile,
// two per row), warp 8 issues the MMAs (the whole warp runs the loop, one elected lane executes the
// instruction), warp 9 loads with TMA.  Every wait is bounded.
#include "mla.h"
#include "cuda_common.h"
#include "attention_internal.h"
#include "sm100_primitives.cuh"
#include "../common/tensor_map.h"

#include <atomic>
#include <cstddef>
#include <stdexcept>

namespace dscuda {
namespace {

using namespace sm100;

constexpr int BIG = 128;                     // rows of the stationary tile (TMEM lanes)
constexpr int SUB = 64;                      // rows of the streamed tile
constexpr int BIG_CHUNK = BIG * 128;         // 16 KB: [128 rows x 64 bf16]
constexpr int SUB_CHUNK = SUB * 128;         //  8 KB: [64 rows x 64 bf16]
constexpr int STAGES = 3;
constexpr int STAGE_BYTES = 5 * SUB_CHUNK;   // 3 chunks of QK width + 2 chunks of V width
constexpr int RESIDENT_BYTES = 5 * BIG_CHUNK;
constexpr int MISC_BYTES = 2048;
constexpr int DS_TILE_BYTES = BIG * SUB * 2;  // one [128 keys x 64 queries] bf16 tile of dS^T in the scratch
constexpr int SMEM_BYTES = RESIDENT_BYTES + STAGES * STAGE_BYTES + MISC_BYTES + 1024;
constexpr int THREADS = 320;
constexpr int MMA_WARP = 8;
constexpr int LOAD_WARP = 9;
constexpr int TMEM_COLUMNS = 512;
constexpr float LOG2E = 1.4426950408889634F;

__device__ int backward_status = 0;

struct BackwardParams {
    // 128-row boxes (stationary tiles) and 64-row boxes (streamed tiles) of the same tensors
    CUtensorMap q_main_big, q_pe_big, k_main_big, k_pe_big, v_big, do_big;
    CUtensorMap q_main_sub, q_pe_sub, k_main_sub, k_pe_sub, v_sub, do_sub;
    __nv_bfloat16* dq;        // [rows, H, 192]
    __nv_bfloat16* dk_nope;   // [rows, H, 128]
    __nv_bfloat16* dv;        // [rows, H, 128]
    float* dk_pe_parts;       // [rows, heads, 64] fp32: every head's dk_pe contribution, written once
    const float* lse;         // dense [B,H,S]; packed [H,total]
    const float* delta;       // same layout as lse
    // dS^T of the heads [head0, head0 + gridDim.y) goes to this scratch and dQ is computed from it by
    // backward_dq_stream_kernel.  Null: backward_dq_kernel recomputes S and dP instead.
    // The scratch is a sequence of 16 KB tiles: per head of the group, per sequence, one tile per (128-key
    // tile kt, 64-query tile qt >= 2 kt), key tile after key tile (tile kt * QT - kt * (kt - 1) + qt - 2 kt of
    // its sequence, QT = 2 * key tiles of the sequence).  Inside a tile: [8 blocks of 8 queries][128 keys][8 bf16],
    // the layout tcgen05 reads without a swizzle as an MN-major operand (8 keys x 16 bytes form a core matrix).
    CUtensorMap ds_map;       // the scratch as rows of 256 64-bit words (one 8-query block of a tile), boxes of 16 rows x 128 words
    __nv_bfloat16* ds_scratch;
    int head0;
    const int* cu_seqlens;
    int batch;
    int max_seq;
    int total;
    int heads;
    float scale;
    float scale_log2;
};

struct BackwardBarriers {
    uint64_t resident_full;
    uint64_t stage_full[STAGES];
    uint64_t stage_empty[STAGES];
    uint64_t mma_a[2];          // tensor core -> softmax group: first score tile ready
    uint64_t mma_b[2];          // tensor core -> softmax group: second score tile ready
    uint64_t soft_a[2];         // softmax group -> tensor core: first bf16 operand stored
    uint64_t soft_b[2];         // softmax group -> tensor core: second bf16 operand stored
    uint64_t final_full;
    uint32_t tmem_base;
    int abort_flag;
    alignas(16) float lse2[STAGES][SUB];     // dK/dV kernel: LSE * log2 e of the streamed queries, read 16 bytes at a time
    alignas(16) float delta[STAGES][SUB];
};
static_assert(sizeof(BackwardBarriers) <= MISC_BYTES, "barrier block too large");
static_assert(offsetof(BackwardBarriers, lse2) % 16 == 0 && offsetof(BackwardBarriers, delta) % 16 == 0 && (SUB * sizeof(float)) % 16 == 0,
              "16-byte loads of the per-query constants");

// Maps a linear block index to (sequence, block inside the sequence).  Dense:
// blockIdx.z is the batch entry.  Packed: walk cu_seqlens.  Returns false when
// the index is past the last block.
__device__ __forceinline__ bool locate_block(const BackwardParams& p, int rows_per_block, int index, int& row0, int& length,
                                             int& block, int& blocks_in_sequence, size_t& lse_offset, int head, int* sequence_index = nullptr) {
    if (p.cu_seqlens == nullptr) {
        const int b = blockIdx.z;
        if (sequence_index != nullptr) {
            *sequence_index = b;
        }
        row0 = b * p.max_seq;
        length = p.max_seq;
        blocks_in_sequence = (length + rows_per_block - 1) / rows_per_block;
        block = index;
        lse_offset = (static_cast<size_t>(b) * p.heads + head) * p.max_seq;
        return block < blocks_in_sequence;
    }
    for (int sequence = 0; sequence < p.batch; ++sequence) {
        const int begin = p.cu_seqlens[sequence];
        const int tokens = p.cu_seqlens[sequence + 1] - begin;
        const int blocks = (tokens + rows_per_block - 1) / rows_per_block;
        if (index < blocks) {
            if (sequence_index != nullptr) {
                *sequence_index = sequence;
            }
            row0 = begin;
            length = tokens;
            block = index;
            blocks_in_sequence = blocks;
            lse_offset = static_cast<size_t>(head) * p.total + begin;
            return true;
        }
        index -= blocks;
    }
    return false;
}

// Where the dS^T tiles of `sequence` start inside one head's part of the scratch, how many tiles a head
// has in all, and the sequence's number of 128-key tiles.
struct ScratchPlace {
    long long sequence_first;
    long long head_tiles;
    int key_tiles;
};

__device__ __forceinline__ ScratchPlace scratch_place(const BackwardParams& p, int sequence) {
    ScratchPlace place = {0, 0, 0};
    if (p.cu_seqlens == nullptr) {
        const long long kt = (p.max_seq + BIG - 1) / BIG;
        place.key_tiles = static_cast<int>(kt);
        place.sequence_first = sequence * (kt * kt + kt);
        place.head_tiles = p.batch * (kt * kt + kt);
        return place;
    }
    for (int i = 0; i < p.batch; ++i) {
        const long long kt = (p.cu_seqlens[i + 1] - p.cu_seqlens[i] + BIG - 1) / BIG;
        if (i == sequence) {
            place.sequence_first = place.head_tiles;
            place.key_tiles = static_cast<int>(kt);
        }
        place.head_tiles += kt * kt + kt;
    }
    return place;
}

__device__ __forceinline__ void init_barriers(BackwardBarriers* bars, uint32_t stage_full_arrivals) {
    mbar_init(smem_u32(&bars->resident_full), 1);
    for (int i = 0; i < STAGES; ++i) {
        mbar_init(smem_u32(&bars->stage_full[i]), stage_full_arrivals);
        mbar_init(smem_u32(&bars->stage_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
        mbar_init(smem_u32(&bars->mma_a[i]), 1);
        mbar_init(smem_u32(&bars->mma_b[i]), 1);
        mbar_init(smem_u32(&bars->soft_a[i]), 2 * BIG);     // every softmax thread works on every tile
        mbar_init(smem_u32(&bars->soft_b[i]), 2 * BIG);
    }
    mbar_init(smem_u32(&bars->final_full), 1);
    bars->abort_flag = 0;
    mbar_init_fence();
}

__device__ __forceinline__ void store_bf16_row(__nv_bfloat16* dst, const uint32_t* values, int count, float factor) {
    for (int e = 0; e < count; e += 8) {
        uint4 vec;
        vec.x = pack_bf16x2(__uint_as_float(values[e]) * factor, __uint_as_float(values[e + 1]) * factor);
        vec.y = pack_bf16x2(__uint_as_float(values[e + 2]) * factor, __uint_as_float(values[e + 3]) * factor);
        vec.z = pack_bf16x2(__uint_as_float(values[e + 4]) * factor, __uint_as_float(values[e + 5]) * factor);
        vec.w = pack_bf16x2(__uint_as_float(values[e + 6]) * factor, __uint_as_float(values[e + 7]) * factor);
        *reinterpret_cast<uint4*>(dst + e) = vec;
    }
}

// ---------------------------------------------------------------------------
// delta[q] = sum_d dO[q,d] * O[q,d]; half a warp per (row, head).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) delta_kernel(float* delta, const __nv_bfloat16* dout, const __nv_bfloat16* out, const int* cu_seqlens,
                                                    int batch, int max_seq, int total, int heads) {
    const size_t pairs = static_cast<size_t>(total) * heads;
    const size_t warp_stride = static_cast<size_t>(gridDim.x) * (blockDim.x / 32);
    const int lane = threadIdx.x % 32;
    // half a warp per (row, head): 16 lanes x 16 bytes cover the 128 values of dO and of O
    const int half = lane / 16;
    const int part = lane % 16;
    for (size_t base = (static_cast<size_t>(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32) * 2; base < pairs; base += warp_stride * 2) {
        const size_t pair = base + half;
        float sum = 0.0F;
        if (pair < pairs) {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(dout + pair * 128) + part);
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(out + pair * 128) + part);
            const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 x = __bfloat1622float2(a2[e]), y = __bfloat1622float2(b2[e]);
                sum += x.x * y.x + x.y * y.y;
            }
        }
#pragma unroll
        for (int offset = 8; offset > 0; offset >>= 1) {
            sum += __shfl_xor_sync(0xffffffffU, sum, offset);
        }
        if (part == 0 && pair < pairs) {
            const size_t row = pair / heads;
            const int head = static_cast<int>(pair % heads);
            size_t index;
            if (cu_seqlens == nullptr) {
                const size_t b_index = row / max_seq;
                index = (b_index * heads + head) * max_seq + row % max_seq;
            } else {
                index = static_cast<size_t>(head) * total + row;
            }
            delta[index] = sum;
        }
    }
}

// ---------------------------------------------------------------------------
// per-head dk_pe contributions -> fp32 sums and bf16 dk_pe
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) sum_dk_pe_kernel(__nv_bfloat16* dk_pe, float* sums, const float4* parts, size_t rows, int heads) {
    // 16 threads per key row, four columns each; the heads are added in index order, so the sum
    // does not depend on how the CTAs of the key-side kernel were scheduled
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; index < rows * 16; index += stride) {
        const float4* src = parts + (index / 16) * static_cast<size_t>(heads) * 16 + index % 16;
        float4 total = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
#pragma unroll 8
        for (int h = 0; h < heads; ++h) {
            const float4 x = __ldg(src + static_cast<size_t>(h) * 16);
            total.x += x.x;
            total.y += x.y;
            total.z += x.z;
            total.w += x.w;
        }
        reinterpret_cast<float4*>(sums)[index] = total;
        reinterpret_cast<uint2*>(dk_pe)[index] = make_uint2(pack_bf16x2(total.x, total.y), pack_bf16x2(total.z, total.w));
    }
}

// ---------------------------------------------------------------------------
// dQ kernel: stationary 128 query rows, streamed 128-key tiles.
//
// Shared memory: Q (3 chunks of [128 rows x 64 bf16], 48 KB), a ring of three K
// tiles (3 chunks each, 144 KB) and one V slot (2 chunks, 32 KB) that first
// holds dO.  K(j) is read by S(j) and again by dQ(j), which runs a tile and a
// half later, hence three slots; V(j) is only read by dP(j).
// Tensor memory: S at 0..127, dP at 128..255 (dS overwrites it as bf16: keys
// 0-63 at 128..159, keys 64-127 at 192..223), dQ at 256..447, dO (bf16, an MMA
// A operand) at 448..511.
//
// Tensor-core order in steady state: S(j+1) | dQ(j) | dP(j+1).  The softmax is
// split in two stages so that one (S, dP) pair is enough: stage 1 copies S(j) to
// registers (S may then be overwritten by S(j+1)) and computes P while dQ(j-1)
// and dP(j) run; stage 2 reads dP(j), writes dS(j) while S(j+1) runs.  All 256
// softmax threads work on the same tile: thread = (row, half of the keys).
// ---------------------------------------------------------------------------
namespace dqk {
constexpr int KEYS = 128;
constexpr int CHUNK = 128 * 128;                 // [128 rows x 64 bf16], 16 KB
constexpr int Q_BYTES = 3 * CHUNK;
constexpr int K_TILE = 3 * CHUNK;
constexpr int K_SLOTS = 3;
constexpr int V_TILE = 2 * CHUNK;
constexpr int BAR_BYTES = 1024;
constexpr int SMEM_BYTES = Q_BYTES + K_SLOTS * K_TILE + V_TILE + BAR_BYTES;
constexpr uint32_t TMEM_S = 0;
constexpr uint32_t TMEM_DP = 128;
constexpr uint32_t TMEM_DQ = 256;
constexpr uint32_t TMEM_DO = 448;
static_assert(SMEM_BYTES <= 227 * 1024, "dQ kernel shared memory");

struct Barriers {
    uint64_t resident_full;     // Q and dO have landed
    uint64_t do_copied;         // 256 softmax threads: dO is in tensor memory, the V slot is free
    uint64_t k_full[K_SLOTS];
    uint64_t k_empty[K_SLOTS];
    uint64_t v_full;
    uint64_t v_empty;
    uint64_t s_full;            // tensor core -> softmax: S(j) complete
    uint64_t dp_full;           // tensor core -> softmax: dP(j) complete
    uint64_t s_free;            // 256 softmax threads: S(j) is in registers
    uint64_t ds_full;           // 256 softmax threads: dS(j) stored
    uint64_t final_full;
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(Barriers) <= BAR_BYTES, "barrier block too large");
}  // namespace dqk

__global__ void __launch_bounds__(THREADS, 1) backward_dq_kernel(const __grid_constant__ BackwardParams p) {
    using namespace dqk;
    extern __shared__ uint8_t smem_raw[];
    if (*reinterpret_cast<volatile int*>(&backward_status) != 0) {
        return;
    }
    const int head = blockIdx.y;
    int row0, length, block, blocks_in_sequence;
    size_t lse_offset;
    if (!locate_block(p, BIG, blockIdx.x, row0, length, block, blocks_in_sequence, lse_offset, head)) {
        return;
    }
    block = blocks_in_sequence - 1 - block;            // longest first
    const int q_start = block * BIG;
    const int kv_end = min(length, q_start + BIG);
    const int tile_count = (kv_end + KEYS - 1) / KEYS;

    // The layout uses all of the CTA's shared memory, so there is no room to realign: the
    // dynamic region starts 1024-byte aligned when the kernel has no static shared memory.
    const uint32_t smem_base = smem_u32(smem_raw);
    if ((smem_base & 1023U) != 0U) {
        if (threadIdx.x == 0) {
            atomicExch(&backward_status, STATUS_SMEM_MISALIGNED);
        }
        return;
    }
    const uint32_t q_smem = smem_base;
    const uint32_t k_ring = smem_base + Q_BYTES;
    const uint32_t v_smem = k_ring + K_SLOTS * K_TILE;
    Barriers* bars = reinterpret_cast<Barriers*>(smem_raw + Q_BYTES + K_SLOTS * K_TILE + V_TILE);
    volatile int* abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bars->resident_full), 1);
        mbar_init(smem_u32(&bars->do_copied), 256);
        for (int i = 0; i < K_SLOTS; ++i) {
            mbar_init(smem_u32(&bars->k_full[i]), 1);
            mbar_init(smem_u32(&bars->k_empty[i]), 1);
        }
        mbar_init(smem_u32(&bars->v_full), 1);
        mbar_init(smem_u32(&bars->v_empty), 1);
        mbar_init(smem_u32(&bars->s_full), 1);
        mbar_init(smem_u32(&bars->dp_full), 1);
        mbar_init(smem_u32(&bars->s_free), 256);
        mbar_init(smem_u32(&bars->ds_full), 256);
        mbar_init(smem_u32(&bars->final_full), 1);
        bars->abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&bars->tmem_base), TMEM_COLUMNS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

    if (warp == LOAD_WARP) {
        if (lane == 0) {
            bool alive = true;
            {
                const uint32_t bar = smem_u32(&bars->resident_full);
                mbar_arrive_expect_tx(bar, Q_BYTES + V_TILE);
                const int y = row0 + q_start;
                tma_load_2d(q_smem, &p.q_main_big, bar, head * 128, y);
                tma_load_2d(q_smem + CHUNK, &p.q_main_big, bar, head * 128 + 64, y);
                tma_load_2d(q_smem + 2 * CHUNK, &p.q_pe_big, bar, head * 64, y);
                tma_load_2d(v_smem, &p.do_big, bar, head * 128, y);
                tma_load_2d(v_smem + CHUNK, &p.do_big, bar, head * 128 + 64, y);
            }
            auto load_k = [&](int j) {
                const int slot = j % K_SLOTS;
                const int use = j / K_SLOTS;
                if (use > 0 && !mbar_wait(smem_u32(&bars->k_empty[slot]), (use - 1) & 1, abort_flag, &backward_status)) {
                    alive = false;
                    return;
                }
                const uint32_t full = smem_u32(&bars->k_full[slot]);
                mbar_arrive_expect_tx(full, K_TILE);
                const uint32_t dst = k_ring + slot * K_TILE;
                const int ky = row0 + j * KEYS;
                tma_load_2d(dst, &p.k_main_big, full, head * 128, ky);
                tma_load_2d(dst + CHUNK, &p.k_main_big, full, head * 128 + 64, ky);
                tma_load_2d(dst + 2 * CHUNK, &p.k_pe_big, full, 0, ky);
            };
            auto load_v = [&](int j) {
                // the slot is free once dO has been copied out (first tile) or dP(j-1) has run
                const bool ready = j == 0 ? mbar_wait(smem_u32(&bars->do_copied), 0, abort_flag, &backward_status)
                                          : mbar_wait(smem_u32(&bars->v_empty), (j - 1) & 1, abort_flag, &backward_status);
                if (!ready) {
                    alive = false;
                    return;
                }
                const uint32_t full = smem_u32(&bars->v_full);
                mbar_arrive_expect_tx(full, V_TILE);
                const int ky = row0 + j * KEYS;
                tma_load_2d(v_smem, &p.v_big, full, head * 128, ky);
                tma_load_2d(v_smem + CHUNK, &p.v_big, full, head * 128 + 64, ky);
            };
            // K(j) becomes loadable after dQ(j-3), V(j-1) right after that (after dP(j-2)).
            for (int j = 0; j < tile_count && alive; ++j) {
                load_k(j);
                if (j >= 1 && alive) {
                    load_v(j - 1);
                }
            }
            if (alive) {
                load_v(tile_count - 1);
            }
        }
    } else if (warp == MMA_WARP) {
        // Whole warp, uniform control flow; the elected lane executes the tcgen05 instructions.
        const uint32_t leader = elect_one();
        constexpr uint32_t IDESC_SCORE = make_idesc_bf16(BIG, KEYS, false, false);
        constexpr uint32_t IDESC_DQ = make_idesc_bf16(BIG, 192, false, true);
        bool alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->resident_full), 0, abort_flag, &backward_status));
        // S(j) = Q K_j^T
        auto issue_s = [&](int j) {
            const int slot = j % K_SLOTS;
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->k_full[slot]), (j / K_SLOTS) & 1, abort_flag, &backward_status));
            if (alive && j > 0) {
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->s_free), (j - 1) & 1, abort_flag, &backward_status));
            }
            if (!alive) {
                return;
            }
            tc_fence_after_sync();
            const uint32_t k_smem = k_ring + slot * K_TILE;
#pragma unroll
            for (int c = 0; c < 3; ++c) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    mma_ss_elect(tmem_base + TMEM_S, make_kmajor_desc(q_smem + c * CHUNK + k * 32), make_kmajor_desc(k_smem + c * CHUNK + k * 32),
                                 IDESC_SCORE, (c | k) != 0 ? 1U : 0U, leader);
                }
            }
            mma_commit_elect(smem_u32(&bars->s_full), leader);
        };
        // dP(j) = dO V_j^T, dO from tensor memory
        auto issue_dp = [&](int j) {
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->v_full), j & 1, abort_flag, &backward_status));
            if (!alive) {
                return;
            }
            tc_fence_after_sync();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    mma_ts_elect(tmem_base + TMEM_DP, tmem_base + TMEM_DO + c * 32 + k * 8, make_kmajor_desc(v_smem + c * CHUNK + k * 32), IDESC_SCORE,
                                 (c | k) != 0 ? 1U : 0U, leader);
                }
            }
            mma_commit_elect(smem_u32(&bars->v_empty), leader);
            mma_commit_elect(smem_u32(&bars->dp_full), leader);
        };
        if (alive) {
            issue_s(0);
        }
        if (alive) {
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->do_copied), 0, abort_flag, &backward_status));
        }
        if (alive) {
            tc_fence_after_sync();
            issue_dp(0);
        }
        for (int j = 0; j < tile_count && alive; ++j) {
            if (j + 1 < tile_count) {
                issue_s(j + 1);
                if (!alive) {
                    break;
                }
            }
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->ds_full), j & 1, abort_flag, &backward_status));
            if (!alive) {
                break;
            }
            tc_fence_after_sync();
            // dQ += dS(j) K_j: 16 keys per step, the three 64-column blocks of K are 16 KB apart
            const uint32_t k_smem = k_ring + (j % K_SLOTS) * K_TILE;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint32_t ds_tmem = tmem_base + TMEM_DP + (k / 4) * 64 + (k % 4) * 8;
                mma_ts_elect(tmem_base + TMEM_DQ, ds_tmem, make_smem_desc(k_smem + k * 2048, CHUNK, 1024), IDESC_DQ, (j | k) != 0 ? 1U : 0U, leader);
            }
            mma_commit_elect(smem_u32(&bars->k_empty[j % K_SLOTS]), leader);
            if (j + 1 < tile_count) {
                issue_dp(j + 1);
            }
        }
        if (alive) {
            mma_commit_elect(smem_u32(&bars->final_full), leader);
        }
    } else {
        // =================== softmax: thread = (row, half of the keys) =======
        const int half = warp / 4;
        const int r = threadIdx.x % BIG;
        const uint32_t lane_base = static_cast<uint32_t>((warp % 4) * 32) << 16;
        const int q_pos = q_start + r;
        const int q_safe = min(q_pos, length - 1);
        const float lse2 = p.lse[lse_offset + q_safe] * LOG2E;
        const float delta = p.delta[lse_offset + q_safe];
        bool alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->resident_full), 0, abort_flag, &backward_status));
        if (alive) {
            // dO chunk `half`, row r -> 32 packed columns of tensor memory (undo the 128-byte swizzle)
            uint32_t values[32];
            const uint8_t* row = smem_raw + Q_BYTES + K_SLOTS * K_TILE + half * CHUNK + r * 128;
#pragma unroll
            for (int unit = 0; unit < 8; ++unit) {
                const uint4 v = *reinterpret_cast<const uint4*>(row + ((unit ^ (r & 7)) * 16));
                values[unit * 4 + 0] = v.x;
                values[unit * 4 + 1] = v.y;
                values[unit * 4 + 2] = v.z;
                values[unit * 4 + 3] = v.w;
            }
            tmem_st_x32(tmem_base + lane_base + TMEM_DO + half * 32, values);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&bars->do_copied));
        }
        const uint32_t s_tmem = tmem_base + lane_base + TMEM_S + half * 64;
        const uint32_t dp_tmem = tmem_base + lane_base + TMEM_DP + half * 64;
        for (int j = 0; j < tile_count && alive; ++j) {
            // ---- stage 1: S -> registers, P ----
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->s_full), j & 1, abort_flag, &backward_status));
            if (!alive) {
                break;
            }
            tc_fence_after_sync();
            uint32_t sb[64];
            tmem_ld_x32(s_tmem, sb);
            tmem_ld_x32(s_tmem + 32, sb + 32);
            tmem_wait_ld();
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&bars->s_free));
            const int key0 = j * KEYS + half * 64;
            const bool masked = key0 + 63 > q_start;
            float prob[64];          // P * scale
#pragma unroll
            for (int n = 0; n < 64; ++n) {
                float value = exp2_approx(fmaf(__uint_as_float(sb[n]), p.scale_log2, -lse2)) * p.scale;
                if (masked) {
                    value = key0 + n <= q_pos ? value : 0.0F;
                }
                prob[n] = value;
            }
            // ---- stage 2: dS = P (dP - delta) scale ----
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->dp_full), j & 1, abort_flag, &backward_status));
            if (!alive) {
                break;
            }
            tc_fence_after_sync();
            tmem_ld_x32(dp_tmem, sb);
            tmem_ld_x32(dp_tmem + 32, sb + 32);
            tmem_wait_ld();
            uint32_t packed[32];
#pragma unroll
            for (int n = 0; n < 64; n += 2) {
                const float d0 = prob[n] * (__uint_as_float(sb[n]) - delta);
                const float d1 = prob[n + 1] * (__uint_as_float(sb[n + 1]) - delta);
                packed[n / 2] = pack_bf16x2(d0, d1);
            }
            tmem_st_x32(dp_tmem, packed);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&bars->ds_full));
        }
        if (alive) {
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->final_full), 0, abort_flag, &backward_status));
        }
        if (alive) {
            tc_fence_after_sync();
            const bool valid = q_pos < length;
            __nv_bfloat16* dq_row = p.dq + (static_cast<size_t>(row0 + q_pos) * p.heads + head) * 192 + half * 96;
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                uint32_t values[32];
                tmem_ld_x32(tmem_base + lane_base + TMEM_DQ + half * 96 + c * 32, values);
                tmem_wait_ld();
                if (valid) {
                    store_bf16_row(dq_row + c * 32, values, 32, 1.0F);
                }
            }
        }
    }

    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        for (int k = 0; k < 64; ++k) {
            __nanosleep(1000);
        }
    }
    if (warp == MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLUMNS);
    }
}

// ---------------------------------------------------------------------------
// dK/dV kernel: stationary 128 keys (K 3 chunks, V 2 chunks), streamed 64-query
// tiles (Q 3 chunks, dO 2 chunks, LSE and delta of those queries).
// Tensor memory: dV at 0..127, dK at 128..319, three 64-column score buffers
// X0..X2 at 320/384/448.  Tile t (relative) puts S^T in X[(2t)%3] and dP^T in
// X[(2t+1)%3]; P^T and dS^T overwrite them in place as bf16.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS, 1) backward_dkdv_kernel(const __grid_constant__ BackwardParams p) {
    extern __shared__ uint8_t smem_raw[];
    if (*reinterpret_cast<volatile int*>(&backward_status) != 0) {
        return;
    }
    const int head = p.head0 + blockIdx.y;
    int row0, length, block, blocks_in_sequence, sequence;
    size_t lse_offset;
    if (!locate_block(p, BIG, blockIdx.x, row0, length, block, blocks_in_sequence, lse_offset, head, &sequence)) {
        return;
    }
    const int key_start = block * BIG;                 // block 0 has the most queries: longest first
    const int first_tile = key_start / SUB;
    const int tile_count = (length + SUB - 1) / SUB - first_tile;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023U) & ~1023U;
    uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t k_smem = smem_base;                          // 3 chunks
    const uint32_t v_smem = smem_base + 3 * BIG_CHUNK;          // 2 chunks
    const uint32_t stage_smem = smem_base + RESIDENT_BYTES;
    BackwardBarriers* bars = reinterpret_cast<BackwardBarriers*>(smem_aligned + RESIDENT_BYTES + STAGES * STAGE_BYTES);
    volatile int* abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        // stage_full needs two arrivals here: the TMA transaction and the LSE/delta rows
        init_barriers(bars, 2);
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&bars->tmem_base), TMEM_COLUMNS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
    constexpr uint32_t TMEM_DV = 0;
    constexpr uint32_t TMEM_DK = 128;
    constexpr uint32_t TMEM_X = 320;

    if (warp == LOAD_WARP) {
        if (lane == 0) {
            const uint32_t bar = smem_u32(&bars->resident_full);
            mbar_arrive_expect_tx(bar, RESIDENT_BYTES);
            const int y = row0 + key_start;
            tma_load_2d(k_smem, &p.k_main_big, bar, head * 128, y);
            tma_load_2d(k_smem + BIG_CHUNK, &p.k_main_big, bar, head * 128 + 64, y);
            tma_load_2d(k_smem + 2 * BIG_CHUNK, &p.k_pe_big, bar, 0, y);
            tma_load_2d(v_smem, &p.v_big, bar, head * 128, y);
            tma_load_2d(v_smem + BIG_CHUNK, &p.v_big, bar, head * 128 + 64, y);
        }
        bool alive = true;
        for (int t = 0; t < tile_count && alive; ++t) {
            const int stage = t % STAGES;
            const int use = t / STAGES;
            if (use > 0) {
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->stage_empty[stage]), (use - 1) & 1, abort_flag, &backward_status));
                if (!alive) {
                    break;
                }
            }
            const int q0 = (first_tile + t) * SUB;
            const uint32_t full = smem_u32(&bars->stage_full[stage]);
            if (lane == 0) {
                mbar_arrive_expect_tx(full, STAGE_BYTES);
                const uint32_t dst = stage_smem + stage * STAGE_BYTES;
                const int qy = row0 + q0;
                tma_load_2d(dst, &p.q_main_sub, full, head * 128, qy);
                tma_load_2d(dst + SUB_CHUNK, &p.q_main_sub, full, head * 128 + 64, qy);
                tma_load_2d(dst + 2 * SUB_CHUNK, &p.q_pe_sub, full, head * 64, qy);
                tma_load_2d(dst + 3 * SUB_CHUNK, &p.do_sub, full, head * 128, qy);
                tma_load_2d(dst + 4 * SUB_CHUNK, &p.do_sub, full, head * 128 + 64, qy);
            }
#pragma unroll
            for (int e = 0; e < SUB / 32; ++e) {
                const int n = e * 32 + lane;
                const int q_pos = q0 + n;
                float lse_value = 0.0F, delta_value = 0.0F;
                if (q_pos < length) {
                    lse_value = p.lse[lse_offset + q_pos] * LOG2E;
                    delta_value = p.delta[lse_offset + q_pos];
                }
                bars->lse2[stage][n] = lse_value;
                bars->delta[stage][n] = delta_value;
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(full);
            }
        }
    } else if (warp == MMA_WARP) {
        // Whole warp, uniform control flow; the elected lane executes the tcgen05 instructions.
        {
            const uint32_t leader = elect_one();
            constexpr uint32_t IDESC_SCORE = make_idesc_bf16(BIG, SUB, false, false);
            constexpr uint32_t IDESC_DV = make_idesc_bf16(BIG, 128, false, true);
            constexpr uint32_t IDESC_DK = make_idesc_bf16(BIG, 192, false, true);
            bool alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->resident_full), 0, abort_flag, &backward_status));
            auto x_buffer = [&](int index) -> uint32_t { return tmem_base + TMEM_X + (index % 3) * 64; };
            // S^T(t) = K Q_t^T
            auto issue_st = [&](int t) {
                const int stage = t % STAGES;
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->stage_full[stage]), (t / STAGES) & 1, abort_flag, &backward_status));
                if (!alive) {
                    return;
                }
                tc_fence_after_sync();
                const uint32_t q_smem = stage_smem + stage * STAGE_BYTES;
#pragma unroll
                for (int c = 0; c < 3; ++c) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        mma_ss_elect(x_buffer(2 * t), make_kmajor_desc(k_smem + c * BIG_CHUNK + k * 32),
                               make_kmajor_desc(q_smem + c * SUB_CHUNK + k * 32), IDESC_SCORE, (c | k) != 0 ? 1U : 0U, leader);
                    }
                }
                mma_commit_elect(smem_u32(&bars->mma_a[t & 1]), leader);
            };
            // dP^T(t) = V dO_t^T   (the stage is already known to be full)
            auto issue_dpt = [&](int t) {
                const uint32_t do_smem = stage_smem + (t % STAGES) * STAGE_BYTES + 3 * SUB_CHUNK;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        mma_ss_elect(x_buffer(2 * t + 1), make_kmajor_desc(v_smem + c * BIG_CHUNK + k * 32),
                               make_kmajor_desc(do_smem + c * SUB_CHUNK + k * 32), IDESC_SCORE, (c | k) != 0 ? 1U : 0U, leader);
                    }
                }
                mma_commit_elect(smem_u32(&bars->mma_b[t & 1]), leader);
            };
            if (alive) {
                issue_st(0);
            }
            if (alive) {
                issue_dpt(0);
            }
            for (int t = 0; t < tile_count && alive; ++t) {
                const int stage = t % STAGES;
                const uint32_t parity = (t >> 1) & 1;
                if (t + 1 < tile_count) {
                    issue_st(t + 1);
                    if (!alive) {
                        break;
                    }
                }
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->soft_a[t & 1]), parity, abort_flag, &backward_status));
                if (!alive) {
                    break;
                }
                tc_fence_after_sync();
                const uint32_t q_smem = stage_smem + stage * STAGE_BYTES;
                const uint32_t do_smem = q_smem + 3 * SUB_CHUNK;
                // dV += P^T dO_t
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    mma_ts_elect(tmem_base + TMEM_DV, x_buffer(2 * t) + (k / 2) * 32 + (k % 2) * 8, make_smem_desc(do_smem + k * 2048, SUB_CHUNK, 1024), IDESC_DV,
                           (t | k) != 0 ? 1U : 0U, leader);
                }
                if (t + 1 < tile_count) {
                    issue_dpt(t + 1);
                }
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->soft_b[t & 1]), parity, abort_flag, &backward_status));
                if (!alive) {
                    break;
                }
                tc_fence_after_sync();
                // dK += dS^T Q_t
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    mma_ts_elect(tmem_base + TMEM_DK, x_buffer(2 * t + 1) + (k / 2) * 32 + (k % 2) * 8, make_smem_desc(q_smem + k * 2048, SUB_CHUNK, 1024), IDESC_DK,
                           (t | k) != 0 ? 1U : 0U, leader);
                }
                mma_commit_elect(smem_u32(&bars->stage_empty[stage]), leader);
            }
            if (alive) {
                mma_commit_elect(smem_u32(&bars->final_full), leader);
            }
        }
    } else {
        const int group = warp / 4;
        const int r = threadIdx.x % BIG;
        const uint32_t lane_base = static_cast<uint32_t>((warp % 4) * 32) << 16;
        const int key_pos = key_start + r;
        uint4* ds_tiles = nullptr;             // this key tile's first tile of the scratch (query tile 2 * block)
        if (p.ds_scratch != nullptr) {
            const ScratchPlace place = scratch_place(p, sequence);
            const long long first = blockIdx.y * place.head_tiles + place.sequence_first + static_cast<long long>(block) * (2 * place.key_tiles) -
                                    static_cast<long long>(block) * (block - 1);
            ds_tiles = reinterpret_cast<uint4*>(p.ds_scratch) + static_cast<size_t>(first) * (DS_TILE_BYTES / 16);
        }
        bool alive = true;
        // Both groups work on every tile: thread = (key row, 32 of the tile's 64 queries), so a
        // tile's softmax takes half as long and the tensor core rarely waits for it.  Each
        // thread overwrites only columns it has read itself: queries 32g..32g+31 are fp32
        // columns 32g..32g+31 and become bf16 columns 32g..32g+15.
        for (int t = 0; t < tile_count; ++t) {
            const int stage = t % STAGES;
            const uint32_t parity = (t >> 1) & 1;
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->stage_full[stage]), (t / STAGES) & 1, abort_flag, &backward_status) &&
                                                mbar_wait(smem_u32(&bars->mma_a[t & 1]), parity, abort_flag, &backward_status));
            if (!alive) {
                break;
            }
            tc_fence_after_sync();
            const uint32_t st_tmem = tmem_base + lane_base + TMEM_X + ((2 * t) % 3) * 64 + group * 32;
            const uint32_t dpt_tmem = tmem_base + lane_base + TMEM_X + ((2 * t + 1) % 3) * 64 + group * 32;
            // the per-query constants are the same for every lane: 16-byte broadcast loads
            const float4* lse4 = reinterpret_cast<const float4*>(bars->lse2[stage] + group * 32);
            const float4* delta4 = reinterpret_cast<const float4*>(bars->delta[stage] + group * 32);
            const int q0 = (first_tile + t) * SUB + group * 32;
            const bool masked = q0 < key_start + BIG || q0 + 32 > length;
            uint32_t sb[32];
            float prob[32];
            tmem_ld_x32(st_tmem, sb);
            tmem_wait_ld();
            uint32_t packed[16];
#pragma unroll
            for (int n = 0; n < 32; n += 4) {
                const float4 l = lse4[n / 4];
                prob[n] = exp2_approx(fmaf(__uint_as_float(sb[n]), p.scale_log2, -l.x));
                prob[n + 1] = exp2_approx(fmaf(__uint_as_float(sb[n + 1]), p.scale_log2, -l.y));
                prob[n + 2] = exp2_approx(fmaf(__uint_as_float(sb[n + 2]), p.scale_log2, -l.z));
                prob[n + 3] = exp2_approx(fmaf(__uint_as_float(sb[n + 3]), p.scale_log2, -l.w));
            }
            if (masked) {
#pragma unroll
                for (int n = 0; n < 32; ++n) {
                    prob[n] = (key_pos <= q0 + n && q0 + n < length) ? prob[n] : 0.0F;
                }
            }
#pragma unroll
            for (int n = 0; n < 32; n += 2) {
                packed[n / 2] = pack_bf16x2(prob[n], prob[n + 1]);
            }
            tmem_st_x16(st_tmem, packed);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&bars->soft_a[t & 1]));

            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->mma_b[t & 1]), parity, abort_flag, &backward_status));
            if (!alive) {
                break;
            }
            tc_fence_after_sync();
            tmem_ld_x32(dpt_tmem, sb);
            tmem_wait_ld();
#pragma unroll
            for (int n = 0; n < 32; n += 4) {
                const float4 d = delta4[n / 4];
                packed[n / 2] = pack_bf16x2(prob[n] * (__uint_as_float(sb[n]) - d.x) * p.scale, prob[n + 1] * (__uint_as_float(sb[n + 1]) - d.y) * p.scale);
                packed[n / 2 + 1] =
                    pack_bf16x2(prob[n + 2] * (__uint_as_float(sb[n + 2]) - d.z) * p.scale, prob[n + 3] * (__uint_as_float(sb[n + 3]) - d.w) * p.scale);
            }
            tmem_st_x16(dpt_tmem, packed);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&bars->soft_b[t & 1]));
            if (ds_tiles != nullptr) {
                // The same 32 bf16 values go to the scratch for the kernel that turns dS into dQ: four 16-byte
                // units, unit (4 group + e) of this key.  The 32 lanes of a warp write 512 consecutive bytes.
                // Keys past the end of the sequence are written as zeros, so that whatever lies behind
                // the last key in the K tensor cannot reach dQ.
                uint4* dst = ds_tiles + static_cast<size_t>(t) * (DS_TILE_BYTES / 16) + (group * 4) * BIG + r;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint4 value = key_pos < length ? make_uint4(packed[4 * e], packed[4 * e + 1], packed[4 * e + 2], packed[4 * e + 3]) : make_uint4(0, 0, 0, 0);
                    __stcs(dst + e * BIG, value);       // written once, read once by the next kernel: streaming store
                }
            }
        }
        if (alive) {
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->final_full), 0, abort_flag, &backward_status));
        }
        if (alive) {
            tc_fence_after_sync();
            const bool valid = key_pos < length;
            const size_t row = static_cast<size_t>(row0 + key_pos);
            if (group == 0) {
                __nv_bfloat16* dv_row = p.dv + (row * p.heads + head) * 128;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t values[32];
                    tmem_ld_x32(tmem_base + lane_base + TMEM_DV + c * 32, values);
                    tmem_wait_ld();
                    if (valid) {
                        store_bf16_row(dv_row + c * 32, values, 32, 1.0F);
                    }
                }
            } else {
                __nv_bfloat16* dk_row = p.dk_nope + (row * p.heads + head) * 128;
#pragma unroll
                for (int c = 0; c < 6; ++c) {
                    uint32_t values[32];
                    tmem_ld_x32(tmem_base + lane_base + TMEM_DK + c * 32, values);
                    tmem_wait_ld();
                    if (valid) {
                        if (c < 4) {
                            store_bf16_row(dk_row + c * 32, values, 32, 1.0F);
                        } else {
                            uint4* part = reinterpret_cast<uint4*>(p.dk_pe_parts + (row * p.heads + head) * 64 + (c - 4) * 32);
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                part[e] = make_uint4(values[4 * e], values[4 * e + 1], values[4 * e + 2], values[4 * e + 3]);
                            }
                        }
                    }
                }
            }
        }
    }

    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        for (int k = 0; k < 64; ++k) {
            __nanosleep(1000);
        }
    }
    if (warp == MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLUMNS);
    }
}

// ---------------------------------------------------------------------------
// dQ from stored dS: dQ[q, :] = sum over keys <= q of dS[q, key] * K[key, :].
//
// backward_dkdv_kernel has written dS^T (scale included, zeros above the diagonal) to the
// scratch, so this is a causal batched GEMM with nothing to recompute: 384 FLOP per (query,
// key) pair instead of the 1024 of backward_dq_kernel.  CTA = 256 query rows of one (batch,
// head), two 128 x 192 fp32 accumulators in tensor memory; it streams 64-key stages, each the
// 64 keys x 256 queries of dS^T (32 blocks of 8 queries, 1 KB each: an unswizzled MN-major A
// operand) and the [64 keys x 192] rows of K (three swizzled chunks, the MN-major B operand).
// 56 KB per stage, four stages.  Warps 0-3 store the result, warp 4 issues the MMAs, warp 5
// loads.  The kernel is bound by reading dS once from HBM.
// ---------------------------------------------------------------------------
namespace dqs {
constexpr int QROWS = 256;
constexpr int KSUB = 64;
constexpr int DS_BYTES = 4 * SUB_CHUNK;
constexpr int K_BYTES = 3 * SUB_CHUNK;
constexpr int STREAM_STAGE_BYTES = DS_BYTES + K_BYTES;
constexpr int STREAM_STAGES = 4;
constexpr int STREAM_BAR_BYTES = 1024;
constexpr int STREAM_SMEM_BYTES = STREAM_STAGES * STREAM_STAGE_BYTES + STREAM_BAR_BYTES + 1024;
constexpr int STREAM_THREADS = 192;
constexpr int STREAM_MMA_WARP = 4;
constexpr int STREAM_LOAD_WARP = 5;
static_assert(STREAM_SMEM_BYTES <= 227 * 1024, "streamed dQ kernel shared memory");

struct StreamBarriers {
    uint64_t full[STREAM_STAGES];
    uint64_t empty[STREAM_STAGES];
    uint64_t done;
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(StreamBarriers) <= STREAM_BAR_BYTES, "barrier block too large");
}  // namespace dqs

__global__ void __launch_bounds__(dqs::STREAM_THREADS, 1) backward_dq_stream_kernel(const __grid_constant__ BackwardParams p) {
        using namespace dqs;
    extern __shared__ uint8_t smem_raw[];
    if (*reinterpret_cast<volatile int*>(&backward_status) != 0) {
        return;
    }
    const int head = p.head0 + blockIdx.y;
    int row0, length, block, blocks_in_sequence, sequence;
    size_t lse_offset;
    if (!locate_block(p, QROWS, blockIdx.x, row0, length, block, blocks_in_sequence, lse_offset, head, &sequence)) {
        return;
    }
    const int q_start = (blocks_in_sequence - 1 - block) * QROWS;        // longest first
    const int key_end = min(length, q_start + QROWS);
    const int stage_count = (key_end + KSUB - 1) / KSUB;
    const bool second_used = q_start + 128 < length;
    // rows of the scratch view (8-query blocks) before this (head, sequence), and key tiles of the sequence
    const ScratchPlace place = scratch_place(p, sequence);
    const int key_tiles = place.key_tiles;
    const long long ds_row0 = (blockIdx.y * place.head_tiles + place.sequence_first) * 8;
    const int q_tile0 = q_start / SUB;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023U) & ~1023U;
    uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    StreamBarriers* bars = reinterpret_cast<StreamBarriers*>(smem_aligned + STREAM_STAGES * STREAM_STAGE_BYTES);
    volatile int* abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STREAM_STAGES; ++i) {
            mbar_init(smem_u32(&bars->full[i]), 1);
            mbar_init(smem_u32(&bars->empty[i]), 1);
        }
        mbar_init(smem_u32(&bars->done), 1);
        bars->abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == STREAM_MMA_WARP) {
        tmem_alloc(smem_u32(&bars->tmem_base), TMEM_COLUMNS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

    // A stage holds keys [64 s, 64 s + 64).  The first accumulator (rows q_start..q_start+127)
    // takes keys below q_start + 128, the second all of them; stages only the second uses
    // load the two chunks of its rows only.
    if (warp == STREAM_LOAD_WARP) {
        const uint64_t policy = l2_evict_first_policy();       // dS is read once; the K rows are what should stay in L2
        bool alive = true;
        for (int s = 0; s < stage_count && alive; ++s) {
            const int stage = s % STREAM_STAGES;
            if (s >= STREAM_STAGES) {
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->empty[stage]), ((s / STREAM_STAGES) - 1) & 1, abort_flag, &backward_status));
                if (!alive) {
                    break;
                }
            }
            if (lane == 0) {
                const int key0 = s * KSUB;
                const int first_chunk = key0 < q_start + 128 ? 0 : 2;
                const uint32_t full = smem_u32(&bars->full[stage]);
                const uint32_t dst = smem_base + stage * STREAM_STAGE_BYTES;
                mbar_arrive_expect_tx(full, (4 - first_chunk) * SUB_CHUNK + K_BYTES);
                // key tile kt holds its query tiles 2 kt, 2 kt + 1, ... one after the other, 8 rows of the view each
                const int kt = key0 / BIG;
                const long long tile = static_cast<long long>(kt) * (2 * key_tiles) - static_cast<long long>(kt) * (kt - 1) + (q_tile0 - 2 * kt);
                for (int c = first_chunk; c < 4; c += 2) {
                    tma_load_2d_hint(dst + c * SUB_CHUNK, &p.ds_map, full, (key0 % BIG) * 2, static_cast<int>(ds_row0 + (tile + c) * 8), policy);
                }
                const int y = row0 + key0;
                tma_load_2d(dst + DS_BYTES, &p.k_main_sub, full, head * 128, y);
                tma_load_2d(dst + DS_BYTES + SUB_CHUNK, &p.k_main_sub, full, head * 128 + 64, y);
                tma_load_2d(dst + DS_BYTES + 2 * SUB_CHUNK, &p.k_pe_sub, full, 0, y);
            }
        }
    } else if (warp == STREAM_MMA_WARP) {
        const uint32_t leader = elect_one();
        constexpr uint32_t IDESC = make_idesc_bf16(128, 192, true, true);
        bool alive = true;
        for (int s = 0; s < stage_count && alive; ++s) {
            const int stage = s % STREAM_STAGES;
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->full[stage]), (s / STREAM_STAGES) & 1, abort_flag, &backward_status));
            if (!alive) {
                break;
            }
            tc_fence_after_sync();
            const uint32_t ds_smem = smem_base + stage * STREAM_STAGE_BYTES;
            const uint32_t k_smem = ds_smem + DS_BYTES;
            const int key0 = s * KSUB;
            if (key0 < q_start + 128) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    mma_ss_elect(tmem_base, make_smem_desc_plain(ds_smem + k * 256, 128, 1024), make_smem_desc(k_smem + k * 2048, SUB_CHUNK, 1024), IDESC,
                                 (s | k) != 0 ? 1U : 0U, leader);
                }
            }
            if (second_used) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    mma_ss_elect(tmem_base + 192, make_smem_desc_plain(ds_smem + 2 * SUB_CHUNK + k * 256, 128, 1024),
                                 make_smem_desc(k_smem + k * 2048, SUB_CHUNK, 1024), IDESC, (s | k) != 0 ? 1U : 0U, leader);
                }
            }
            mma_commit_elect(smem_u32(&bars->empty[stage]), leader);
        }
        if (alive) {
            mma_commit_elect(smem_u32(&bars->done), leader);
        }
    } else {
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        const bool alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->done), 0, abort_flag, &backward_status));
        if (alive) {
            tc_fence_after_sync();
            for (int j = 0; j < (second_used ? 2 : 1); ++j) {
                const int q_pos = q_start + j * 128 + warp * 32 + lane;
                __nv_bfloat16* dq_row = p.dq + (static_cast<size_t>(row0 + q_pos) * p.heads + head) * 192;
#pragma unroll
                for (int c = 0; c < 6; ++c) {
                    uint32_t values[32];
                    tmem_ld_x32(tmem_base + lane_base + j * 192 + c * 32, values);
                    tmem_wait_ld();
                    if (q_pos < length) {
                        store_bf16_row(dq_row + c * 32, values, 32, 1.0F);
                    }
                }
            }
        }
    }

    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        for (int k = 0; k < 64; ++k) {
            __nanosleep(1000);
        }
    }
    if (warp == STREAM_MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLUMNS);
    }
}

void configure_kernels() {
    static bool done[16] = {};
    int device = 0;
    CUDA_CHECK(cudaGetDevice(&device));
    if (device < 16 && done[device]) {
        return;
    }
    CUDA_CHECK(cudaFuncSetAttribute(backward_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dqk::SMEM_BYTES));
    CUDA_CHECK(cudaFuncSetAttribute(backward_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    CUDA_CHECK(cudaFuncSetAttribute(backward_dq_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dqs::STREAM_SMEM_BYTES));
    if (device < 16) {
        done[device] = true;
    }
}

std::size_t accumulator_bytes(int total_tokens) {
    // fp32 dk_pe sums, rounded up so that the delta array behind it stays 256-byte aligned
    return (static_cast<std::size_t>(total_tokens) * 64 * sizeof(float) + 255) / 256 * 256;
}

std::size_t delta_bytes(int total_tokens, int heads) {
    return (static_cast<std::size_t>(total_tokens) * heads * sizeof(float) + 255) / 256 * 256;
}

std::size_t parts_bytes(int total_tokens, int heads) {
    return (static_cast<std::size_t>(total_tokens) * heads * 64 * sizeof(float) + 255) / 256 * 256;
}

// dS^T of a group of heads stays in scratch between the two main kernels.  The group is as many heads as
// fit in ds_scratch_limit (20 GiB unless the caller sets another); 0 = not even one head fits, and the
// backward recomputes S and dP in a dQ kernel of its own instead.
std::atomic<std::size_t> ds_scratch_limit{std::size_t{20} << 30};

// An upper bound, computable without the lengths, on the 16 KB tiles of dS^T one head needs: a sequence of
// k key tiles takes k * k + k.  Every sequence is at most max_sequence_length long (first bound) and the
// squares of the lengths add up to at most max_sequence_length * total_tokens (second bound; k <=
// length / 128 + 1).  Dense batches meet the first bound exactly.
std::size_t ds_tiles_per_head(int batch_size, int max_sequence_length, int total_tokens) {
    const std::size_t key_tiles = (static_cast<std::size_t>(max_sequence_length) + BIG - 1) / BIG;
    const std::size_t by_longest = static_cast<std::size_t>(batch_size) * (key_tiles * key_tiles + key_tiles);
    const std::size_t by_total = static_cast<std::size_t>(max_sequence_length) * static_cast<std::size_t>(total_tokens) / (BIG * BIG) + 1 +
                                 3 * static_cast<std::size_t>(total_tokens) / BIG + 1 + 2 * static_cast<std::size_t>(batch_size);
    return by_longest < by_total ? by_longest : by_total;
}

int ds_group_heads(int batch_size, int max_sequence_length, int total_tokens, int heads) {
    const std::size_t per_head = ds_tiles_per_head(batch_size, max_sequence_length, total_tokens) * DS_TILE_BYTES;
    const std::size_t fit = ds_scratch_limit.load() / per_head;
    return static_cast<int>(fit < static_cast<std::size_t>(heads) ? fit : static_cast<std::size_t>(heads));
}

}  // namespace

namespace internal {

int backward_device_status(bool reset) {
    int status = 0;
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemcpyFromSymbol(&status, backward_status, sizeof(int)));
    if (reset && status != 0) {
        const int zero = 0;
        CUDA_CHECK(cudaMemcpyToSymbol(backward_status, &zero, sizeof(int)));
    }
    return status;
}

}  // namespace internal

std::size_t mla_prefill_backward_scratch_limit(long long bytes) {
    return bytes < 0 ? ds_scratch_limit.load() : ds_scratch_limit.exchange(static_cast<std::size_t>(bytes));
}

int mla_prefill_backward_launches(int batch_size, int max_sequence_length, int total_tokens, int heads, bool packed) {
    (void)packed;       // dense and packed batches take the same route
    const int group = ds_group_heads(batch_size, max_sequence_length, total_tokens, heads);
    // delta, the two main kernels (once per group of heads), the dk_pe sum
    return group > 0 ? 2 + 2 * ((heads + group - 1) / group) : 4;
}

std::size_t mla_prefill_backward_workspace_bytes(int batch_size, int max_sequence_length, int total_tokens, int heads) {
    if (total_tokens <= 0 || heads <= 0) {
        return 0;
    }
    // dk_pe sums, then delta [tokens, heads], then the per-head dk_pe contributions [tokens, heads, 64],
    // then dS^T of one group of heads
    const std::size_t scratch = static_cast<std::size_t>(ds_group_heads(batch_size, max_sequence_length, total_tokens, heads)) *
                                ds_tiles_per_head(batch_size, max_sequence_length, total_tokens) * DS_TILE_BYTES;
    return accumulator_bytes(total_tokens) + delta_bytes(total_tokens, heads) + parts_bytes(total_tokens, heads) + scratch;
}

void mla_prefill_backward_cuda(__nv_bfloat16* dq, __nv_bfloat16* dk_nope, __nv_bfloat16* dk_pe, __nv_bfloat16* dv,
                               const __nv_bfloat16* output_gradient, const __nv_bfloat16* output, const float* logsumexp,
                               const __nv_bfloat16* q_nope, const __nv_bfloat16* q_pe, const __nv_bfloat16* k_nope, const __nv_bfloat16* k_pe,
                               const __nv_bfloat16* v, const int* cu_seqlens, void* workspace, int batch_size, int max_sequence_length,
                               int total_tokens, int heads, int nope_size, int rope_size, int value_size, float scale, cudaStream_t stream) {
    internal::check_prefill_shape(cu_seqlens, batch_size, max_sequence_length, total_tokens, heads, nope_size, rope_size, value_size, scale);
    for (const void* pointer : {static_cast<const void*>(dq), static_cast<const void*>(dk_nope), static_cast<const void*>(dk_pe),
                                static_cast<const void*>(dv), static_cast<const void*>(output_gradient), static_cast<const void*>(output),
                                static_cast<const void*>(logsumexp), static_cast<const void*>(q_nope), static_cast<const void*>(q_pe),
                                static_cast<const void*>(k_nope), static_cast<const void*>(k_pe), static_cast<const void*>(v),
                                static_cast<const void*>(workspace)}) {
        if (pointer == nullptr) {
            throw std::invalid_argument("null tensor pointer");
        }
        if ((reinterpret_cast<std::uintptr_t>(pointer) & 15U) != 0) {
            throw std::invalid_argument("tensor pointers must be 16-byte aligned");
        }
    }
    float* accumulator = static_cast<float*>(workspace);
    float* delta = reinterpret_cast<float*>(static_cast<char*>(workspace) + accumulator_bytes(total_tokens));
    float* parts = reinterpret_cast<float*>(static_cast<char*>(workspace) + accumulator_bytes(total_tokens) + delta_bytes(total_tokens, heads));

    BackwardParams params{};
    const std::uint64_t rows = static_cast<std::uint64_t>(total_tokens);
    const std::uint64_t wide = static_cast<std::uint64_t>(heads) * 128;
    const std::uint64_t narrow = static_cast<std::uint64_t>(heads) * 64;
    params.q_main_big = make_bf16_tile_map(q_nope, rows, wide, wide, BIG);
    params.q_pe_big = make_bf16_tile_map(q_pe, rows, narrow, narrow, BIG);
    params.k_main_big = make_bf16_tile_map(k_nope, rows, wide, wide, BIG);
    params.k_pe_big = make_bf16_tile_map(k_pe, rows, 64, 64, BIG);
    params.v_big = make_bf16_tile_map(v, rows, wide, wide, BIG);
    params.do_big = make_bf16_tile_map(output_gradient, rows, wide, wide, BIG);
    params.q_main_sub = make_bf16_tile_map(q_nope, rows, wide, wide, SUB);
    params.q_pe_sub = make_bf16_tile_map(q_pe, rows, narrow, narrow, SUB);
    params.k_main_sub = make_bf16_tile_map(k_nope, rows, wide, wide, SUB);
    params.k_pe_sub = make_bf16_tile_map(k_pe, rows, 64, 64, SUB);
    params.v_sub = make_bf16_tile_map(v, rows, wide, wide, SUB);
    params.do_sub = make_bf16_tile_map(output_gradient, rows, wide, wide, SUB);
    params.dq = dq;
    params.dk_nope = dk_nope;
    params.dv = dv;
    params.dk_pe_parts = parts;
    params.lse = logsumexp;
    params.delta = delta;
    params.cu_seqlens = cu_seqlens;
    params.batch = batch_size;
    params.max_seq = max_sequence_length;
    params.total = total_tokens;
    params.heads = heads;
    params.scale = scale;
    params.scale_log2 = scale * LOG2E;
    configure_kernels();

    const std::size_t pairs = static_cast<std::size_t>(total_tokens) * heads;
    const unsigned delta_blocks = static_cast<unsigned>(pairs / 8 + 1 < 148 * 32 ? pairs / 8 + 1 : 148 * 32);
    delta_kernel<<<delta_blocks, 256, 0, stream>>>(delta, output_gradient, output, cu_seqlens, batch_size, max_sequence_length, total_tokens, heads);
    CUDA_CHECK(cudaGetLastError());

    const int group = ds_group_heads(batch_size, max_sequence_length, total_tokens, heads);
    if (group > 0) {
        // per group of heads: the key-side kernel (which leaves dS^T in the scratch) and then dQ from it
        params.ds_scratch = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(workspace) + accumulator_bytes(total_tokens) + delta_bytes(total_tokens, heads) +
                                                             parts_bytes(total_tokens, heads));
        params.ds_map = make_u64_rows_map(params.ds_scratch, static_cast<std::uint64_t>(group) * ds_tiles_per_head(batch_size, max_sequence_length, total_tokens) * 8,
                                          256, 128, 16);
        dim3 key_grid, query_grid;
        if (cu_seqlens == nullptr) {
            key_grid = dim3((max_sequence_length + BIG - 1) / BIG, 1, batch_size);
            query_grid = dim3((max_sequence_length + dqs::QROWS - 1) / dqs::QROWS, 1, batch_size);
        } else {
            key_grid = dim3(total_tokens / BIG + batch_size, 1, 1);
            query_grid = dim3(total_tokens / dqs::QROWS + batch_size, 1, 1);
        }
        for (int head0 = 0; head0 < heads; head0 += group) {
            const int count = heads - head0 < group ? heads - head0 : group;
            params.head0 = head0;
            key_grid.y = count;
            query_grid.y = count;
            backward_dkdv_kernel<<<key_grid, THREADS, SMEM_BYTES, stream>>>(params);
            CUDA_CHECK(cudaGetLastError());
            backward_dq_stream_kernel<<<query_grid, dqs::STREAM_THREADS, dqs::STREAM_SMEM_BYTES, stream>>>(params);
            CUDA_CHECK(cudaGetLastError());
        }
    } else {
        dim3 grid;
        if (cu_seqlens == nullptr) {
            grid = dim3((max_sequence_length + BIG - 1) / BIG, heads, batch_size);
        } else {
            grid = dim3(total_tokens / BIG + batch_size, heads, 1);
        }
        params.ds_scratch = nullptr;
        params.head0 = 0;
        backward_dq_kernel<<<grid, THREADS, dqk::SMEM_BYTES, stream>>>(params);
        CUDA_CHECK(cudaGetLastError());
        backward_dkdv_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(params);
        CUDA_CHECK(cudaGetLastError());
    }
    const std::size_t quads = static_cast<std::size_t>(total_tokens) * 16;
    const unsigned sum_blocks = static_cast<unsigned>(quads / 256 + 1 < 148 * 8 ? quads / 256 + 1 : 148 * 8);
    sum_dk_pe_kernel<<<sum_blocks, 256, 0, stream>>>(dk_pe, accumulator, reinterpret_cast<const float4*>(parts), static_cast<std::size_t>(total_tokens), heads);
    CUDA_CHECK(cudaGetLastError());
}

}  // namespace dscuda
