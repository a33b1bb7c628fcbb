// Causal absorbed-latent MLA forward on sm_100a (mla_compressed_attention_forward_cuda): every
// head shares one compressed key/value row of 576 bf16 (512 latent + 64 rotary); the latent part is
// also the value.  The 128 rows of a tile are consecutive (token, head) pairs of one sequence and each
// row sees keys 0..its token.
//
// A 128x512 fp32 output tile would fill all of tensor memory, so a tile is
// handled by two CTAs: both compute S = Q K^T (K = 576) and each accumulates
// one 256-column half of O = P V.  Tensor memory per CTA: O 256 columns, two S
// buffers of 64 columns (P overwrites S in place as bf16), and 128 columns that
// hold the four 64-column chunks of Q facing this CTA's V chunks, as an MMA A
// operand.  Shared memory holds the other five Q chunks (80 KB) and two rings of
// key chunks, two tiles deep each: the five 8 KB chunks of a tile that only S
// needs, released as soon as S is computed, and the four that are also this
// CTA's V, released after P V.
//
// Warps 0-3: softmax / epilogue (one thread per row); warp 4: MMA issue (the
// whole warp runs the loop, one elected lane executes the instruction); warp 5:
// TMA loads.  All waits are bounded.  (The paged decode lives in absorbed_decode.cu.)
#include "mla.h"
#include "cuda_common.h"
#include "attention_internal.h"
#include "sm100_primitives.cuh"
#include "../common/tensor_map.h"

#include <algorithm>
#include <mutex>
#include <stdexcept>
#include <string>

namespace dscuda {
namespace {

using namespace sm100;

constexpr int ROWS = 128;                       // rows per tile = TMEM lanes
constexpr int KEYS = 64;                        // keys per tile
constexpr int RANK = MLA_KV_RANK;               // 512
constexpr int ROPE = MLA_ROPE_SIZE;             // 64
constexpr int WIDTH = RANK + ROPE;              // 576
constexpr int CHUNKS = WIDTH / 64;              // 9 column chunks of 64
constexpr int HALF_V = RANK / 2;                // value columns per CTA
constexpr int Q_TMEM_CHUNKS = 4;                // the Q chunks that face this CTA's V chunks live in tensor memory
constexpr int Q_SMEM_CHUNKS = CHUNKS - Q_TMEM_CHUNKS;
constexpr int Q_CHUNK_BYTES = ROWS * 128;       // 16 KB
constexpr int K_CHUNK_BYTES = KEYS * 128;       // 8 KB
constexpr int A_CHUNKS = 5;                     // key chunks of a tile that only S needs
constexpr int B_CHUNKS = 4;                     // key chunks of a tile that are also this CTA's V
constexpr int A_UNIT_BYTES = A_CHUNKS * K_CHUNK_BYTES;       // 40 KB
constexpr int B_UNIT_BYTES = B_CHUNKS * K_CHUNK_BYTES;       // 32 KB
constexpr int A_SLOTS = 2;
constexpr int B_SLOTS = 2;
constexpr int Q_SMEM_BYTES = Q_SMEM_CHUNKS * Q_CHUNK_BYTES;  // 80 KB
constexpr int A_RING_BYTES = A_SLOTS * A_UNIT_BYTES;         // 80 KB
constexpr int B_RING_BYTES = B_SLOTS * B_UNIT_BYTES;         // 64 KB
constexpr int MISC_BYTES = 1024;
constexpr int SMEM_BYTES = Q_SMEM_BYTES + A_RING_BYTES + B_RING_BYTES + MISC_BYTES + 1024;
constexpr int THREADS = 192;
constexpr int MMA_WARP = 4;
constexpr int LOAD_WARP = 5;
constexpr int TMEM_COLUMNS = 512;
constexpr int TMEM_O = 0;                       // 256 columns
constexpr int TMEM_S = 256;                     // 2 x 64 columns
constexpr int TMEM_Q = 384;                     // 128 columns = 4 chunks x 32
constexpr float RESCALE_THRESHOLD = 8.0F;
static_assert(Q_TMEM_CHUNKS * Q_CHUNK_BYTES <= B_RING_BYTES, "Q staging must fit in the value ring");
static_assert(SMEM_BYTES <= 232448, "shared memory budget");

__device__ int absorbed_status = 0;

struct AbsorbedParams {
    CUtensorMap q_lat;      // [rows, 512] box 128 x 64
    CUtensorMap q_rope;     // [rows, 64]  box 128 x 64
    CUtensorMap k_lat;      // [rows, 512] box 64 x 64
    CUtensorMap k_rope;     // [rows, 64]  box 64 x 64
    int batch;
    int sequence;           // T
    int heads;
    __nv_bfloat16* out;     // [B,T,H,512]
    float* lse;             // [B,H,T]
    float scale;
    float scale_log2;
};

struct AbsorbedBarriers {
    uint64_t q_full;            // Q chunks that stay in shared memory (one phase per segment)
    uint64_t q_stage_full;      // Q chunks on their way to tensor memory
    uint64_t q_tmem_ready;      // 128 arrivals: those chunks are in tensor memory
    uint64_t full_a[A_SLOTS];   // ring of the five key chunks only S needs
    uint64_t empty_a[A_SLOTS];
    uint64_t full_b[B_SLOTS];   // ring of the four chunks that are also this CTA's V
    uint64_t empty_b[B_SLOTS];
    uint64_t s_full[2];         // per S buffer
    uint64_t p_full[2];         // per S buffer
    uint64_t o_final;           // one phase per segment: the last P V has finished
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(AbsorbedBarriers) <= MISC_BYTES, "barrier block too large");

// The work of one CTA: key tiles [0, tile_end) for the 128 rows `row_tile` of sequence `b`.
struct Segment {
    int b;
    int row_tile;
    int tile_begin;
    int tile_end;
};

struct Walker {
    bool done;
};

// Every role thread calls this in a loop; a CTA has exactly one segment.
__device__ __forceinline__ bool next_segment(const AbsorbedParams& p, Walker& w, Segment& seg) {
    if (w.done) {
        return false;
    }
    const int rows_total = p.sequence * p.heads;
    const int first = (blockIdx.y >> 1) * ROWS;
    const int last_token = (min(first + ROWS, rows_total) - 1) / p.heads;
    seg.b = blockIdx.z;
    seg.row_tile = blockIdx.y >> 1;
    seg.tile_begin = 0;
    seg.tile_end = last_token / KEYS + 1;
    w.done = true;
    return true;
}

__global__ void __launch_bounds__(THREADS, 1) absorbed_attention_kernel(const __grid_constant__ AbsorbedParams p) {
    extern __shared__ uint8_t smem_raw[];
    if (*reinterpret_cast<volatile int*>(&absorbed_status) == STATUS_WAIT_TIMEOUT) {
        return;
    }
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    // grid (1, 2*row_tiles, B)
    const int half = blockIdx.y & 1;      // which 256 value columns

    // ---- shared memory ------------------------------------------------------
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023U) & ~1023U;
    uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t q_smem = smem_base;
    const uint32_t a_ring = smem_base + Q_SMEM_BYTES;
    const uint32_t b_ring = a_ring + A_RING_BYTES;
    uint8_t* b_ring_ptr = smem_aligned + Q_SMEM_BYTES + A_RING_BYTES;
    AbsorbedBarriers* bars = reinterpret_cast<AbsorbedBarriers*>(smem_aligned + Q_SMEM_BYTES + A_RING_BYTES + B_RING_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bars->q_full), 1);
        mbar_init(smem_u32(&bars->q_stage_full), 1);
        mbar_init(smem_u32(&bars->q_tmem_ready), ROWS);
        for (int i = 0; i < A_SLOTS; ++i) {
            mbar_init(smem_u32(&bars->full_a[i]), 1);
            mbar_init(smem_u32(&bars->empty_a[i]), 1);
        }
        for (int i = 0; i < B_SLOTS; ++i) {
            mbar_init(smem_u32(&bars->full_b[i]), 1);
            mbar_init(smem_u32(&bars->empty_b[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&bars->s_full[i]), 1);
            mbar_init(smem_u32(&bars->p_full[i]), ROWS);
        }
        mbar_init(smem_u32(&bars->o_final), 1);
        bars->abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&bars->tmem_base), TMEM_COLUMNS);
        tmem_relinquish();
    }
    if (warp == LOAD_WARP && lane == 0) {
        tma_prefetch_descriptor(&p.q_lat);
        tma_prefetch_descriptor(&p.q_rope);
        tma_prefetch_descriptor(&p.k_lat);
        tma_prefetch_descriptor(&p.k_rope);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

    // Key chunk c holds columns 64c..64c+63 (c = 8: the rotary columns).  Chunks
    // v_first..v_first+3 are this CTA's V (the "B" group); the matching four Q chunks
    // sit in tensor memory.  The other five key chunks are the "A" group; their Q
    // chunks stay in shared memory.  A tile's S is accumulated A group first
    // (Q from shared memory), B group second (Q from tensor memory): the opposite
    // order on one accumulator costs about three times the issue time.
    const int v_first = half * 4;
    auto a_chunk = [&](int i) -> int { return half == 0 ? 4 + i : (i < 4 ? i : 8); };

    Walker walker;
    walker.done = false;
    Segment seg;
    int segment_index = 0;      // segments this CTA has started (every role counts the same)
    int tile_index = 0;         // key tiles this CTA has started, over all segments

    if (warp == LOAD_WARP) {
        // =================== TMA producer ===================================
        // All 32 lanes walk the loop; lane 0 waits on barriers and issues the loads.
        bool alive = true;
        while (alive && next_segment(p, walker, seg)) {
            const int tile_count = seg.tile_end - seg.tile_begin;
            const int q_row0 = seg.b * p.sequence * p.heads + seg.row_tile * ROWS;
            const uint32_t seg_parity = segment_index & 1;
            if (lane == 0) {
                // Q is staged through the value ring and (three chunks) kept in shared
                // memory: every tile issued so far must have finished its P V.
                for (int back = 1; back <= B_SLOTS && alive; ++back) {
                    const int tile = tile_index - back;
                    if (tile >= 0) {
                        alive = mbar_wait(smem_u32(&bars->empty_b[tile % B_SLOTS]), (tile / B_SLOTS) & 1, abort_flag, &absorbed_status);
                    }
                }
                if (alive) {
                    const uint32_t bar = smem_u32(&bars->q_full);
                    mbar_arrive_expect_tx(bar, Q_SMEM_BYTES);
                    for (int c = 0; c < Q_SMEM_CHUNKS; ++c) {
                        const int chunk = a_chunk(c);
                        if (chunk < 8) {
                            tma_load_2d(q_smem + c * Q_CHUNK_BYTES, &p.q_lat, bar, chunk * 64, q_row0);
                        } else {
                            tma_load_2d(q_smem + c * Q_CHUNK_BYTES, &p.q_rope, bar, 0, q_row0);
                        }
                    }
                    const uint32_t stage_bar = smem_u32(&bars->q_stage_full);
                    mbar_arrive_expect_tx(stage_bar, Q_TMEM_CHUNKS * Q_CHUNK_BYTES);
                    for (int c = 0; c < Q_TMEM_CHUNKS; ++c) {
                        tma_load_2d(b_ring + c * Q_CHUNK_BYTES, &p.q_lat, stage_bar, (v_first + c) * 64, q_row0);
                    }
                }
            }
            alive = __shfl_sync(0xffffffffU, alive ? 1 : 0, 0) != 0;
            for (int j = 0; j < tile_count && alive; ++j) {
                const int token = (seg.tile_begin + j) * KEYS;
                if (lane == 0) {
                    const int tile = tile_index + j;
                    const int y = seg.b * p.sequence + token;
                    // "A" group: free once the S of two tiles ago has been computed
                    const int slot_a = tile % A_SLOTS;
                    if (tile >= A_SLOTS) {
                        alive = mbar_wait(smem_u32(&bars->empty_a[slot_a]), (tile / A_SLOTS - 1) & 1, abort_flag, &absorbed_status);
                    }
                    if (alive) {
                        const uint32_t bar = smem_u32(&bars->full_a[slot_a]);
                        mbar_arrive_expect_tx(bar, A_UNIT_BYTES);
                        for (int i = 0; i < A_CHUNKS; ++i) {
                            const int c = a_chunk(i);
                            const uint32_t dst = a_ring + slot_a * A_UNIT_BYTES + i * K_CHUNK_BYTES;
                            if (c < 8) {
                                tma_load_2d(dst, &p.k_lat, bar, c * 64, y);
                            } else {
                                tma_load_2d(dst, &p.k_rope, bar, 0, y);
                            }
                        }
                    }
                    // "B" group: the first tile of a segment waits for the Q staging to be
                    // consumed, later ones for the P V of three tiles ago
                    const int slot_b = tile % B_SLOTS;
                    if (alive && j == 0) {
                        alive = mbar_wait(smem_u32(&bars->q_tmem_ready), seg_parity, abort_flag, &absorbed_status);
                    } else if (alive && j >= B_SLOTS) {
                        alive = mbar_wait(smem_u32(&bars->empty_b[slot_b]), (tile / B_SLOTS - 1) & 1, abort_flag, &absorbed_status);
                    }
                    if (alive) {
                        const uint32_t bar = smem_u32(&bars->full_b[slot_b]);
                        mbar_arrive_expect_tx(bar, B_UNIT_BYTES);
                        for (int i = 0; i < B_CHUNKS; ++i) {
                            tma_load_2d(b_ring + slot_b * B_UNIT_BYTES + i * K_CHUNK_BYTES, &p.k_lat, bar, (v_first + i) * 64, y);
                        }
                    }
                }
                alive = __shfl_sync(0xffffffffU, alive ? 1 : 0, 0) != 0;
            }
            tile_index += tile_count;
            segment_index += 1;
        }
    } else if (warp == MMA_WARP) {
        // =================== MMA issuer =====================================
        // Whole warp, uniform control flow; the elected lane executes the tcgen05 instructions.
        {
            const uint32_t leader = elect_one();
            constexpr uint32_t IDESC_QK = make_idesc_bf16(ROWS, KEYS, false, false);
            constexpr uint32_t IDESC_PV = make_idesc_bf16(ROWS, HALF_V, false, true);
            constexpr uint32_t HI = smem_desc_hi(1024);
            constexpr uint32_t CHUNK_LO = K_CHUNK_BYTES >> 4;
            const uint32_t q_lo = smem_desc_lo(q_smem, 16);
            const uint32_t a_lo = smem_desc_lo(a_ring, 16);
            const uint32_t b_lo = smem_desc_lo(b_ring, 16);
            const uint32_t v_lo = smem_desc_lo(b_ring, K_CHUNK_BYTES);
            bool alive = true;
            // A group of tile `tile`: five slices with Q from shared memory, starts the accumulator
            auto issue_a_part = [&](int tile) {
                const int slot_a = tile % A_SLOTS;
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->full_a[slot_a]), (tile / A_SLOTS) & 1, abort_flag, &absorbed_status));
                if (!alive) {
                    return;
                }
                tc_fence_after_sync();
                const uint32_t s_tmem = tmem_base + TMEM_S + (tile & 1) * KEYS;
#pragma unroll
                for (int i = 0; i < A_CHUNKS; ++i) {
                    const uint32_t k_lo = a_lo + (slot_a * A_CHUNKS + i) * CHUNK_LO;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        mma_ss_split_elect(s_tmem, q_lo + i * (Q_CHUNK_BYTES >> 4) + 2 * k, HI, k_lo + 2 * k, HI, IDESC_QK, (i | k) != 0 ? 1U : 0U, leader);
                    }
                }
                mma_commit_elect(smem_u32(&bars->empty_a[slot_a]), leader);
            };
            // B group of tile `tile`: four slices with Q from tensor memory, completes S
            auto issue_b_part = [&](int tile) {
                const int slot_b = tile % B_SLOTS;
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->full_b[slot_b]), (tile / B_SLOTS) & 1, abort_flag, &absorbed_status));
                if (!alive) {
                    return;
                }
                tc_fence_after_sync();
                const uint32_t s_tmem = tmem_base + TMEM_S + (tile & 1) * KEYS;
#pragma unroll
                for (int i = 0; i < B_CHUNKS; ++i) {
                    const uint32_t k_lo = b_lo + (slot_b * B_CHUNKS + i) * CHUNK_LO;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        mma_ts_split_elect(s_tmem, tmem_base + TMEM_Q + i * 32 + k * 8, k_lo + 2 * k, HI, IDESC_QK, 1U, leader);
                    }
                }
                mma_commit_elect(smem_u32(&bars->s_full[tile & 1]), leader);
            };
            while (alive && next_segment(p, walker, seg)) {
                const int tile_count = seg.tile_end - seg.tile_begin;
                const uint32_t seg_parity = segment_index & 1;
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->q_full), seg_parity, abort_flag, &absorbed_status) &&
                                                    mbar_wait(smem_u32(&bars->q_tmem_ready), seg_parity, abort_flag, &absorbed_status));
                if (alive) {
                    tc_fence_after_sync();
                    issue_a_part(tile_index);
                }
                if (alive) {
                    issue_b_part(tile_index);
                }
                for (int j = 0; j < tile_count && alive; ++j) {
                    const int tile = tile_index + j;
                    const int slot_b = tile % B_SLOTS;
                    // the next tile's A group runs on the tensor core while this tile's softmax is computed
                    if (j + 1 < tile_count) {
                        issue_a_part(tile + 1);
                        if (!alive) {
                            break;
                        }
                    }
                    // ---- O (+)= P V ----
                    alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->p_full[tile & 1]), (tile >> 1) & 1, abort_flag, &absorbed_status));
                    if (!alive) {
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t p_tmem = tmem_base + TMEM_S + (tile & 1) * KEYS;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        mma_ts_split_elect(tmem_base + TMEM_O, p_tmem + k * 8, v_lo + slot_b * B_CHUNKS * CHUNK_LO + k * (2048 >> 4), HI, IDESC_PV,
                                     (j | k) != 0 ? 1U : 0U, leader);
                    }
                    mma_commit_elect(smem_u32(&bars->empty_b[slot_b]), leader);
                    if (j + 1 < tile_count) {
                        issue_b_part(tile + 1);
                    }
                }
                if (alive) {
                    mma_commit_elect(smem_u32(&bars->o_final), leader);
                }
                tile_index += tile_count;
                segment_index += 1;
            }
        }
    } else {
        // =================== softmax + epilogue =============================
        const int r = threadIdx.x;                       // row of the tile, 0..127
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        const uint32_t o_tmem = tmem_base + lane_base + TMEM_O;
        bool alive = true;

        while (alive && next_segment(p, walker, seg)) {
            const int tile_count = seg.tile_end - seg.tile_begin;
            const uint32_t seg_parity = segment_index & 1;
            int valid_rows;      // rows of the tile that exist
            int kv_end;          // keys >= kv_end are never visible in this segment
            int min_limit;       // smallest per-row key limit; tiles past it need masking
            int limit;           // this row sees keys < limit
            {
                const int rows_total = p.sequence * p.heads;
                const int first = seg.row_tile * ROWS;
                valid_rows = min(ROWS, rows_total - first);
                kv_end = (first + valid_rows - 1) / p.heads + 1;
                min_limit = first / p.heads + 1;
                limit = (first + min(r, valid_rows - 1)) / p.heads + 1;
            }

            // ---- move the four staged Q chunks to tensor memory ---
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->q_stage_full), seg_parity, abort_flag, &absorbed_status));
            if (!alive) {
                break;
            }
            {
#pragma unroll
                for (int c = 0; c < Q_TMEM_CHUNKS; ++c) {
                    uint32_t values[32];
                    const uint8_t* row = b_ring_ptr + c * Q_CHUNK_BYTES + r * 128;
#pragma unroll
                    for (int unit = 0; unit < 8; ++unit) {
                        const uint4 v = *reinterpret_cast<const uint4*>(row + ((unit ^ (r & 7)) * 16));
                        values[unit * 4 + 0] = v.x;
                        values[unit * 4 + 1] = v.y;
                        values[unit * 4 + 2] = v.z;
                        values[unit * 4 + 3] = v.w;
                    }
                    tmem_st_x32(tmem_base + lane_base + TMEM_Q + c * 32, values);
                }
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(smem_u32(&bars->q_tmem_ready));
            }

            float m_ref = 0.0F;
            float l_sum = 0.0F;
            for (int j = 0; j < tile_count && alive; ++j) {
                const int tile = tile_index + j;
                const uint32_t s_tmem = tmem_base + lane_base + TMEM_S + (tile & 1) * KEYS;
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->s_full[tile & 1]), (tile >> 1) & 1, abort_flag, &absorbed_status));
                if (!alive) {
                    break;
                }
                tc_fence_after_sync();
                uint32_t sb[KEYS];
                tmem_ld_x32(s_tmem, sb);
                tmem_ld_x32(s_tmem + 32, sb + 32);
                tmem_wait_ld();
                const int token0 = (seg.tile_begin + j) * KEYS;
                if (token0 + KEYS > min_limit) {
#pragma unroll
                    for (int n = 0; n < KEYS; ++n) {
                        sb[n] = token0 + n < limit ? sb[n] : 0xff800000U;
                    }
                }
                if (token0 + KEYS > kv_end) {
                    // Keys past the end of the tile's visible range belong to the next sequence or lie
                    // outside the tensor; zero their rows so that 0 * V stays 0 in P V.
                    uint8_t* v_rows = b_ring_ptr + (tile % B_SLOTS) * B_UNIT_BYTES;
                    const int first_bad = kv_end - token0;               // 1..63
                    const int bad_units = (KEYS - first_bad) * 8 * 4;    // 16-byte units in 4 chunks
                    for (int u = r; u < bad_units; u += ROWS) {
                        const int chunk = u / ((KEYS - first_bad) * 8);
                        const int within = u % ((KEYS - first_bad) * 8);
                        *reinterpret_cast<uint4*>(v_rows + chunk * K_CHUNK_BYTES + (first_bad + within / 8) * 128 + (within % 8) * 16) =
                            make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();
                }
                // three-input maxima, four independent chains
                float mx0 = __uint_as_float(sb[0]), mx1 = __uint_as_float(sb[1]), mx2 = __uint_as_float(sb[2]), mx3 = __uint_as_float(sb[3]);
#pragma unroll
                for (int n = 4; n + 7 < KEYS; n += 8) {
                    mx0 = max3(mx0, __uint_as_float(sb[n]), __uint_as_float(sb[n + 1]));
                    mx1 = max3(mx1, __uint_as_float(sb[n + 2]), __uint_as_float(sb[n + 3]));
                    mx2 = max3(mx2, __uint_as_float(sb[n + 4]), __uint_as_float(sb[n + 5]));
                    mx3 = max3(mx3, __uint_as_float(sb[n + 6]), __uint_as_float(sb[n + 7]));
                }
                mx0 = max3(mx0, __uint_as_float(sb[KEYS - 4]), __uint_as_float(sb[KEYS - 3]));
                mx1 = max3(mx1, __uint_as_float(sb[KEYS - 2]), __uint_as_float(sb[KEYS - 1]));
                mx0 = fmaxf(mx0, mx2);
                mx1 = fmaxf(mx1, mx3);
                const float tile_max = fmaxf(mx0, mx1);
                if (j == 0) {
                    m_ref = tile_max;
                } else {
                    const bool grow = (tile_max - m_ref) * p.scale_log2 > RESCALE_THRESHOLD;
                    if (__any_sync(0xffffffffU, grow)) {
                        // S of this tile was issued after P V of the previous one, so its
                        // completion implies that O is quiescent here.
                        float alpha = 1.0F;
                        if (grow) {
                            alpha = exp2_approx((m_ref - tile_max) * p.scale_log2);
                            m_ref = tile_max;
                            l_sum *= alpha;
                        }
#pragma unroll
                        for (int c = 0; c < HALF_V / 32; ++c) {
                            uint32_t o[32];
                            tmem_ld_x32(o_tmem + c * 32, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int e = 0; e < 32; ++e) {
                                o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                            }
                            tmem_st_x32(o_tmem + c * 32, o);
                        }
                    }
                }
                const float bias = -m_ref * p.scale_log2;
                // packed fp32 pairs: one FMA and one add per two scores
                float2 sums = make_float2(0.0F, 0.0F);
                const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
                const float2 bias2 = make_float2(bias, bias);
#pragma unroll
                for (int c = 0; c < KEYS / 32; ++c) {
                    uint32_t packed[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const float2 x = fma2(make_float2(__uint_as_float(sb[c * 32 + 2 * e]), __uint_as_float(sb[c * 32 + 2 * e + 1])), scale2, bias2);
                        const float2 pr = make_float2(exp2_approx(x.x), exp2_approx(x.y));
                        sums = add2(sums, pr);
                        packed[e] = pack_bf16x2(pr.x, pr.y);
                    }
                    tmem_st_x16(s_tmem + c * 16, packed);
                }
                const float sum0 = sums.x, sum1 = sums.y;
                l_sum += sum0 + sum1;
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(smem_u32(&bars->p_full[tile & 1]));
            }

            if (alive) {
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->o_final), seg_parity, abort_flag, &absorbed_status));
            }
            if (!alive) {
                break;
            }
            tc_fence_after_sync();
            const bool valid = r < valid_rows;
            {
                const int row = seg.row_tile * ROWS + r;                 // (token, head) index inside the sequence
                const float inverse = 1.0F / l_sum;
                __nv_bfloat16* out_row = p.out + (static_cast<size_t>(seg.b) * p.sequence * p.heads + row) * RANK + half * HALF_V;
#pragma unroll
                for (int c = 0; c < HALF_V / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld_x32(o_tmem + c * 32, o);
                    tmem_wait_ld();
                    if (valid) {
#pragma unroll
                        for (int e = 0; e < 32; e += 8) {
                            uint4 vec;
                            vec.x = pack_bf16x2(__uint_as_float(o[e]) * inverse, __uint_as_float(o[e + 1]) * inverse);
                            vec.y = pack_bf16x2(__uint_as_float(o[e + 2]) * inverse, __uint_as_float(o[e + 3]) * inverse);
                            vec.z = pack_bf16x2(__uint_as_float(o[e + 4]) * inverse, __uint_as_float(o[e + 5]) * inverse);
                            vec.w = pack_bf16x2(__uint_as_float(o[e + 6]) * inverse, __uint_as_float(o[e + 7]) * inverse);
                            *reinterpret_cast<uint4*>(out_row + c * 32 + e) = vec;
                        }
                    }
                }
                if (valid && half == 0) {
                    const int token = row / p.heads;
                    const int head = row % p.heads;
                    p.lse[(static_cast<size_t>(seg.b) * p.heads + head) * p.sequence + token] = m_ref * p.scale + logf(l_sum);
                }
            }
            // the accumulator and the Q columns in tensor memory may be overwritten by
            // the next segment only after every row has been read out
            tc_fence_before_sync();
            tile_index += tile_count;
            segment_index += 1;
        }
    }

    // ---- teardown -----------------------------------------------------------
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

void configure_kernel() {
    static bool done[16] = {};
    int device = 0;
    CUDA_CHECK(cudaGetDevice(&device));
    if (device < 16 && done[device]) {
        return;
    }
    CUDA_CHECK(cudaFuncSetAttribute(absorbed_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    if (device < 16) {
        done[device] = true;
    }
}

void check_absorbed_shape(int kv_rank, int rope_size) {
    // kernels/attention/mla/sm89.cu:20-24 of the reference: same condition, same message.
    if (kv_rank != MLA_KV_RANK || rope_size != MLA_ROPE_SIZE) {
        throw std::invalid_argument("MLA requires C=512 and RoPE=64");
    }
}

void check_aligned(std::initializer_list<const void*> pointers) {
    for (const void* pointer : pointers) {
        if (pointer == nullptr) {
            throw std::invalid_argument("null tensor pointer");
        }
        if ((reinterpret_cast<std::uintptr_t>(pointer) & 15U) != 0) {
            throw std::invalid_argument("tensor pointers must be 16-byte aligned");
        }
    }
}

}  // namespace

namespace internal {


int absorbed_device_status(bool reset) {
    int status = 0;
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemcpyFromSymbol(&status, absorbed_status, sizeof(int)));
    if (reset && status != 0) {
        const int zero = 0;
        CUDA_CHECK(cudaMemcpyToSymbol(absorbed_status, &zero, sizeof(int)));
    }
    return status;
}

}  // namespace internal

void mla_compressed_attention_forward_cuda(__nv_bfloat16* output, float* logsumexp, const __nv_bfloat16* query_latent,
                                           const __nv_bfloat16* query_rope, const __nv_bfloat16* kv_latent, const __nv_bfloat16* key_rope,
                                           int batch_size, int sequence_length, int heads, int kv_rank, int rope_size, float scale,
                                           cudaStream_t stream) {
    check_absorbed_shape(kv_rank, rope_size);
    if (batch_size <= 0 || sequence_length <= 0 || heads <= 0) {
        throw std::invalid_argument("MLA forward requires positive batch, sequence length and heads");
    }
    if (!(scale > 0.0F)) {
        throw std::invalid_argument("MLA forward requires a positive softmax scale");
    }
    const long long rows_per_sequence = static_cast<long long>(sequence_length) * heads;
    if (rows_per_sequence * batch_size > 0x7fffffffLL || batch_size > 65535 || (rows_per_sequence + ROWS - 1) / ROWS * 2 > 65535) {
        throw std::invalid_argument("MLA forward shape exceeds the supported index range");
    }
    check_aligned({output, logsumexp, query_latent, query_rope, kv_latent, key_rope});
    AbsorbedParams params{};
    const std::uint64_t q_rows = static_cast<std::uint64_t>(rows_per_sequence) * batch_size;
    const std::uint64_t k_rows = static_cast<std::uint64_t>(sequence_length) * batch_size;
    params.q_lat = make_bf16_tile_map(query_latent, q_rows, RANK, RANK, ROWS);
    params.q_rope = make_bf16_tile_map(query_rope, q_rows, ROPE, ROPE, ROWS);
    params.k_lat = make_bf16_tile_map(kv_latent, k_rows, RANK, RANK, KEYS);
    params.k_rope = make_bf16_tile_map(key_rope, k_rows, ROPE, ROPE, KEYS);
    params.batch = batch_size;
    params.sequence = sequence_length;
    params.heads = heads;
    params.out = output;
    params.lse = logsumexp;
    params.scale = scale;
    params.scale_log2 = scale * 1.4426950408889634F;
    configure_kernel();
    const dim3 grid(1, static_cast<unsigned>((rows_per_sequence + ROWS - 1) / ROWS * 2), batch_size);
    absorbed_attention_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(params);
    CUDA_CHECK(cudaGetLastError());
}

}  // namespace dscuda
