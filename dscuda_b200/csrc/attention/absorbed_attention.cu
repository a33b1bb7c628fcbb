// Absorbed-latent MLA on sm_100a: every head shares one compressed key/value
// row of 576 bf16 (512 latent + 64 rotary); the latent part is also the value.
// One kernel serves two entry points:
//
//   * causal prefill forward (mla_compressed_attention_forward_cuda): the 128
//     rows of a tile are consecutive (token, head) pairs of one sequence and
//     each row sees keys 0..its token;
//   * paged split-KV decode (mla_decode_forward_cuda): the 128 rows are the
//     heads of one sequence's single query token, keys come from 64-token tiles
//     of the paged cache found through the block table, and each CTA writes an
//     unnormalised partial (max, sum, output) that a second kernel merges.
//
// A 128x512 fp32 output tile would fill all of tensor memory, so a tile is
// handled by two CTAs: both compute S = Q K^T (K = 576) and each accumulates
// one 256-column half of O = P V.  Tensor memory per CTA: O 256 columns, two S
// buffers of 64 columns (P overwrites S in place as bf16), and 128 columns that
// hold the first 256 columns of Q as an MMA A operand, which leaves shared
// memory for the remaining Q columns (80 KB) and two 72 KB key-tile stages.
//
// Warps 0-3: softmax / epilogue (one thread per row); warp 4: MMA issue;
// warp 5: TMA loads.  All waits are bounded.
#include "mla.h"
#include "cuda_common.h"
#include "attention_internal.h"
#include "sm100_primitives.cuh"
#include "../common/tensor_map.h"

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
constexpr int Q_TMEM_CHUNKS = 4;                // Q columns 0..255 live in tensor memory
constexpr int Q_SMEM_CHUNKS = CHUNKS - Q_TMEM_CHUNKS;
constexpr int Q_CHUNK_BYTES = ROWS * 128;       // 16 KB
constexpr int K_CHUNK_BYTES = KEYS * 128;       // 8 KB
constexpr int STAGE_BYTES = CHUNKS * K_CHUNK_BYTES;          // 72 KB
constexpr int Q_SMEM_BYTES = Q_SMEM_CHUNKS * Q_CHUNK_BYTES;  // 80 KB
constexpr int MISC_BYTES = 1024;
constexpr int SMEM_BYTES = Q_SMEM_BYTES + 2 * STAGE_BYTES + MISC_BYTES + 1024;
constexpr int THREADS = 192;
constexpr int MMA_WARP = 4;
constexpr int LOAD_WARP = 5;
constexpr int TMEM_COLUMNS = 512;
constexpr int TMEM_O = 0;                       // 256 columns
constexpr int TMEM_S = 256;                     // 2 x 64 columns
constexpr int TMEM_Q = 384;                     // 128 columns = 4 chunks x 32
constexpr float RESCALE_THRESHOLD = 8.0F;
static_assert(Q_TMEM_CHUNKS * Q_CHUNK_BYTES <= STAGE_BYTES, "Q staging must fit in one key stage");

enum Mode : int { MODE_CAUSAL_PREFILL = 0, MODE_PAGED_DECODE = 1 };

__device__ int absorbed_status = 0;

// Scratch for mla_decode_forward_static_cuda: room for STATIC_DECODE_RECORDS
// split partials of (maximum, sum, 512 outputs).  It lives in the image of the
// library, so every GPU that loads the library keeps these 16.1 MiB until the
// process ends.  The name below is only a host-side handle in host code; the
// device address is looked up once per device with cudaGetSymbolAddress.
constexpr std::size_t STATIC_DECODE_RECORDS = 8192;
static __device__ __align__(256) float decode_static_scratch[STATIC_DECODE_RECORDS * (MLA_KV_RANK + 2)];

struct AbsorbedParams {
    CUtensorMap q_lat;      // [rows, 512] box 128 x 64
    CUtensorMap q_rope;     // [rows, 64]  box 128 x 64
    CUtensorMap k_lat;      // [rows, 512] box 64 x 64
    CUtensorMap k_rope;     // [rows, 64]  box 64 x 64
    int mode;
    int batch;
    int sequence;           // prefill: T
    int heads;
    __nv_bfloat16* out;     // prefill: [B,T,H,512]
    float* lse;             // prefill: [B,H,T]
    const int* block_table; // decode: [B, pages]
    const int* lengths;     // decode: [B]
    float* workspace;       // decode: [B,H,splits,2+512]
    int page_size;
    int pages;
    int splits;
    float scale;
    float scale_log2;
#ifdef DSCUDA_DEBUG_DUMP
    float* debug;           // [128*64 raw S of the first tile][128*258 unnormalised O half, l, m] of CTA (0,0,0)
#endif
};

struct AbsorbedBarriers {
    uint64_t q_full;            // Q chunks that stay in shared memory
    uint64_t q_stage_full;      // Q chunks on their way to tensor memory
    uint64_t q_tmem_ready;      // 128 arrivals: those chunks are in tensor memory
    uint64_t full_a[2];         // per stage: the five key chunks only S needs
    uint64_t full_b[2];         // per stage: the four chunks that are also this CTA's V
    uint64_t empty_a[2];
    uint64_t empty_b[2];
    uint64_t s_full[2];
    uint64_t p_full[2];
    uint64_t o_done;            // one completion per P V
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(AbsorbedBarriers) <= MISC_BYTES, "barrier block too large");

__global__ void __launch_bounds__(THREADS, 1) absorbed_attention_kernel(const __grid_constant__ AbsorbedParams p) {
    extern __shared__ uint8_t smem_raw[];
    if (*reinterpret_cast<volatile int*>(&absorbed_status) != 0) {
        return;
    }
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const int half = blockIdx.y & 1;            // which 256 value columns
    const int row_tile = blockIdx.y >> 1;
    const int b = blockIdx.z;

    // ---- work description --------------------------------------------------
    int q_row0;          // first row of the Q tile in the 2-D Q view
    int valid_rows;      // rows of the tile that exist
    int tile_begin;      // first 64-key tile
    int tile_end;        // one past the last
    int kv_end;          // keys >= kv_end are never visible to this CTA
    int min_limit;       // smallest per-row key limit; tiles past it need masking
    int split = 0;
    if (p.mode == MODE_CAUSAL_PREFILL) {
        const int rows_total = p.sequence * p.heads;
        const int first = row_tile * ROWS;
        q_row0 = b * rows_total + first;
        valid_rows = min(ROWS, rows_total - first);
        const int last_token = (first + valid_rows - 1) / p.heads;
        kv_end = last_token + 1;
        min_limit = first / p.heads + 1;
        tile_begin = 0;
        tile_end = (kv_end + KEYS - 1) / KEYS;
    } else {
        split = blockIdx.x;
        const int first = row_tile * ROWS;
        q_row0 = b * p.heads + first;
        valid_rows = min(ROWS, p.heads - first);
        const int length = p.lengths[b];
        const int tiles_total = (length + KEYS - 1) / KEYS;
        const int per_split = (tiles_total + p.splits - 1) / p.splits;
        tile_begin = min(split * per_split, tiles_total);
        tile_end = min(tile_begin + per_split, tiles_total);
        kv_end = min(length, tile_end * KEYS);
        min_limit = kv_end;
    }
    const int tile_count = tile_end - tile_begin;

    if (tile_count <= 0) {
        // An empty split still owns a partial slot: mark it as carrying no weight.
        if (p.mode == MODE_PAGED_DECODE && half == 0 && threadIdx.x < valid_rows) {
            const int head = row_tile * ROWS + threadIdx.x;
            float* record = p.workspace + ((static_cast<size_t>(b) * p.heads + head) * p.splits + split) * (RANK + 2);
            record[0] = -INFINITY;
            record[1] = 0.0F;
        }
        return;
    }

    // ---- shared memory ------------------------------------------------------
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023U) & ~1023U;
    uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t q_smem = smem_base;
    const uint32_t stage_smem = smem_base + Q_SMEM_BYTES;
    AbsorbedBarriers* bars = reinterpret_cast<AbsorbedBarriers*>(smem_aligned + Q_SMEM_BYTES + 2 * STAGE_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bars->q_full), 1);
        mbar_init(smem_u32(&bars->q_stage_full), 1);
        mbar_init(smem_u32(&bars->q_tmem_ready), ROWS);
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&bars->full_a[i]), 1);
            mbar_init(smem_u32(&bars->full_b[i]), 1);
            mbar_init(smem_u32(&bars->empty_a[i]), 1);
            mbar_init(smem_u32(&bars->empty_b[i]), 1);
            mbar_init(smem_u32(&bars->s_full[i]), 1);
            mbar_init(smem_u32(&bars->p_full[i]), ROWS);
        }
        mbar_init(smem_u32(&bars->o_done), 1);
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

    // first and last (exclusive) chunk of a stage that doubles as this CTA's V
    const int v_first = half * 4;

    if (warp == LOAD_WARP) {
        // =================== TMA producer ===================================
        if (lane == 0) {
            // Q columns 256..575 stay in shared memory.
            {
                const uint32_t bar = smem_u32(&bars->q_full);
                mbar_arrive_expect_tx(bar, Q_SMEM_BYTES);
                for (int c = 0; c < Q_SMEM_CHUNKS; ++c) {
                    const int chunk = Q_TMEM_CHUNKS + c;
                    if (chunk < 8) {
                        tma_load_2d(q_smem + c * Q_CHUNK_BYTES, &p.q_lat, bar, chunk * 64, q_row0);
                    } else {
                        tma_load_2d(q_smem + c * Q_CHUNK_BYTES, &p.q_rope, bar, 0, q_row0);
                    }
                }
            }
            // Q columns 0..255 pass through stage 1 on their way to tensor memory.
            {
                const uint32_t bar = smem_u32(&bars->q_stage_full);
                mbar_arrive_expect_tx(bar, Q_TMEM_CHUNKS * Q_CHUNK_BYTES);
                for (int c = 0; c < Q_TMEM_CHUNKS; ++c) {
                    tma_load_2d(stage_smem + STAGE_BYTES + c * Q_CHUNK_BYTES, &p.q_lat, bar, c * 64, q_row0);
                }
            }
            bool alive = true;
            for (int j = 0; j < tile_count && alive; ++j) {
                const int stage = j & 1;
                if (j == 1) {
                    alive = mbar_wait(smem_u32(&bars->q_tmem_ready), 0, abort_flag, &absorbed_status);
                } else if (j >= 2) {
                    const uint32_t parity = ((j >> 1) - 1) & 1;
                    alive = mbar_wait(smem_u32(&bars->empty_a[stage]), parity, abort_flag, &absorbed_status) &&
                            mbar_wait(smem_u32(&bars->empty_b[stage]), parity, abort_flag, &absorbed_status);
                }
                if (!alive) {
                    break;
                }
                const int token = (tile_begin + j) * KEYS;
                int y;
                if (p.mode == MODE_CAUSAL_PREFILL) {
                    y = b * p.sequence + token;
                } else {
                    const int page = token / p.page_size;
                    y = __ldg(p.block_table + static_cast<size_t>(b) * p.pages + page) * p.page_size + token % p.page_size;
                }
                const uint32_t bar_a = smem_u32(&bars->full_a[stage]);
                const uint32_t bar_b = smem_u32(&bars->full_b[stage]);
                mbar_arrive_expect_tx(bar_a, 5 * K_CHUNK_BYTES);
                mbar_arrive_expect_tx(bar_b, 4 * K_CHUNK_BYTES);
                const uint32_t dst = stage_smem + stage * STAGE_BYTES;
                for (int c = 0; c < CHUNKS; ++c) {
                    const bool is_v = c >= v_first && c < v_first + 4;
                    const uint32_t bar = is_v ? bar_b : bar_a;
                    if (c < 8) {
                        tma_load_2d(dst + c * K_CHUNK_BYTES, &p.k_lat, bar, c * 64, y);
                    } else {
                        tma_load_2d(dst + c * K_CHUNK_BYTES, &p.k_rope, bar, 0, y);
                    }
                }
            }
        }
    } else if (warp == MMA_WARP) {
        // =================== MMA issuer =====================================
        if (lane == 0) {
            constexpr uint32_t IDESC_QK = make_idesc_bf16(ROWS, KEYS, false, false);
            constexpr uint32_t IDESC_PV = make_idesc_bf16(ROWS, HALF_V, false, true);
            bool alive = mbar_wait(smem_u32(&bars->q_full), 0, abort_flag, &absorbed_status) &&
                         mbar_wait(smem_u32(&bars->q_tmem_ready), 0, abort_flag, &absorbed_status);
            auto issue_qk = [&](int j) {
                const int stage = j & 1;
                const uint32_t parity = (j >> 1) & 1;
                alive = mbar_wait(smem_u32(&bars->full_a[stage]), parity, abort_flag, &absorbed_status) &&
                        mbar_wait(smem_u32(&bars->full_b[stage]), parity, abort_flag, &absorbed_status);
                if (!alive) {
                    return;
                }
                tc_fence_after_sync();
                const uint32_t d = tmem_base + TMEM_S + stage * KEYS;
                const uint32_t k_stage = stage_smem + stage * STAGE_BYTES;
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t k_desc = make_kmajor_desc(k_stage + c * K_CHUNK_BYTES + k * 32);
                        const uint32_t accumulate = (c | k) != 0 ? 1U : 0U;
                        if (c < Q_TMEM_CHUNKS) {
                            mma_ts(d, tmem_base + TMEM_Q + c * 32 + k * 8, k_desc, IDESC_QK, accumulate);
                        } else {
                            mma_ss(d, make_kmajor_desc(q_smem + (c - Q_TMEM_CHUNKS) * Q_CHUNK_BYTES + k * 32), k_desc, IDESC_QK,
                                   accumulate);
                        }
                    }
                }
                mma_commit(smem_u32(&bars->s_full[stage]));
                mma_commit(smem_u32(&bars->empty_a[stage]));
            };
            if (alive) {
                issue_qk(0);
            }
            for (int j = 0; j < tile_count && alive; ++j) {
                if (j + 1 < tile_count) {
                    issue_qk(j + 1);
                    if (!alive) {
                        break;
                    }
                }
                const int stage = j & 1;
                alive = mbar_wait(smem_u32(&bars->p_full[stage]), (j >> 1) & 1, abort_flag, &absorbed_status);
                if (!alive) {
                    break;
                }
                tc_fence_after_sync();
                const uint32_t v_smem = stage_smem + stage * STAGE_BYTES + v_first * K_CHUNK_BYTES;
                const uint32_t p_tmem = tmem_base + TMEM_S + stage * KEYS;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    mma_ts(tmem_base + TMEM_O, p_tmem + k * 8, make_smem_desc(v_smem + k * 2048, K_CHUNK_BYTES, 1024), IDESC_PV,
                           (j | k) != 0 ? 1U : 0U);
                }
                mma_commit(smem_u32(&bars->empty_b[stage]));
                mma_commit(smem_u32(&bars->o_done));
            }
        }
    } else {
        // =================== softmax + epilogue =============================
        const int r = threadIdx.x;                       // row of the tile, 0..127
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        const uint32_t o_tmem = tmem_base + lane_base + TMEM_O;
        bool alive = true;

        // ---- move Q columns 0..255 from the staging area to tensor memory ---
        alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->q_stage_full), 0, abort_flag, &absorbed_status));
        if (alive) {
            const uint8_t* staging = smem_aligned + Q_SMEM_BYTES + STAGE_BYTES;
#pragma unroll
            for (int c = 0; c < Q_TMEM_CHUNKS; ++c) {
                uint32_t values[32];
                const uint8_t* row = staging + c * Q_CHUNK_BYTES + r * 128;
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

        // per-row visibility limit: key index < limit
        int limit;
        if (p.mode == MODE_CAUSAL_PREFILL) {
            limit = (row_tile * ROWS + min(r, valid_rows - 1)) / p.heads + 1;
        } else {
            limit = kv_end;
        }
        float m_ref = 0.0F;
        float l_sum = 0.0F;

        for (int j = 0; j < tile_count && alive; ++j) {
            const int stage = j & 1;
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->s_full[stage]), (j >> 1) & 1, abort_flag, &absorbed_status));
            if (!alive) {
                break;
            }
            tc_fence_after_sync();
            const uint32_t s_tmem = tmem_base + lane_base + TMEM_S + stage * KEYS;
            uint32_t sb[KEYS];
            tmem_ld_x32(s_tmem, sb);
            tmem_ld_x32(s_tmem + 32, sb + 32);
            tmem_wait_ld();
#ifdef DSCUDA_DEBUG_DUMP
            if (p.debug != nullptr && j == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
                for (int n = 0; n < KEYS; ++n) {
                    p.debug[r * KEYS + n] = __uint_as_float(sb[n]);
                }
            }
#endif
            const int token0 = (tile_begin + j) * KEYS;
            if (token0 + KEYS > min_limit) {
#pragma unroll
                for (int n = 0; n < KEYS; ++n) {
                    sb[n] = token0 + n < limit ? sb[n] : 0xff800000U;
                }
            }
            if (token0 + KEYS > kv_end) {
                // Keys past the end may hold anything (the cache page is only
                // partly written); zero them so that 0 * V stays 0 in P V.
                uint8_t* v_rows = smem_aligned + Q_SMEM_BYTES + stage * STAGE_BYTES + v_first * K_CHUNK_BYTES;
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
            float mx0 = __uint_as_float(sb[0]), mx1 = __uint_as_float(sb[1]);
#pragma unroll
            for (int n = 2; n < KEYS; n += 2) {
                mx0 = fmaxf(mx0, __uint_as_float(sb[n]));
                mx1 = fmaxf(mx1, __uint_as_float(sb[n + 1]));
            }
            const float tile_max = fmaxf(mx0, mx1);
            if (j == 0) {
                m_ref = tile_max;
            } else {
                const bool grow = (tile_max - m_ref) * p.scale_log2 > RESCALE_THRESHOLD;
                if (__any_sync(0xffffffffU, grow)) {
                    // O must be quiescent: wait for P V of the previous tile.
                    alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->o_done), (j - 1) & 1, abort_flag, &absorbed_status));
                    if (!alive) {
                        break;
                    }
                    tc_fence_after_sync();
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
            float sum0 = 0.0F, sum1 = 0.0F;
#pragma unroll
            for (int c = 0; c < KEYS / 32; ++c) {
                uint32_t packed[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const float p0 = exp2_approx(fmaf(__uint_as_float(sb[c * 32 + 2 * e]), p.scale_log2, bias));
                    const float p1 = exp2_approx(fmaf(__uint_as_float(sb[c * 32 + 2 * e + 1]), p.scale_log2, bias));
                    sum0 += p0;
                    sum1 += p1;
                    packed[e] = pack_bf16x2(p0, p1);
                }
                tmem_st_x16(s_tmem + c * 16, packed);
            }
            l_sum += sum0 + sum1;
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&bars->p_full[stage]));
        }

        if (alive) {
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->o_done), (tile_count - 1) & 1, abort_flag, &absorbed_status));
        }
        if (alive) {
            tc_fence_after_sync();
            const bool valid = r < valid_rows;
#ifdef DSCUDA_DEBUG_DUMP
            if (p.debug != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
                float* dump = p.debug + ROWS * KEYS + r * 258;
                for (int c = 0; c < HALF_V / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld_x32(o_tmem + c * 32, o);
                    tmem_wait_ld();
                    for (int e = 0; e < 32; ++e) {
                        dump[c * 32 + e] = __uint_as_float(o[e]);
                    }
                }
                dump[256] = l_sum;
                dump[257] = m_ref;
            }
#endif
            if (p.mode == MODE_CAUSAL_PREFILL) {
                const int row = row_tile * ROWS + r;                 // (token, head) index inside the sequence
                const float inverse = 1.0F / l_sum;
                __nv_bfloat16* out_row = p.out + (static_cast<size_t>(b) * p.sequence * p.heads + row) * RANK + half * HALF_V;
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
                    p.lse[(static_cast<size_t>(b) * p.heads + head) * p.sequence + token] = m_ref * p.scale + logf(l_sum);
                }
            } else {
                const int head = row_tile * ROWS + r;
                float* record = p.workspace + ((static_cast<size_t>(b) * p.heads + (valid ? head : 0)) * p.splits + split) * (RANK + 2);
                if (valid && half == 0) {
                    record[0] = m_ref * p.scale;
                    record[1] = l_sum;
                }
#pragma unroll
                for (int c = 0; c < HALF_V / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld_x32(o_tmem + c * 32, o);
                    tmem_wait_ld();
                    if (valid) {
                        float2* dst = reinterpret_cast<float2*>(record + 2 + half * HALF_V + c * 32);
#pragma unroll
                        for (int e = 0; e < 32; e += 2) {
                            dst[e / 2] = make_float2(__uint_as_float(o[e]), __uint_as_float(o[e + 1]));
                        }
                    }
                }
            }
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

// Merges the split partials of one (sequence, head): weights exp(m_s - max m),
// normalises, writes bf16 output and the natural-log LSE.
__global__ void __launch_bounds__(128) decode_combine_kernel(__nv_bfloat16* output, float* logsumexp, const float* workspace, int heads,
                                                             int splits) {
    const int row = blockIdx.y * heads + blockIdx.x;
    const float* records = workspace + static_cast<size_t>(row) * splits * (RANK + 2);
    float maximum = -INFINITY;
    for (int s = 0; s < splits; ++s) {
        const float l = records[static_cast<size_t>(s) * (RANK + 2) + 1];
        if (l > 0.0F) {
            maximum = fmaxf(maximum, records[static_cast<size_t>(s) * (RANK + 2)]);
        }
    }
    float normalizer = 0.0F;
    float acc[4] = {0.0F, 0.0F, 0.0F, 0.0F};
    const int column = threadIdx.x * 4;
    for (int s = 0; s < splits; ++s) {
        const float* record = records + static_cast<size_t>(s) * (RANK + 2);
        const float l = record[1];
        if (l > 0.0F) {
            const float weight = __expf(record[0] - maximum);
            normalizer += weight * l;
            const float2 lo = *reinterpret_cast<const float2*>(record + 2 + column);
            const float2 hi = *reinterpret_cast<const float2*>(record + 4 + column);
            acc[0] += weight * lo.x;
            acc[1] += weight * lo.y;
            acc[2] += weight * hi.x;
            acc[3] += weight * hi.y;
        }
    }
    const float inverse = 1.0F / normalizer;
    uint2 packed;
    packed.x = pack_bf16x2(acc[0] * inverse, acc[1] * inverse);
    packed.y = pack_bf16x2(acc[2] * inverse, acc[3] * inverse);
    *reinterpret_cast<uint2*>(output + static_cast<size_t>(row) * RANK + column) = packed;
    if (threadIdx.x == 0) {
        logsumexp[row] = maximum + logf(normalizer);
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

#ifdef DSCUDA_DEBUG_DUMP
float* absorbed_debug_buffer = nullptr;
#endif

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
    params.mode = MODE_CAUSAL_PREFILL;
    params.batch = batch_size;
    params.sequence = sequence_length;
    params.heads = heads;
    params.out = output;
    params.lse = logsumexp;
    params.splits = 1;
    params.page_size = KEYS;
    params.scale = scale;
    params.scale_log2 = scale * 1.4426950408889634F;
#ifdef DSCUDA_DEBUG_DUMP
    params.debug = internal::absorbed_debug_buffer;
#endif
    configure_kernel();
    const dim3 grid(1, static_cast<unsigned>((rows_per_sequence + ROWS - 1) / ROWS * 2), batch_size);
    absorbed_attention_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(params);
    CUDA_CHECK(cudaGetLastError());
}

std::size_t mla_decode_workspace_elements(int batch_size, int heads, int splits, int kv_rank) {
    // kernels/attention/mla/sm89.cu:539-541 of the reference.
    return static_cast<std::size_t>(batch_size) * heads * splits * (kv_rank + 2);
}

void mla_decode_forward_cuda(__nv_bfloat16* output, float* logsumexp, const __nv_bfloat16* query, const __nv_bfloat16* paged_kv_cache,
                             const int* block_table, const int* cache_lengths, float* workspace, int batch_size, int heads, int kv_rank,
                             int rope_size, int page_size, int pages_per_sequence, int splits, float scale, cudaStream_t stream) {
    check_absorbed_shape(kv_rank, rope_size);
    if (batch_size <= 0 || heads <= 0 || pages_per_sequence <= 0 || splits <= 0) {
        throw std::invalid_argument("MLA decode requires positive batch, heads, pages and splits");
    }
    if (page_size <= 0 || page_size % KEYS != 0) {
        throw std::invalid_argument("MLA decode requires page_size to be a positive multiple of 64");
    }
    if (!(scale > 0.0F)) {
        throw std::invalid_argument("MLA decode requires a positive softmax scale");
    }
    if (batch_size > 65535 || splits > 65535 || static_cast<long long>(batch_size) * heads > 0x7fffffffLL) {
        throw std::invalid_argument("MLA decode shape exceeds the supported index range");
    }
    check_aligned({output, logsumexp, query, paged_kv_cache, workspace});
    if (block_table == nullptr || cache_lengths == nullptr) {
        throw std::invalid_argument("null tensor pointer");
    }
    AbsorbedParams params{};
    const std::uint64_t q_rows = static_cast<std::uint64_t>(batch_size) * heads;
    // The number of physical pages is not part of the interface; the view is
    // given the largest row count a tensor map can hold and only rows named by
    // the block table are ever touched.
    const std::uint64_t k_rows = 1ULL << 31;
    params.q_lat = make_bf16_tile_map(query, q_rows, RANK, WIDTH, ROWS);
    params.q_rope = make_bf16_tile_map(query + RANK, q_rows, ROPE, WIDTH, ROWS);
    params.k_lat = make_bf16_tile_map(paged_kv_cache, k_rows, RANK, WIDTH, KEYS);
    params.k_rope = make_bf16_tile_map(paged_kv_cache + RANK, k_rows, ROPE, WIDTH, KEYS);
    params.mode = MODE_PAGED_DECODE;
    params.batch = batch_size;
    params.sequence = 1;
    params.heads = heads;
    params.block_table = block_table;
    params.lengths = cache_lengths;
    params.workspace = workspace;
    params.page_size = page_size;
    params.pages = pages_per_sequence;
    params.splits = splits;
    params.scale = scale;
    params.scale_log2 = scale * 1.4426950408889634F;
#ifdef DSCUDA_DEBUG_DUMP
    params.debug = internal::absorbed_debug_buffer;
#endif
    configure_kernel();
    const dim3 grid(splits, static_cast<unsigned>((heads + ROWS - 1) / ROWS * 2), batch_size);
    absorbed_attention_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(params);
    CUDA_CHECK(cudaGetLastError());
    decode_combine_kernel<<<dim3(heads, batch_size), 128, 0, stream>>>(output, logsumexp, workspace, heads, splits);
    CUDA_CHECK(cudaGetLastError());
}

std::size_t mla_decode_static_capacity() {
    return STATIC_DECODE_RECORDS;
}

void mla_decode_forward_static_cuda(__nv_bfloat16* output, float* logsumexp, const __nv_bfloat16* query,
                                    const __nv_bfloat16* paged_kv_cache, const int* block_table, const int* cache_lengths, int batch_size,
                                    int heads, int kv_rank, int rope_size, int page_size, int pages_per_sequence, int splits, float scale,
                                    cudaStream_t stream) {
    check_absorbed_shape(kv_rank, rope_size);
    if (batch_size <= 0 || heads <= 0 || splits <= 0) {
        throw std::invalid_argument("MLA decode requires positive batch, heads, pages and splits");
    }
    const unsigned long long records = static_cast<unsigned long long>(batch_size) * heads * splits;
    if (records > STATIC_DECODE_RECORDS) {
        throw std::invalid_argument("static-scratch MLA decode holds at most " + std::to_string(STATIC_DECODE_RECORDS) +
                                    " split partials (batch*heads*splits = " + std::to_string(records) +
                                    "); lower splits or use the entry point that takes a workspace");
    }
    // Device address of the scratch array, looked up once per device while that
    // device is current.  The first call on a device does this set-up.
    constexpr int MAX_DEVICES = 64;
    static float* scratch_address[MAX_DEVICES] = {};
    static std::mutex lock;
    int device = 0;
    CUDA_CHECK(cudaGetDevice(&device));
    if (device < 0 || device >= MAX_DEVICES) {
        throw std::runtime_error("static-scratch MLA decode supports device ordinals below 64");
    }
    float* scratch = nullptr;
    {
        std::lock_guard<std::mutex> guard(lock);
        if (scratch_address[device] == nullptr) {
            void* address = nullptr;
            CUDA_CHECK(cudaGetSymbolAddress(&address, decode_static_scratch));
            scratch_address[device] = static_cast<float*>(address);
        }
        scratch = scratch_address[device];
    }
    mla_decode_forward_cuda(output, logsumexp, query, paged_kv_cache, block_table, cache_lengths, scratch, batch_size, heads, kv_rank,
                            rope_size, page_size, pages_per_sequence, splits, scale, stream);
}

}  // namespace dscuda
