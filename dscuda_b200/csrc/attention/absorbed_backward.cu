// Backward of the absorbed-latent causal MLA forward
// (mla_compressed_attention_backward_cuda) on the sm_100a tensor cores.
//
// The interface gives no scratch memory, the gradients of the shared latent /
// rotary key sum over every head and every later query, and the operands are wide
// (576 score columns, 512 value columns), so the work is split the way the
// reference splits it (kernels/attention/mla/sm89.cu:295 query side, :356 key
// side): one kernel owns the key-side gradients, one owns the query-side
// gradients, and each recomputes P from the saved LSE.  Both are tcgen05 kernels
// and share one tile shape: a score tile is S^T = K Q^T with 128 keys on the
// tensor-memory lanes and 64 (token, head) rows on the columns, so that one
// thread owns one key, the per-row constants (LSE, delta, token index) are read
// from shared memory, and P^T / dS^T come out in the form the gradient products
// want.  Wide operands stream through shared memory in 64-column chunks.
//
// One call launches, on the caller's stream:
//   1. absorbed_delta_kernel: delta[row] = sum_c dO[row,c] O[row,c], kept in the
//      first four bytes of each dquery_rope row (an output the last kernel
//      overwrites, so no scratch is needed);
//   2. absorbed_backward_key_kernel: CTA = (128-key tile, one 256-column half of
//      dlatent, one part of the rows).  The key tile (9 chunks, 144 KB) stays in
//      shared memory; the 64-row tiles at or after the diagonal stream by: the 17
//      chunks of query_latent | query_rope | dO give S^T and dP^T = latent dO^T, and
//      the 9 chunks this half needs again stay in the ring until after the
//      softmax, as the B operands of dlatent += dS^T query_latent + P^T dO and
//      dkey_rope += dS^T query_rope (P^T and dS^T are bf16 A operands in tensor
//      memory).  Single writer per output element, no atomics;
//   3. absorbed_backward_query_kernel: CTA = 64 (token, head) rows, resident as the
//      B operands query_latent | query_rope | dO (136 KB); every 128-key tile up
//      to the diagonal streams by twice: for S^T / dP^T, and again as the
//      MN-major A operand of dQ^T += K^T dS^T (output columns on the lanes, rows on
//      the columns; dS^T goes through shared memory as the B operand).
//
// Warps 0-7: softmax (thread = key x 32 of the 64 rows); warp 8: MMA issue (whole
// warp, one elected lane executes); warp 9: TMA loads.  Every wait is bounded.
#include "mla.h"
#include "cuda_common.h"
#include "attention_internal.h"
#include "sm100_primitives.cuh"
#include "../common/tensor_map.h"

#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <stdexcept>

namespace dscuda {
namespace {

using namespace sm100;

constexpr int RANK = MLA_KV_RANK;             // 512
constexpr int ROPE = MLA_ROPE_SIZE;           // 64
constexpr int CHUNKS = (RANK + ROPE) / 64;    // 9 column chunks of 64; chunk 8 is the rotary part
constexpr int LATENT_CHUNKS = RANK / 64;      // 8
constexpr int KEYS = 128;                     // keys per tile = MMA M = tensor-memory lanes
constexpr int ROWS = 64;                      // (token, head) rows per tile = MMA N
constexpr int KEY_CHUNK = KEYS * 128;         // 16 KB: [128 keys x 64 bf16]
constexpr int ROW_CHUNK = ROWS * 128;         //  8 KB: [64 rows x 64 bf16]
constexpr int THREADS = 320;
constexpr int MMA_WARP = 8;
constexpr int LOAD_WARP = 9;
constexpr int TMEM_COLUMNS = 512;
constexpr int MISC_BYTES = 2048;
constexpr float LOG2E = 1.4426950408889634F;

__device__ int absorbed_backward_status = 0;

struct AbsorbedBackwardParams {
    CUtensorMap q_lat;      // [B*T*H, 512] box 64 x 64
    CUtensorMap q_rope;     // [B*T*H, 64]  box 64 x 64
    CUtensorMap d_out;      // [B*T*H, 512] box 64 x 64
    CUtensorMap k_lat;      // [B*T, 512]   box 128 x 64
    CUtensorMap k_rope;     // [B*T, 64]    box 128 x 64
    __nv_bfloat16* dq_lat;  // [B,T,H,512]
    __nv_bfloat16* dq_rope; // [B,T,H,64]; the first float of each row holds delta until the query kernel overwrites it
    __nv_bfloat16* dlatent; // [B,T,512]
    __nv_bfloat16* dk_rope; // [B,T,64]
    const float* lse;       // [B,H,T]
    int batch;
    int sequence;
    int heads;
    int key_chunk;          // key side: at most this many 64-row tiles per CTA
    int key_direct;         // key side: 1 when every key tile has a single part (results go straight to the outputs)
    float scale;
    float scale_log2;
};

// Key side work split.  Key tile kt meets the 64-row tiles from floor(kt*128*H/64) to the end of
// the sequence; that range is cut into ceil(count / key_chunk) parts of equal size, one CTA each,
// so that the first key tiles (which meet every row) do not set the kernel's duration.  With more
// than one part the CTAs write fp32 partial sums, part p of key row (b, key) at
// scratch[((p*B + b)*T + key)*576 ..], and absorbed_backward_reduce_kernel adds them in part
// order.  The scratch is the dquery_latent output, which the query-side kernel overwrites last.
__device__ __forceinline__ int key_tile_row_tiles(const AbsorbedBackwardParams& p, int key_tile) {
    const int rows_per_sequence = p.sequence * p.heads;
    return (rows_per_sequence + 63) / 64 - static_cast<int>((static_cast<long long>(key_tile) * 128 * p.heads) / 64);
}

__device__ __forceinline__ int key_tile_parts(const AbsorbedBackwardParams& p, int key_tile) {
    return (key_tile_row_tiles(p, key_tile) + p.key_chunk - 1) / p.key_chunk;
}

// Per-row constants of a 64-row tile, written by the load warp, read by every softmax thread.
struct RowConstants {
    alignas(16) float lse2[ROWS];     // LSE * log2 e
    alignas(16) float delta[ROWS];
    alignas(16) int token[ROWS];      // token index of the row, -1 for rows past the end of the sequence
};

__device__ __forceinline__ float stored_delta(const AbsorbedBackwardParams& p, size_t global_row) {
    return *reinterpret_cast<const float*>(p.dq_rope + global_row * ROPE);
}

// Lanes of one warp fill the constants of rows [row0, row0 + 64) of sequence `b`.
__device__ __forceinline__ void fill_row_constants(const AbsorbedBackwardParams& p, RowConstants& rc, int b, int row0, int lane) {
    const int rows_per_sequence = p.sequence * p.heads;
#pragma unroll
    for (int e = 0; e < ROWS / 32; ++e) {
        const int n = e * 32 + lane;
        const int row = row0 + n;
        float lse_value = 0.0F, delta_value = 0.0F;
        int token = -1;
        if (row < rows_per_sequence) {
            token = row / p.heads;
            const int head = row - token * p.heads;
            lse_value = p.lse[(static_cast<size_t>(b) * p.heads + head) * p.sequence + token] * LOG2E;
            delta_value = stored_delta(p, static_cast<size_t>(b) * rows_per_sequence + row);
        }
        rc.lse2[n] = lse_value;
        rc.delta[n] = delta_value;
        rc.token[n] = token;
    }
}

// One thread's share of a score tile: key `key_pos` (its tensor-memory lane) against 32 of the
// tile's 64 rows.  Reads S^T and dP^T (fp32) from tensor memory and returns P^T and
// dS^T = P^T (dP^T - delta) scale as packed bf16 pairs.  A key is visible to a row when
// key_pos <= token(row); rows past the end have token -1.
__device__ __forceinline__ void score_tile_share(const AbsorbedBackwardParams& p, uint32_t st_tmem, uint32_t dpt_tmem, const RowConstants& rc,
                                                 int group, int key_pos, bool masked, uint32_t (&p_packed)[16], uint32_t (&ds_packed)[16]) {
    uint32_t sb[32];
    float prob[32];
    tmem_ld_x32(st_tmem, sb);
    tmem_wait_ld();
    const float4* lse4 = reinterpret_cast<const float4*>(rc.lse2 + group * 32);
    const float4* delta4 = reinterpret_cast<const float4*>(rc.delta + group * 32);
    const int4* token4 = reinterpret_cast<const int4*>(rc.token + group * 32);
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
        for (int n = 0; n < 32; n += 4) {
            const int4 t = token4[n / 4];
            prob[n] = key_pos <= t.x ? prob[n] : 0.0F;
            prob[n + 1] = key_pos <= t.y ? prob[n + 1] : 0.0F;
            prob[n + 2] = key_pos <= t.z ? prob[n + 2] : 0.0F;
            prob[n + 3] = key_pos <= t.w ? prob[n + 3] : 0.0F;
        }
    }
#pragma unroll
    for (int n = 0; n < 32; n += 2) {
        p_packed[n / 2] = pack_bf16x2(prob[n], prob[n + 1]);
    }
    tmem_ld_x32(dpt_tmem, sb);
    tmem_wait_ld();
#pragma unroll
    for (int n = 0; n < 32; n += 4) {
        const float4 d = delta4[n / 4];
        ds_packed[n / 2] = pack_bf16x2(prob[n] * (__uint_as_float(sb[n]) - d.x) * p.scale, prob[n + 1] * (__uint_as_float(sb[n + 1]) - d.y) * p.scale);
        ds_packed[n / 2 + 1] =
            pack_bf16x2(prob[n + 2] * (__uint_as_float(sb[n + 2]) - d.z) * p.scale, prob[n + 3] * (__uint_as_float(sb[n + 3]) - d.w) * p.scale);
    }
}

__device__ __forceinline__ void store_bf16x32(__nv_bfloat16* dst, const uint32_t* values) {
#pragma unroll
    for (int e = 0; e < 32; e += 8) {
        uint4 vec;
        vec.x = pack_bf16x2(__uint_as_float(values[e]), __uint_as_float(values[e + 1]));
        vec.y = pack_bf16x2(__uint_as_float(values[e + 2]), __uint_as_float(values[e + 3]));
        vec.z = pack_bf16x2(__uint_as_float(values[e + 4]), __uint_as_float(values[e + 5]));
        vec.w = pack_bf16x2(__uint_as_float(values[e + 6]), __uint_as_float(values[e + 7]));
        *reinterpret_cast<uint4*>(dst + e) = vec;
    }
}

__device__ __forceinline__ void store_f32x32(float* dst, const uint32_t* values) {
#pragma unroll
    for (int e = 0; e < 32; e += 4) {
        *reinterpret_cast<uint4*>(dst + e) = make_uint4(values[e], values[e + 1], values[e + 2], values[e + 3]);
    }
}

// ---------------------------------------------------------------------------
// delta[row] = sum_c dO[row,c] * O[row,c]; one warp per (token, head) row.  The result is parked
// in the first four bytes of the row's dquery_rope output.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) absorbed_delta_kernel(__nv_bfloat16* dq_rope, const __nv_bfloat16* dout, const __nv_bfloat16* out,
                                                             size_t rows) {
    const int lane = threadIdx.x % 32;
    const size_t warp_stride = static_cast<size_t>(gridDim.x) * (blockDim.x / 32);
    for (size_t row = static_cast<size_t>(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32; row < rows; row += warp_stride) {
        float sum = 0.0F;
#pragma unroll
        for (int part = 0; part < 2; ++part) {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(dout + row * RANK) + part * 32 + lane);
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(out + row * RANK) + part * 32 + lane);
            const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 x = __bfloat1622float2(a2[e]), y = __bfloat1622float2(b2[e]);
                sum += x.x * y.x + x.y * y.y;
            }
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            sum += __shfl_xor_sync(0xffffffffU, sum, offset);
        }
        if (lane == 0) {
            *reinterpret_cast<float*>(dq_rope + row * ROPE) = sum;
        }
    }
}

// ---------------------------------------------------------------------------
// Key side.  Tensor memory: dlatent half 0..255, dkey_rope 256..319, S^T 320..383 (P^T overwrites
// it as bf16), dP^T 384..447 (dS^T likewise).  Shared memory: the key tile (9 x 16 KB), a ring of
// five 16 KB units, constants.  A unit is one TMA transaction of one or two 8 KB row chunks.
// Per row tile, nine units in this order: the other half's two query_latent pairs and two dO
// pairs, then this half's two query_latent pairs, query_rope, and this half's two dO pairs.  All
// nine feed S^T / dP^T; the last five (exactly the ring) are not released after that: they stay
// where they are and serve as the B operands of the gradient products after the softmax, so a
// row tile is streamed once (136 KB), and they are released in the order they were loaded.
// ---------------------------------------------------------------------------
namespace ks {
constexpr int RING_SLOTS = 5;
constexpr int SLOT_BYTES = 2 * ROW_CHUNK;
constexpr int RESIDENT_BYTES = CHUNKS * KEY_CHUNK;
constexpr int SMEM_BYTES = RESIDENT_BYTES + RING_SLOTS * SLOT_BYTES + MISC_BYTES + 1024;
constexpr int UNITS_PER_TILE = 9;
constexpr int RETAINED_FROM = 4;          // units 4..8 of a tile are kept for the gradient products
constexpr uint32_t TMEM_DLAT = 0;
constexpr uint32_t TMEM_DROPE = 256;
constexpr uint32_t TMEM_X0 = 320;
constexpr uint32_t TMEM_X1 = 384;
static_assert(SMEM_BYTES <= 232448, "key-side shared memory");

struct Shared {
    uint64_t resident_full;
    uint64_t unit_full[RING_SLOTS];
    uint64_t unit_empty[RING_SLOTS];
    uint64_t rows_ready[2];
    uint64_t s_ready;           // tensor core -> softmax: S^T and dP^T of the tile are complete
    uint64_t p_ready;           // 256 softmax threads: P^T and dS^T are stored
    uint64_t final_full;
    uint32_t tmem_base;
    int abort_flag;
    int masked[2];
    RowConstants rows[2];
};
static_assert(sizeof(Shared) <= MISC_BYTES, "key-side barrier block too large");
}  // namespace ks

__global__ void __launch_bounds__(THREADS, 1) absorbed_backward_key_kernel(const __grid_constant__ AbsorbedBackwardParams p) {
    using namespace ks;
    extern __shared__ uint8_t smem_raw[];
    if (*reinterpret_cast<volatile int*>(&absorbed_backward_status) == STATUS_WAIT_TIMEOUT) {
        return;
    }
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const int b = blockIdx.z;
    const int half = blockIdx.y;                         // which 256 columns of dlatent
    // blockIdx.x counts (key tile, part) pairs, key tile 0 first
    int key_tile = 0, part = static_cast<int>(blockIdx.x), parts = key_tile_parts(p, 0);
    while (part >= parts) {
        part -= parts;
        ++key_tile;
        parts = key_tile_parts(p, key_tile);
    }
    const int key_start = key_tile * KEYS;
    const int rows_per_sequence = p.sequence * p.heads;
    const int tiles_of_key_tile = key_tile_row_tiles(p, key_tile);
    const int first_tile = (rows_per_sequence + ROWS - 1) / ROWS - tiles_of_key_tile +
                           static_cast<int>(static_cast<long long>(part) * tiles_of_key_tile / parts);
    const int tile_count = static_cast<int>(static_cast<long long>(part + 1) * tiles_of_key_tile / parts) -
                           static_cast<int>(static_cast<long long>(part) * tiles_of_key_tile / parts);

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023U) & ~1023U;
    uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t k_smem = smem_base;
    const uint32_t ring = smem_base + RESIDENT_BYTES;
    Shared* sh = reinterpret_cast<Shared*>(smem_aligned + RESIDENT_BYTES + RING_SLOTS * SLOT_BYTES);
    volatile int* abort_flag = &sh->abort_flag;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&sh->resident_full), 1);
        for (int i = 0; i < RING_SLOTS; ++i) {
            mbar_init(smem_u32(&sh->unit_full[i]), 1);
            mbar_init(smem_u32(&sh->unit_empty[i]), 1);
        }
        mbar_init(smem_u32(&sh->rows_ready[0]), 1);
        mbar_init(smem_u32(&sh->rows_ready[1]), 1);
        mbar_init(smem_u32(&sh->s_ready), 1);
        mbar_init(smem_u32(&sh->p_ready), 256);
        mbar_init(smem_u32(&sh->final_full), 1);
        sh->abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&sh->tmem_base), TMEM_COLUMNS);
        tmem_relinquish();
    }
    if (warp == LOAD_WARP && lane == 0) {
        tma_prefetch_descriptor(&p.q_lat);
        tma_prefetch_descriptor(&p.q_rope);
        tma_prefetch_descriptor(&p.d_out);
        tma_prefetch_descriptor(&p.k_lat);
        tma_prefetch_descriptor(&p.k_rope);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&sh->tmem_base);

    if (warp == LOAD_WARP) {
        // =================== TMA producer ===================================
        if (lane == 0) {
            const uint32_t bar = smem_u32(&sh->resident_full);
            mbar_arrive_expect_tx(bar, RESIDENT_BYTES);
            const int y = b * p.sequence + key_start;
            for (int c = 0; c < LATENT_CHUNKS; ++c) {
                tma_load_2d(k_smem + c * KEY_CHUNK, &p.k_lat, bar, c * 64, y);
            }
            tma_load_2d(k_smem + LATENT_CHUNKS * KEY_CHUNK, &p.k_rope, bar, 0, y);
        }
        bool alive = true;
        int unit = 0;                                    // units issued so far
        for (int t = 0; t < tile_count && alive; ++t) {
            const int row0 = (first_tile + t) * ROWS;
            // The constants of tile t-2 (same buffer) were last read before P^T(t-2) was stored,
            // and the ring (5 units) cannot run a whole tile (14 units) ahead of the tensor core.
            fill_row_constants(p, sh->rows[t & 1], b, row0, lane);
            if (lane == 0) {
                sh->masked[t & 1] = (row0 / p.heads < key_start + KEYS - 1 || row0 + ROWS > rows_per_sequence) ? 1 : 0;
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(&sh->rows_ready[t & 1]));
                const int y = b * rows_per_sequence + row0;
                for (int u = 0; u < UNITS_PER_TILE && alive; ++u, ++unit) {
                    const int slot = unit % RING_SLOTS;
                    if (unit >= RING_SLOTS) {
                        alive = mbar_wait(smem_u32(&sh->unit_empty[slot]), (unit / RING_SLOTS - 1) & 1, abort_flag, &absorbed_backward_status);
                        if (!alive) {
                            break;
                        }
                    }
                    const uint32_t full = smem_u32(&sh->unit_full[slot]);
                    const uint32_t dst = ring + slot * SLOT_BYTES;
                    // which tensor and which chunk pair this unit carries
                    const CUtensorMap* map;
                    int chunk;                           // first chunk; -1: the single rotary chunk
                    if (u < 2) {
                        map = &p.q_lat, chunk = 4 * (1 - half) + 2 * u;
                    } else if (u < 4) {
                        map = &p.d_out, chunk = 4 * (1 - half) + 2 * (u - 2);
                    } else if (u < 6) {
                        map = &p.q_lat, chunk = 4 * half + 2 * (u - 4);
                    } else if (u == 6) {
                        map = &p.q_rope, chunk = -1;
                    } else {
                        map = &p.d_out, chunk = 4 * half + 2 * (u - 7);
                    }
                    if (chunk < 0) {
                        mbar_arrive_expect_tx(full, ROW_CHUNK);
                        tma_load_2d(dst, map, full, 0, y);
                    } else {
                        mbar_arrive_expect_tx(full, 2 * ROW_CHUNK);
                        tma_load_2d(dst, map, full, chunk * 64, y);
                        tma_load_2d(dst + ROW_CHUNK, map, full, (chunk + 1) * 64, y);
                    }
                }
            }
            alive = __shfl_sync(0xffffffffU, alive ? 1 : 0, 0) != 0;
            unit = __shfl_sync(0xffffffffU, unit, 0);
        }
    } else if (warp == MMA_WARP) {
        // =================== MMA issuer (whole warp, elected lane executes) ==
        const uint32_t leader = elect_one();
        constexpr uint32_t IDESC_SCORE = make_idesc_bf16(KEYS, ROWS, false, false);
        constexpr uint32_t IDESC_GRAD = make_idesc_bf16(KEYS, 128, false, true);      // B = two row chunks side by side, MN-major
        constexpr uint32_t IDESC_ROPE = make_idesc_bf16(KEYS, 64, false, true);
        bool alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->resident_full), 0, abort_flag, &absorbed_backward_status));
        for (int t = 0; t < tile_count && alive; ++t) {
            const int base = t * UNITS_PER_TILE;         // number of the tile's first unit
            // ---- S^T = K Q^T (9 chunks), dP^T = latent dO^T (8 chunks) ----
            for (int u = 0; u < UNITS_PER_TILE && alive; ++u) {
                const int slot = (base + u) % RING_SLOTS;
                alive = __all_sync(0xffffffffU,
                                   mbar_wait(smem_u32(&sh->unit_full[slot]), ((base + u) / RING_SLOTS) & 1, abort_flag, &absorbed_backward_status));
                if (!alive) {
                    break;
                }
                tc_fence_after_sync();
                const uint32_t src = ring + slot * SLOT_BYTES;
                const bool is_dout = (u >= 2 && u < 4) || u >= 7;
                int first_chunk, chunks_here = 2;
                if (u < 2) {
                    first_chunk = 4 * (1 - half) + 2 * u;
                } else if (u < 4) {
                    first_chunk = 4 * (1 - half) + 2 * (u - 2);
                } else if (u < 6) {
                    first_chunk = 4 * half + 2 * (u - 4);
                } else if (u == 6) {
                    first_chunk = LATENT_CHUNKS, chunks_here = 1;
                } else {
                    first_chunk = 4 * half + 2 * (u - 7);
                }
                const uint32_t acc = tmem_base + (is_dout ? TMEM_X1 : TMEM_X0);
                for (int cc = 0; cc < chunks_here; ++cc) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const bool first = (u == 0 || u == 2) && cc == 0 && k == 0;
                        mma_ss_elect(acc, make_kmajor_desc(k_smem + (first_chunk + cc) * KEY_CHUNK + k * 32),
                                     make_kmajor_desc(src + cc * ROW_CHUNK + k * 32), IDESC_SCORE, first ? 0U : 1U, leader);
                    }
                }
                if (u < RETAINED_FROM) {
                    mma_commit_elect(smem_u32(&sh->unit_empty[slot]), leader);
                }
            }
            if (!alive) {
                break;
            }
            mma_commit_elect(smem_u32(&sh->s_ready), leader);
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->p_ready), t & 1, abort_flag, &absorbed_backward_status));
            if (!alive) {
                break;
            }
            tc_fence_after_sync();
            // ---- gradient products on the five retained units, in the order they were loaded:
            //      dlatent half += dS^T query_latent (2 units), dkey_rope += dS^T query_rope,
            //      dlatent half += P^T dO (2 units) ----
            for (int u = RETAINED_FROM; u < UNITS_PER_TILE; ++u) {
                const int slot = (base + u) % RING_SLOTS;
                const uint32_t src = ring + slot * SLOT_BYTES;
                if (u == 6) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        mma_ts_elect(tmem_base + TMEM_DROPE, tmem_base + TMEM_X1 + (k / 2) * 32 + (k % 2) * 8, make_smem_desc(src + k * 2048, ROW_CHUNK, 1024),
                                     IDESC_ROPE, (t | k) != 0 ? 1U : 0U, leader);
                    }
                } else {
                    const bool from_dout = u >= 7;
                    const uint32_t operand = tmem_base + (from_dout ? TMEM_X0 : TMEM_X1);     // P^T for dO, dS^T for query_latent
                    const uint32_t acc = tmem_base + TMEM_DLAT + ((from_dout ? u - 7 : u - 4) & 1) * 128;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        mma_ts_elect(acc, operand + (k / 2) * 32 + (k % 2) * 8, make_smem_desc(src + k * 2048, ROW_CHUNK, 1024), IDESC_GRAD,
                                     (from_dout || t != 0 || k != 0) ? 1U : 0U, leader);
                    }
                }
                mma_commit_elect(smem_u32(&sh->unit_empty[slot]), leader);
            }
        }
        if (alive) {
            mma_commit_elect(smem_u32(&sh->final_full), leader);
        }
    } else {
        // =================== softmax: thread = (key, 32 of the 64 rows) ======
        const int group = warp / 4;
        const int r = threadIdx.x % KEYS;
        const uint32_t lane_base = static_cast<uint32_t>((warp % 4) * 32) << 16;
        const int key_pos = key_start + r;
        const uint32_t st_tmem = tmem_base + lane_base + TMEM_X0 + group * 32;
        const uint32_t dpt_tmem = tmem_base + lane_base + TMEM_X1 + group * 32;
        bool alive = true;
        for (int t = 0; t < tile_count; ++t) {
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->rows_ready[t & 1]), (t >> 1) & 1, abort_flag, &absorbed_backward_status) &&
                                                mbar_wait(smem_u32(&sh->s_ready), t & 1, abort_flag, &absorbed_backward_status));
            if (!alive) {
                break;
            }
            tc_fence_after_sync();
            uint32_t p_packed[16], ds_packed[16];
            score_tile_share(p, st_tmem, dpt_tmem, sh->rows[t & 1], group, key_pos, sh->masked[t & 1] != 0, p_packed, ds_packed);
            tmem_st_x16(st_tmem, p_packed);
            tmem_st_x16(dpt_tmem, ds_packed);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&sh->p_ready));
        }
        if (alive) {
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->final_full), 0, abort_flag, &absorbed_backward_status));
        }
        if (alive) {
            tc_fence_after_sync();
            const bool valid = key_pos < p.sequence;
            const size_t key_row = static_cast<size_t>(b) * p.sequence + key_pos;
            // group g handles dlatent columns 128g..128g+127 of this half and dkey_rope columns 32g..32g+31
            __nv_bfloat16* dlat_row = p.dlatent + key_row * RANK + half * 256 + group * 128;
            float* partial_row = reinterpret_cast<float*>(p.dq_lat) +
                                 ((static_cast<size_t>(part) * p.batch + b) * p.sequence + key_pos) * (RANK + ROPE);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t values[32];
                tmem_ld_x32(tmem_base + lane_base + TMEM_DLAT + group * 128 + c * 32, values);
                tmem_wait_ld();
                if (valid && p.key_direct != 0) {
                    store_bf16x32(dlat_row + c * 32, values);
                } else if (valid) {
                    store_f32x32(partial_row + half * 256 + group * 128 + c * 32, values);
                }
            }
            if (half == 0) {
                uint32_t values[32];
                tmem_ld_x32(tmem_base + lane_base + TMEM_DROPE + group * 32, values);
                tmem_wait_ld();
                if (valid && p.key_direct != 0) {
                    store_bf16x32(p.dk_rope + key_row * ROPE + group * 32, values);
                } else if (valid) {
                    store_f32x32(partial_row + RANK + group * 32, values);
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
// Adds the key side's fp32 partial sums of one key row, in part order (so the result does not
// depend on scheduling), and writes bf16 dlatent / dkey_rope.  One CTA of 144 threads per key
// row, four columns per thread.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(144) absorbed_backward_reduce_kernel(const __grid_constant__ AbsorbedBackwardParams p) {
    const int key = blockIdx.x;
    const int b = blockIdx.y;
    const int parts = key_tile_parts(p, key / KEYS);
    const float* scratch = reinterpret_cast<const float*>(p.dq_lat);
    const int column = threadIdx.x * 4;
    float4 sum = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
    for (int part = 0; part < parts; ++part) {
        const float4 v = *reinterpret_cast<const float4*>(scratch + ((static_cast<size_t>(part) * p.batch + b) * p.sequence + key) * (RANK + ROPE) + column);
        sum.x += v.x;
        sum.y += v.y;
        sum.z += v.z;
        sum.w += v.w;
    }
    uint2 packed;
    packed.x = pack_bf16x2(sum.x, sum.y);
    packed.y = pack_bf16x2(sum.z, sum.w);
    const size_t key_row = static_cast<size_t>(b) * p.sequence + key;
    if (column < RANK) {
        *reinterpret_cast<uint2*>(p.dlatent + key_row * RANK + column) = packed;
    } else {
        *reinterpret_cast<uint2*>(p.dk_rope + key_row * ROPE + (column - RANK)) = packed;
    }
}

// ---------------------------------------------------------------------------
// Query side.  Tensor memory: dQ^T as five 64-column blocks at 0..319 (block m holds output
// columns 128m..128m+127 on the lanes and the 64 rows on the columns; block 4 is the rotary part
// on lanes 0..63), S^T 320..383, dP^T 384..447.  Shared memory: the 64 rows' query_latent (8
// chunks), query_rope (1) and dO (8) as 8 KB K-major chunks, a 16 KB dS^T tile (the MN-major B
// operand of dQ^T += K^T dS^T), a ring of two 32 KB units (pairs of 16 KB key chunks), constants.
// Per key tile: 5 units (chunk pairs 0-1 .. 6-7, then the rotary chunk alone) for S^T and dP^T,
// the softmax, and the same 5 units again as the MN-major A operand of the gradient product.
// The rotary unit's second half is whatever the slot held before: its products land on lanes
// 64..127 of block 4, which nothing reads.
// ---------------------------------------------------------------------------
namespace qs {
constexpr int RING_SLOTS = 2;
constexpr int SLOT_BYTES = 2 * KEY_CHUNK;
constexpr int Q_BYTES = CHUNKS * ROW_CHUNK;
constexpr int DO_BYTES = LATENT_CHUNKS * ROW_CHUNK;
constexpr int DS_BYTES = KEYS * 128;
constexpr int SMEM_BYTES = Q_BYTES + DO_BYTES + DS_BYTES + RING_SLOTS * SLOT_BYTES + MISC_BYTES + 1024;
constexpr int UNITS_PER_TILE = 10;
constexpr uint32_t TMEM_DQT = 0;
constexpr uint32_t TMEM_X0 = 320;
constexpr uint32_t TMEM_X1 = 384;
static_assert(SMEM_BYTES <= 232448, "query-side shared memory");

struct Shared {
    uint64_t resident_full;
    uint64_t unit_full[RING_SLOTS];
    uint64_t unit_empty[RING_SLOTS];
    uint64_t rows_ready;
    uint64_t s_ready;
    uint64_t ds_ready;          // 256 softmax threads: dS^T is in shared memory
    uint64_t final_full;
    uint32_t tmem_base;
    int abort_flag;
    RowConstants rows;
};
static_assert(sizeof(Shared) <= MISC_BYTES, "query-side barrier block too large");
}  // namespace qs

__global__ void __launch_bounds__(THREADS, 1) absorbed_backward_query_kernel(const __grid_constant__ AbsorbedBackwardParams p) {
    using namespace qs;
    extern __shared__ uint8_t smem_raw[];
    if (*reinterpret_cast<volatile int*>(&absorbed_backward_status) == STATUS_WAIT_TIMEOUT) {
        return;
    }
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const int b = blockIdx.z;
    const int rows_per_sequence = p.sequence * p.heads;
    const int row0 = static_cast<int>(gridDim.x - 1 - blockIdx.x) * ROWS;       // late rows see the most keys: longest first
    const int last_row = min(row0 + ROWS, rows_per_sequence) - 1;
    const int first_token = row0 / p.heads;
    const int tile_count = (last_row / p.heads) / KEYS + 1;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023U) & ~1023U;
    uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t q_smem = smem_base;
    const uint32_t do_smem = q_smem + Q_BYTES;
    const uint32_t ds_smem = do_smem + DO_BYTES;
    uint8_t* ds_ptr = smem_aligned + Q_BYTES + DO_BYTES;
    const uint32_t ring = ds_smem + DS_BYTES;
    Shared* sh = reinterpret_cast<Shared*>(smem_aligned + Q_BYTES + DO_BYTES + DS_BYTES + RING_SLOTS * SLOT_BYTES);
    volatile int* abort_flag = &sh->abort_flag;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&sh->resident_full), 1);
        for (int i = 0; i < RING_SLOTS; ++i) {
            mbar_init(smem_u32(&sh->unit_full[i]), 1);
            mbar_init(smem_u32(&sh->unit_empty[i]), 1);
        }
        mbar_init(smem_u32(&sh->rows_ready), 1);
        mbar_init(smem_u32(&sh->s_ready), 1);
        mbar_init(smem_u32(&sh->ds_ready), 256);
        mbar_init(smem_u32(&sh->final_full), 1);
        sh->abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&sh->tmem_base), TMEM_COLUMNS);
        tmem_relinquish();
    }
    if (warp == LOAD_WARP && lane == 0) {
        tma_prefetch_descriptor(&p.q_lat);
        tma_prefetch_descriptor(&p.q_rope);
        tma_prefetch_descriptor(&p.d_out);
        tma_prefetch_descriptor(&p.k_lat);
        tma_prefetch_descriptor(&p.k_rope);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&sh->tmem_base);

    if (warp == LOAD_WARP) {
        // =================== TMA producer ===================================
        fill_row_constants(p, sh->rows, b, row0, lane);
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(smem_u32(&sh->rows_ready));
            const uint32_t bar = smem_u32(&sh->resident_full);
            mbar_arrive_expect_tx(bar, Q_BYTES + DO_BYTES);
            const int y = b * rows_per_sequence + row0;
            for (int c = 0; c < LATENT_CHUNKS; ++c) {
                tma_load_2d(q_smem + c * ROW_CHUNK, &p.q_lat, bar, c * 64, y);
                tma_load_2d(do_smem + c * ROW_CHUNK, &p.d_out, bar, c * 64, y);
            }
            tma_load_2d(q_smem + LATENT_CHUNKS * ROW_CHUNK, &p.q_rope, bar, 0, y);
            bool alive = true;
            int unit = 0;
            for (int j = 0; j < tile_count && alive; ++j) {
                const int ky = b * p.sequence + j * KEYS;
                for (int u = 0; u < UNITS_PER_TILE && alive; ++u, ++unit) {
                    const int slot = unit % RING_SLOTS;
                    if (unit >= RING_SLOTS) {
                        alive = mbar_wait(smem_u32(&sh->unit_empty[slot]), (unit / RING_SLOTS - 1) & 1, abort_flag, &absorbed_backward_status);
                        if (!alive) {
                            break;
                        }
                    }
                    const uint32_t full = smem_u32(&sh->unit_full[slot]);
                    const uint32_t dst = ring + slot * SLOT_BYTES;
                    const int pair = u % 5;
                    if (pair == 4) {
                        mbar_arrive_expect_tx(full, KEY_CHUNK);
                        tma_load_2d(dst, &p.k_rope, full, 0, ky);
                    } else {
                        mbar_arrive_expect_tx(full, 2 * KEY_CHUNK);
                        tma_load_2d(dst, &p.k_lat, full, pair * 128, ky);
                        tma_load_2d(dst + KEY_CHUNK, &p.k_lat, full, pair * 128 + 64, ky);
                    }
                }
            }
        }
    } else if (warp == MMA_WARP) {
        // =================== MMA issuer (whole warp, elected lane executes) ==
        const uint32_t leader = elect_one();
        constexpr uint32_t IDESC_SCORE = make_idesc_bf16(KEYS, ROWS, false, false);
        constexpr uint32_t IDESC_DQT = make_idesc_bf16(128, ROWS, true, true);        // A = key chunks MN-major, B = dS^T MN-major
        bool alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->resident_full), 0, abort_flag, &absorbed_backward_status));
        int unit = 0;
        auto wait_unit = [&]() -> uint32_t {
            const int slot = unit % RING_SLOTS;
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->unit_full[slot]), (unit / RING_SLOTS) & 1, abort_flag, &absorbed_backward_status));
            tc_fence_after_sync();
            return ring + slot * SLOT_BYTES;
        };
        auto release_unit = [&]() {
            mma_commit_elect(smem_u32(&sh->unit_empty[unit % RING_SLOTS]), leader);
            ++unit;
        };
        for (int j = 0; j < tile_count && alive; ++j) {
            // ---- S^T = K Q^T, dP^T = latent dO^T ----
            for (int u = 0; u < 5 && alive; ++u) {
                const uint32_t src = wait_unit();
                if (!alive) {
                    break;
                }
                const int chunks_here = u == 4 ? 1 : 2;
                for (int cc = 0; cc < chunks_here; ++cc) {
                    const int chunk = 2 * u + cc;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        mma_ss_elect(tmem_base + TMEM_X0, make_kmajor_desc(src + cc * KEY_CHUNK + k * 32), make_kmajor_desc(q_smem + chunk * ROW_CHUNK + k * 32),
                                     IDESC_SCORE, (chunk | k) != 0 ? 1U : 0U, leader);
                    }
                    if (chunk < LATENT_CHUNKS) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            mma_ss_elect(tmem_base + TMEM_X1, make_kmajor_desc(src + cc * KEY_CHUNK + k * 32),
                                         make_kmajor_desc(do_smem + chunk * ROW_CHUNK + k * 32), IDESC_SCORE, (chunk | k) != 0 ? 1U : 0U, leader);
                        }
                    }
                }
                release_unit();
            }
            if (!alive) {
                break;
            }
            // this commit also covers the gradient products of the previous tile, the last readers of the dS^T tile
            mma_commit_elect(smem_u32(&sh->s_ready), leader);
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->ds_ready), j & 1, abort_flag, &absorbed_backward_status));
            if (!alive) {
                break;
            }
            tc_fence_after_sync();
            // ---- dQ^T block m += (key chunks 2m, 2m+1)^T dS^T ----
            for (int m = 0; m < 5 && alive; ++m) {
                const uint32_t src = wait_unit();
                if (!alive) {
                    break;
                }
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    mma_ss_elect(tmem_base + TMEM_DQT + m * ROWS, make_smem_desc(src + k * 2048, KEY_CHUNK, 1024), make_smem_desc(ds_smem + k * 2048, 16, 1024),
                                 IDESC_DQT, (j | k) != 0 ? 1U : 0U, leader);
                }
                release_unit();
            }
        }
        if (alive) {
            mma_commit_elect(smem_u32(&sh->final_full), leader);
        }
    } else {
        // =================== softmax: thread = (key, 32 of the 64 rows) ======
        const int group = warp / 4;
        const int r = threadIdx.x % KEYS;
        const uint32_t lane_base = static_cast<uint32_t>((warp % 4) * 32) << 16;
        const uint32_t st_tmem = tmem_base + lane_base + TMEM_X0 + group * 32;
        const uint32_t dpt_tmem = tmem_base + lane_base + TMEM_X1 + group * 32;
        const bool ragged = row0 + ROWS > rows_per_sequence;
        bool alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->rows_ready), 0, abort_flag, &absorbed_backward_status));
        for (int j = 0; j < tile_count && alive; ++j) {
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->s_ready), j & 1, abort_flag, &absorbed_backward_status));
            if (!alive) {
                break;
            }
            tc_fence_after_sync();
            const int key_pos = j * KEYS + r;
            const bool masked = ragged || j * KEYS + KEYS - 1 > first_token;
            uint32_t p_packed[16], ds_packed[16];
            score_tile_share(p, st_tmem, dpt_tmem, sh->rows, group, key_pos, masked, p_packed, ds_packed);
            // row r of the MN-major tile: 64 rows = eight 16-byte units, swizzled by the key index
            uint8_t* row = ds_ptr + r * 128;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int unit16 = group * 4 + i;
                *reinterpret_cast<uint4*>(row + ((unit16 ^ (r & 7)) * 16)) =
                    make_uint4(ds_packed[4 * i], ds_packed[4 * i + 1], ds_packed[4 * i + 2], ds_packed[4 * i + 3]);
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&sh->ds_ready));
        }
        if (alive) {
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->final_full), 0, abort_flag, &absorbed_backward_status));
        }
        if (alive) {
            tc_fence_after_sync();
            // thread = output column (lane r of block m), values = rows 32*group .. 32*group+31
            const size_t first_global_row = static_cast<size_t>(b) * rows_per_sequence + row0 + group * 32;
            const int rows_here = min(32, rows_per_sequence - (row0 + group * 32));
#pragma unroll
            for (int m = 0; m < 5; ++m) {
                uint32_t values[32];
                tmem_ld_x32(tmem_base + lane_base + TMEM_DQT + m * ROWS + group * 32, values);
                tmem_wait_ld();
                if (m < 4) {
                    __nv_bfloat16* dst = p.dq_lat + first_global_row * RANK + m * 128 + r;
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        if (e < rows_here) {
                            dst[static_cast<size_t>(e) * RANK] = __float2bfloat16(__uint_as_float(values[e]));
                        }
                    }
                } else if (r < ROPE) {
                    __nv_bfloat16* dst = p.dq_rope + first_global_row * ROPE + r;
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        if (e < rows_here) {
                            dst[static_cast<size_t>(e) * ROPE] = __float2bfloat16(__uint_as_float(values[e]));
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

int multiprocessors() {
    static int cached[64] = {};
    int device = 0;
    CUDA_CHECK(cudaGetDevice(&device));
    if (device >= 0 && device < 64 && cached[device] > 0) {
        return cached[device];
    }
    int count = 0;
    CUDA_CHECK(cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device));
    if (device >= 0 && device < 64) {
        cached[device] = count;
    }
    return count > 0 ? count : 148;
}

void configure_kernels() {
    static bool done[16] = {};
    int device = 0;
    CUDA_CHECK(cudaGetDevice(&device));
    if (device < 16 && done[device]) {
        return;
    }
    CUDA_CHECK(cudaFuncSetAttribute(absorbed_backward_key_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ks::SMEM_BYTES));
    CUDA_CHECK(cudaFuncSetAttribute(absorbed_backward_query_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, qs::SMEM_BYTES));
    if (device < 16) {
        done[device] = true;
    }
}

}  // namespace

namespace internal {

int absorbed_backward_device_status(bool reset) {
    int status = 0;
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemcpyFromSymbol(&status, absorbed_backward_status, sizeof(int)));
    if (reset && status != 0) {
        const int zero = 0;
        CUDA_CHECK(cudaMemcpyToSymbol(absorbed_backward_status, &zero, sizeof(int)));
    }
    return status;
}

}  // namespace internal

void mla_compressed_attention_backward_cuda(__nv_bfloat16* dquery_latent, __nv_bfloat16* dquery_rope, __nv_bfloat16* dkv_latent,
                                            __nv_bfloat16* dkey_rope, const __nv_bfloat16* output_gradient, const __nv_bfloat16* output,
                                            const float* logsumexp, const __nv_bfloat16* query_latent, const __nv_bfloat16* query_rope,
                                            const __nv_bfloat16* kv_latent, const __nv_bfloat16* key_rope, int batch_size, int sequence_length,
                                            int heads, int kv_rank, int rope_size, float scale, cudaStream_t stream) {
    // kernels/attention/mla/sm89.cu:20-24 of the reference: same condition, same message.
    if (kv_rank != MLA_KV_RANK || rope_size != MLA_ROPE_SIZE) {
        throw std::invalid_argument("MLA requires C=512 and RoPE=64");
    }
    if (batch_size <= 0 || sequence_length <= 0 || heads <= 0) {
        throw std::invalid_argument("MLA backward requires positive batch, sequence length and heads");
    }
    if (!(scale > 0.0F)) {
        throw std::invalid_argument("MLA backward requires a positive softmax scale");
    }
    const long long rows_per_sequence = static_cast<long long>(sequence_length) * heads;
    if (rows_per_sequence * batch_size > 0x7fffffffLL || batch_size > 65535) {
        throw std::invalid_argument("MLA backward shape exceeds the supported index range");
    }
    for (const void* pointer : {static_cast<const void*>(dquery_latent), static_cast<const void*>(dquery_rope), static_cast<const void*>(dkv_latent),
                                static_cast<const void*>(dkey_rope), static_cast<const void*>(output_gradient), static_cast<const void*>(output),
                                static_cast<const void*>(logsumexp), static_cast<const void*>(query_latent), static_cast<const void*>(query_rope),
                                static_cast<const void*>(kv_latent), static_cast<const void*>(key_rope)}) {
        if (pointer == nullptr) {
            throw std::invalid_argument("null tensor pointer");
        }
        if ((reinterpret_cast<std::uintptr_t>(pointer) & 15U) != 0) {
            throw std::invalid_argument("tensor pointers must be 16-byte aligned");
        }
    }
    AbsorbedBackwardParams params{};
    const std::uint64_t q_rows = static_cast<std::uint64_t>(rows_per_sequence) * batch_size;
    const std::uint64_t k_rows = static_cast<std::uint64_t>(sequence_length) * batch_size;
    params.q_lat = make_bf16_tile_map(query_latent, q_rows, RANK, RANK, ROWS);
    params.q_rope = make_bf16_tile_map(query_rope, q_rows, ROPE, ROPE, ROWS);
    params.d_out = make_bf16_tile_map(output_gradient, q_rows, RANK, RANK, ROWS);
    params.k_lat = make_bf16_tile_map(kv_latent, k_rows, RANK, RANK, KEYS);
    params.k_rope = make_bf16_tile_map(key_rope, k_rows, ROPE, ROPE, KEYS);
    params.dq_lat = dquery_latent;
    params.dq_rope = dquery_rope;
    params.dlatent = dkv_latent;
    params.dk_rope = dkey_rope;
    params.lse = logsumexp;
    params.batch = batch_size;
    params.sequence = sequence_length;
    params.heads = heads;
    params.scale = scale;
    params.scale_log2 = scale * LOG2E;
    configure_kernels();

    const std::size_t rows = static_cast<std::size_t>(q_rows);
    const unsigned delta_blocks = static_cast<unsigned>(rows / 8 + 1 < 148 * 16 ? rows / 8 + 1 : 148 * 16);
    absorbed_delta_kernel<<<delta_blocks, 256, 0, stream>>>(dquery_rope, output_gradient, output, rows);
    CUDA_CHECK(cudaGetLastError());
    // Key side split (see key_tile_parts): about four waves of CTAs of equal length, never more
    // parts per key tile than fp32 partial rows fit into the dquery_latent buffer.
    const int key_tiles = (sequence_length + KEYS - 1) / KEYS;
    const long long row_tiles = (rows_per_sequence + ROWS - 1) / ROWS;
    auto tiles_of = [&](int key_tile) { return row_tiles - (static_cast<long long>(key_tile) * KEYS * heads) / ROWS; };
    long long tile_units = 0;
    for (int kt = 0; kt < key_tiles; ++kt) {
        tile_units += tiles_of(kt);
    }
    const int sms = multiprocessors();
    const long long max_parts = std::max<long long>(1, std::min<long long>(64, static_cast<long long>(heads) * RANK * 2 / ((RANK + ROPE) * 4)));
    long long chunk = std::max<long long>(16, (2 * batch_size * tile_units + 4LL * sms - 1) / (4LL * sms));
    chunk = std::max(chunk, (row_tiles + max_parts - 1) / max_parts);
    long long part_count = 0;
    for (int kt = 0; kt < key_tiles; ++kt) {
        part_count += (tiles_of(kt) + chunk - 1) / chunk;
    }
    params.key_chunk = static_cast<int>(std::min<long long>(chunk, 0x7fffffffLL));
    params.key_direct = part_count == key_tiles ? 1 : 0;
    const dim3 key_grid(static_cast<unsigned>(part_count), 2, batch_size);
    absorbed_backward_key_kernel<<<key_grid, THREADS, ks::SMEM_BYTES, stream>>>(params);
    CUDA_CHECK(cudaGetLastError());
    if (params.key_direct == 0) {
        absorbed_backward_reduce_kernel<<<dim3(sequence_length, batch_size), 144, 0, stream>>>(params);
        CUDA_CHECK(cudaGetLastError());
    }
    const dim3 query_grid(static_cast<unsigned>((rows_per_sequence + ROWS - 1) / ROWS), 1, batch_size);
    absorbed_backward_query_kernel<<<query_grid, THREADS, qs::SMEM_BYTES, stream>>>(params);
    CUDA_CHECK(cudaGetLastError());
}

}  // namespace dscuda
