// Causal attention forward for sm_100a: S = Q K^T on tcgen05 tensor cores with
// the accumulator in tensor memory, online softmax in registers (one thread per
// query row), P written back to tensor memory as bf16 and used as the A operand
// of O += P V.  Two instantiations:
//
//   * non-absorbed MLA prefill: 192-wide QK (128 "nope" columns per head plus
//     64 rotary columns whose key side is shared by all heads), 128-wide V;
//   * plain D=128 grouped-query attention (the flash_attention.h contract).
//
// Work unit: one CTA owns 256 consecutive query rows of one (sequence, head) as
// two 128-row tiles that take turns on the tensor core, so the softmax of one
// overlaps the MMAs of the other.  K and V stream through a ring of 16 KB
// shared-memory chunks filled by TMA (one plain load per CTA; K/V reuse between
// CTAs is served by L2).
//
// Warp roles (384 threads): warps 0-3 softmax/epilogue of tile 0, warps 4-7 of
// tile 1, warp 8 issues every MMA (the whole warp runs the loop, one elected
// lane executes the instruction), warp 9 issues every TMA load from one thread,
// warps 10-11 only complete the third warpgroup so that it can hand registers
// to the softmax warps.  All waits are bounded; a wait that runs out raises the
// device status word and the CTA tears down normally (tensor memory freed).
#include "mla.h"
#include "flash_attention.h"
#include "cuda_common.h"
#include "attention_internal.h"
#include "sm100_primitives.cuh"
#include "../common/tensor_map.h"

#include <stdexcept>

namespace dscuda {
namespace {

using namespace sm100;

constexpr int TILE_M = 128;                 // query rows per tile (= TMEM lanes)
constexpr int TILE_N = 128;                 // keys per K/V tile
constexpr int HEAD_V = 128;                 // value width
constexpr int CHUNK_BYTES = 16384;          // [128 rows x 64 bf16] or [64 keys x 128 bf16]
constexpr int V_CHUNKS = TILE_N / 64;       // V tile = 2 chunks of 64 keys
constexpr int FORWARD_THREADS = 384;     // warps 10 and 11 only complete the third warpgroup for setmaxnreg
constexpr int MMA_WARP = 8;
constexpr int LOAD_WARP = 9;
constexpr int TMEM_COLUMNS = 512;           // S0 | S1 | O0 | O1, 128 columns each
constexpr int MISC_BYTES = 1024;
constexpr float RESCALE_THRESHOLD = 8.0F;   // log2 units; below it the old row maximum is kept

__device__ int forward_status = 0;

struct ForwardParams {
    CUtensorMap q_main;     // [rows, Hq*128], box 128 x 64
    CUtensorMap q_pe;       // [rows, Hq*64],  box 128 x 64 (unused when KQ == 2)
    CUtensorMap k_main;     // [rows, Hkv*128], box 128 x 64
    CUtensorMap k_pe;       // [rows, 64],      box 128 x 64 (unused when KQ == 2)
    CUtensorMap v;          // [rows, Hkv*128], box 64 x 64
    __nv_bfloat16* out;     // [rows, Hq, 128]
    float* lse;             // dense [B,Hq,S]; packed [Hq,total]
    const int* cu_seqlens;  // null = dense
    int batch;              // sequences
    int max_seq;            // dense: S
    int total;              // rows of every tensor
    int heads;              // query heads
    int group;              // query heads per K/V head
    float scale;            // softmax scale
    float scale_log2;       // scale * log2(e)
};

template <int KQ>
struct ForwardLayout {
    static constexpr int Q_CHUNKS = 2 * KQ;
    static constexpr int RING = 14 - Q_CHUNKS;      // 8 chunks for KQ=3, 10 for KQ=2
    static constexpr int PER_TILE = KQ + V_CHUNKS;  // ring chunks one K/V tile takes
    static constexpr int Q_BYTES = Q_CHUNKS * CHUNK_BYTES;
    static constexpr int RING_BYTES = RING * CHUNK_BYTES;
    static constexpr int SMEM_BYTES = Q_BYTES + RING_BYTES + MISC_BYTES + 1024;  // + alignment slack
};

struct ForwardBarriers {
    uint64_t q_full[2];
    uint64_t s_full[2];
    uint64_t p_full[2];
    uint64_t p_half[2];        // the first 64 keys of P are stored: the first half of P V may start
    uint64_t ring_full[10];
    uint64_t ring_empty[10];
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(ForwardBarriers) <= MISC_BYTES, "barrier block too large");

template <int KQ>
__global__ void __launch_bounds__(FORWARD_THREADS, 1) attention_forward_kernel(const __grid_constant__ ForwardParams p) {
    using L = ForwardLayout<KQ>;
    extern __shared__ uint8_t smem_raw[];

    if (*reinterpret_cast<volatile int*>(&forward_status) != 0) {
        return;
    }

    // ---- which rows does this CTA own? ------------------------------------
    int row0;      // first row of the sequence inside the packed tensors
    int length;    // tokens of the sequence
    int qblock;    // 256-row block inside the sequence
    const int head = blockIdx.y;
    float* lse_base;
    if (p.cu_seqlens == nullptr) {
        const int b = blockIdx.z;
        row0 = b * p.max_seq;
        length = p.max_seq;
        qblock = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
        lse_base = p.lse + (static_cast<size_t>(b) * p.heads + head) * p.max_seq;
    } else {
        int index = blockIdx.x;
        int sequence = 0;
        int begin = 0;
        int blocks = 0;
        for (; sequence < p.batch; ++sequence) {
            begin = p.cu_seqlens[sequence];
            const int tokens = p.cu_seqlens[sequence + 1] - begin;
            blocks = (tokens + 2 * TILE_M - 1) / (2 * TILE_M);
            if (index < blocks) {
                length = tokens;
                break;
            }
            index -= blocks;
        }
        if (sequence == p.batch) {
            return;
        }
        row0 = begin;
        qblock = blocks - 1 - index;
        lse_base = p.lse + static_cast<size_t>(head) * p.total + row0;
    }
    const int q_start = qblock * 2 * TILE_M;
    if (q_start >= length) {
        return;
    }
    const int tiles[2] = {q_start / TILE_N + 1, (q_start + TILE_M < length) ? q_start / TILE_N + 2 : 0};
    const int tile_count = tiles[1] > 0 ? tiles[1] : tiles[0];
    const int kv_head = head / p.group;

    // ---- shared memory carve-up -------------------------------------------
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023U) & ~1023U;
    const uint32_t q_smem = smem_base;
    const uint32_t ring_smem = smem_base + L::Q_BYTES;
    ForwardBarriers* bars = reinterpret_cast<ForwardBarriers*>(smem_raw + (smem_base - smem_u32(smem_raw)) + L::Q_BYTES + L::RING_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&bars->q_full[i]), 1);
            mbar_init(smem_u32(&bars->s_full[i]), 1);
            mbar_init(smem_u32(&bars->p_full[i]), TILE_M);
            mbar_init(smem_u32(&bars->p_half[i]), TILE_M);
        }
        for (int i = 0; i < L::RING; ++i) {
            mbar_init(smem_u32(&bars->ring_full[i]), 1);
            mbar_init(smem_u32(&bars->ring_empty[i]), 1);
        }
        bars->abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&bars->tmem_base), TMEM_COLUMNS);
        tmem_relinquish();
    }
    if (warp == LOAD_WARP && lane == 0) {
        tma_prefetch_descriptor(&p.q_main);
        tma_prefetch_descriptor(&p.k_main);
        tma_prefetch_descriptor(&p.v);
        if (KQ == 3) {
            tma_prefetch_descriptor(&p.q_pe);
            tma_prefetch_descriptor(&p.k_pe);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

    // Registers: the CTA starts with 168 per thread (12 warps).  The softmax keeps a 128-column
    // score row in registers and spills at 168, so warps 8-11 hand registers to warps 0-7.  The
    // two setmaxnreg instructions sit inside the role branches: after a join of branches with
    // different limits the compiler assumes the lower one for all the code that follows.
    constexpr int REG_LO = 88;
    constexpr int REG_HI = 208;
    // The increase blocks until the CTA's pool holds the registers: what warps 8-11 release must
    // cover what warps 0-7 request, or the kernel never starts (launch allocation: 168 each).
    static_assert(8 * (REG_HI - 168) <= 4 * (168 - REG_LO), "register redistribution exceeds the CTA's allocation");
    if (warp >= 8) {
        reg_dealloc<REG_LO>();      // one instruction for the whole warpgroup; warps 10 and 11 do nothing else
        if (warp == LOAD_WARP) {
            // =================== TMA producer ===================================
            if (lane == 0) {
                auto load_q = [&](int i) {
                    const uint32_t bar = smem_u32(&bars->q_full[i]);
                    mbar_arrive_expect_tx(bar, KQ * CHUNK_BYTES);
                    const int y = row0 + q_start + i * TILE_M;
                    for (int c = 0; c < KQ; ++c) {
                        const uint32_t dst = q_smem + (i * KQ + c) * CHUNK_BYTES;
                        if (KQ == 3 && c == 2) {
                            tma_load_2d(dst, &p.q_pe, bar, head * 64, y);
                        } else {
                            tma_load_2d(dst, &p.q_main, bar, head * 128 + c * 64, y);
                        }
                    }
                };
                bool alive = true;
                int chunk = 0;
                // Returns the destination of ring chunk `chunk` once it is free, 0 on abort.
                auto acquire = [&](uint32_t& bar) -> uint32_t {
                    const int slot = chunk % L::RING;
                    const int use = chunk / L::RING;
                    if (use > 0 && !mbar_wait(smem_u32(&bars->ring_empty[slot]), (use - 1) & 1, abort_flag, &forward_status)) {
                        alive = false;
                        return 0;
                    }
                    bar = smem_u32(&bars->ring_full[slot]);
                    mbar_arrive_expect_tx(bar, CHUNK_BYTES);
                    ++chunk;
                    return ring_smem + slot * CHUNK_BYTES;
                };
                load_q(0);
                for (int j = 0; j < tile_count && alive; ++j) {
                    const int y = row0 + j * TILE_N;
                    for (int c = 0; c < KQ && alive; ++c) {
                        uint32_t bar;
                        const uint32_t dst = acquire(bar);
                        if (dst == 0) {
                            break;
                        }
                        if (KQ == 3 && c == 2) {
                            tma_load_2d(dst, &p.k_pe, bar, 0, y);
                        } else {
                            tma_load_2d(dst, &p.k_main, bar, kv_head * 128 + c * 64, y);
                        }
                    }
                    if (j == 0 && tiles[1] > 0) {
                        load_q(1);
                    }
                    for (int half = 0; half < V_CHUNKS && alive; ++half) {
                        uint32_t bar;
                        const uint32_t dst = acquire(bar);
                        if (dst == 0) {
                            break;
                        }
                        tma_load_2d(dst, &p.v, bar, kv_head * 128, y + half * 64);
                        tma_load_2d(dst + CHUNK_BYTES / 2, &p.v, bar, kv_head * 128 + 64, y + half * 64);
                    }
                }
            }
        } else if (warp == MMA_WARP) {
            // =================== MMA issuer =====================================
            // The whole warp runs the loop (uniform control flow, uniform operands); one elected
            // lane executes the tcgen05 instructions.  A lane-0 branch issues at well under the
            // tensor core's rate once the softmax warps compete for the scheduler.
            {
                const uint32_t leader = elect_one();
                constexpr uint32_t IDESC_QK = make_idesc_bf16(TILE_M, TILE_N, false, false);
                constexpr uint32_t IDESC_PV = make_idesc_bf16(TILE_M, HEAD_V, false, true);
                bool alive = true;
                auto wait_chunk = [&](int chunk) -> uint32_t {
                    const int slot = chunk % L::RING;
                    if (!__all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->ring_full[slot]), (chunk / L::RING) & 1, abort_flag, &forward_status))) {
                        alive = false;
                    }
                    return ring_smem + slot * CHUNK_BYTES;
                };
                auto release_chunk = [&](int chunk) {
                    mma_commit_elect(smem_u32(&bars->ring_empty[chunk % L::RING]), leader);
                };
                // S_i = Q_i K_j^T
                auto issue_qk = [&](int i, int j) {
                    const uint32_t d = tmem_base + i * TILE_N;
                    for (int c = 0; c < KQ && alive; ++c) {
                        const uint32_t k_chunk = wait_chunk(j * L::PER_TILE + c);
                        if (!alive) {
                            return;
                        }
                        tc_fence_after_sync();
                        const uint32_t q_chunk = q_smem + (i * KQ + c) * CHUNK_BYTES;
    #pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            mma_ss_elect(d, make_kmajor_desc(q_chunk + k * 32), make_kmajor_desc(k_chunk + k * 32), IDESC_QK,
                                   (c | k) != 0 ? 1U : 0U, leader);
                        }
                    }
                    mma_commit_elect(smem_u32(&bars->s_full[i]), leader);
                    const bool last_user = (i == 1) || (j >= tiles[1]);
                    if (last_user) {
                        for (int c = 0; c < KQ; ++c) {
                            release_chunk(j * L::PER_TILE + c);
                        }
                    }
                };
                // O_i (+)= P_i V_j
                auto issue_pv = [&](int i, int j) {
                    const uint32_t d = tmem_base + 2 * TILE_N + i * HEAD_V;
                    const uint32_t p_tmem = tmem_base + i * TILE_N;
                    for (int half = 0; half < V_CHUNKS && alive; ++half) {
                        const uint32_t v_chunk = wait_chunk(j * L::PER_TILE + KQ + half);
                        if (alive) {
                            // keys 0-63 of P are ready before keys 64-127
                            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(half == 0 ? &bars->p_half[i] : &bars->p_full[i]), j & 1, abort_flag,
                                                                      &forward_status));
                        }
                        if (!alive) {
                            return;
                        }
                        tc_fence_after_sync();
    #pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            // 16 keys per step: 8 packed columns of P, 16 rows (2048 B) of V.
                            mma_ts_elect(d, p_tmem + half * 32 + k * 8, make_smem_desc(v_chunk + k * 2048, CHUNK_BYTES / 2, 1024), IDESC_PV,
                                   (j | half | k) != 0 ? 1U : 0U, leader);
                        }
                    }
                    const bool last_user = (i == 1) || (j >= tiles[1]);
                    if (last_user) {
                        for (int half = 0; half < V_CHUNKS; ++half) {
                            release_chunk(j * L::PER_TILE + KQ + half);
                        }
                    }
                };

                for (int i = 0; i < 2 && alive; ++i) {
                    if (tiles[i] > 0) {
                        alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->q_full[i]), 0, abort_flag, &forward_status));
                        if (alive) {
                            issue_qk(i, 0);
                        }
                    }
                }
                for (int j = 0; j < tile_count && alive; ++j) {
                    for (int i = 0; i < 2 && alive; ++i) {
                        if (j >= tiles[i]) {
                            continue;
                        }
                        issue_pv(i, j);
                        if (!alive) {
                            break;
                        }
                        if (j + 1 < tiles[i]) {
                            issue_qk(i, j + 1);
                        } else {
                            mma_commit_elect(smem_u32(&bars->s_full[i]), leader);   // O_i is final
                        }
                    }
                }
            }
        }
    } else {
        // =================== softmax + epilogue =============================
        reg_alloc<REG_HI>();
        const int i = warp / 4;                       // tile of this warpgroup
        const int r = threadIdx.x % TILE_M;           // row inside the tile
        const uint32_t lane_base = static_cast<uint32_t>((warp % 4) * 32) << 16;
        const uint32_t s_tmem = tmem_base + lane_base + i * TILE_N;
        const uint32_t o_tmem = tmem_base + lane_base + 2 * TILE_N + i * HEAD_V;
        const int count = tiles[i];
        const int q_pos = q_start + i * TILE_M + r;
        float m_ref = 0.0F;       // reference maximum of the raw scores (lags the true one by < threshold)
        float l_sum = 0.0F;       // sum of exp2((s - m_ref) * scale_log2)
        bool alive = true;

        for (int j = 0; j < count; ++j) {
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->s_full[i]), j & 1, abort_flag, &forward_status));
            if (!alive) {
                break;
            }
            tc_fence_after_sync();
            uint32_t sb[TILE_N];
#pragma unroll
            for (int c = 0; c < TILE_N / 32; ++c) {
                tmem_ld_x32(s_tmem + c * 32, sb + c * 32);
            }
            tmem_wait_ld();
            if (j == count - 1) {
                // diagonal tile: key n of the tile is allowed for row r iff n <= r
#pragma unroll
                for (int n = 0; n < TILE_N; ++n) {
                    sb[n] = n <= r ? sb[n] : 0xff800000U;
                }
            }
            // three-input maxima: 64 instructions for 128 scores, four independent chains
            float mx0 = __uint_as_float(sb[0]), mx1 = __uint_as_float(sb[1]), mx2 = __uint_as_float(sb[2]), mx3 = __uint_as_float(sb[3]);
#pragma unroll
            for (int n = 4; n + 7 < TILE_N; n += 8) {
                mx0 = max3(mx0, __uint_as_float(sb[n]), __uint_as_float(sb[n + 1]));
                mx1 = max3(mx1, __uint_as_float(sb[n + 2]), __uint_as_float(sb[n + 3]));
                mx2 = max3(mx2, __uint_as_float(sb[n + 4]), __uint_as_float(sb[n + 5]));
                mx3 = max3(mx3, __uint_as_float(sb[n + 6]), __uint_as_float(sb[n + 7]));
            }
            mx0 = max3(mx0, __uint_as_float(sb[TILE_N - 4]), __uint_as_float(sb[TILE_N - 3]));
            mx1 = max3(mx1, __uint_as_float(sb[TILE_N - 2]), __uint_as_float(sb[TILE_N - 1]));
            const float tile_max = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            if (j == 0) {
                m_ref = tile_max;
            } else {
                const bool grow = (tile_max - m_ref) * p.scale_log2 > RESCALE_THRESHOLD;
                if (__any_sync(0xffffffffU, grow)) {
                    float alpha = 1.0F;
                    if (grow) {
                        alpha = exp2_approx((m_ref - tile_max) * p.scale_log2);
                        m_ref = tile_max;
                        l_sum *= alpha;
                    }
                    // S_i(j) complete implies P_i(j-1) V complete: O_i is quiescent here.
#pragma unroll
                    for (int c = 0; c < HEAD_V / 32; ++c) {
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
            for (int c = 0; c < TILE_N / 32; ++c) {
                uint32_t packed[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const float2 x = fma2(make_float2(__uint_as_float(sb[c * 32 + 2 * e]), __uint_as_float(sb[c * 32 + 2 * e + 1])), scale2, bias2);
                    const float2 pr = make_float2(exp2_approx(x.x), exp2_approx(x.y));
                    sums = add2(sums, pr);
                    packed[e] = pack_bf16x2(pr.x, pr.y);
                }
                tmem_st_x16(s_tmem + c * 16, packed);      // P aliases the first 64 columns of S
                if (c == 1) {
                    tmem_wait_st();
                    tc_fence_before_sync();
                    mbar_arrive(smem_u32(&bars->p_half[i]));
                }
            }
            const float sum0 = sums.x, sum1 = sums.y;
            l_sum += sum0 + sum1;
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&bars->p_full[i]));
        }

        if (alive && count > 0) {
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&bars->s_full[i]), count & 1, abort_flag, &forward_status));
        }
        if (alive && count > 0) {
            tc_fence_after_sync();
            const bool valid = q_pos < length;
            const float inverse = 1.0F / l_sum;
            __nv_bfloat16* out_row = p.out + (static_cast<size_t>(row0 + q_pos) * p.heads + head) * HEAD_V;
#pragma unroll
            for (int c = 0; c < HEAD_V / 32; ++c) {
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
            if (valid) {
                lse_base[q_pos] = m_ref * p.scale + logf(l_sum);
            }
        }
    }

    // ---- teardown: every path reaches this point ---------------------------
    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        // give loads that may still be in flight time to land before the CTA's
        // shared memory is handed to another CTA
        for (int k = 0; k < 64; ++k) {
            __nanosleep(1000);
        }
    }
    if (warp == MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLUMNS);
    }
}

template <int KQ>
void configure_forward_kernel() {
    static bool done[16] = {};
    int device = 0;
    CUDA_CHECK(cudaGetDevice(&device));
    if (device < 16 && done[device]) {
        return;
    }
    CUDA_CHECK(cudaFuncSetAttribute(attention_forward_kernel<KQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    ForwardLayout<KQ>::SMEM_BYTES));
    if (device < 16) {
        done[device] = true;
    }
}

void check_pointers(std::initializer_list<const void*> pointers) {
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

void launch_prefill_forward(__nv_bfloat16* output, float* logsumexp, const __nv_bfloat16* q_nope, const __nv_bfloat16* q_pe,
                            const __nv_bfloat16* k_nope, const __nv_bfloat16* k_pe, const __nv_bfloat16* v, const int* cu_seqlens,
                            int batch_size, int max_sequence_length, int total_tokens, int heads, float scale,
                            cudaStream_t stream) {
    check_pointers({output, logsumexp, q_nope, q_pe, k_nope, k_pe, v});
    ForwardParams params{};
    const std::uint64_t rows = static_cast<std::uint64_t>(total_tokens);
    params.q_main = make_bf16_tile_map(q_nope, rows, static_cast<std::uint64_t>(heads) * 128, static_cast<std::uint64_t>(heads) * 128, 128);
    params.q_pe = make_bf16_tile_map(q_pe, rows, static_cast<std::uint64_t>(heads) * 64, static_cast<std::uint64_t>(heads) * 64, 128);
    params.k_main = make_bf16_tile_map(k_nope, rows, static_cast<std::uint64_t>(heads) * 128, static_cast<std::uint64_t>(heads) * 128, 128);
    params.k_pe = make_bf16_tile_map(k_pe, rows, 64, 64, 128);
    params.v = make_bf16_tile_map(v, rows, static_cast<std::uint64_t>(heads) * 128, static_cast<std::uint64_t>(heads) * 128, 64);
    params.out = output;
    params.lse = logsumexp;
    params.cu_seqlens = cu_seqlens;
    params.batch = batch_size;
    params.max_seq = max_sequence_length;
    params.total = total_tokens;
    params.heads = heads;
    params.group = 1;
    params.scale = scale;
    params.scale_log2 = scale * 1.4426950408889634F;
    configure_forward_kernel<3>();
    dim3 grid;
    if (cu_seqlens == nullptr) {
        grid = dim3((max_sequence_length + 255) / 256, heads, batch_size);
    } else {
        grid = dim3(total_tokens / 256 + batch_size, heads, 1);
    }
    attention_forward_kernel<3><<<grid, FORWARD_THREADS, ForwardLayout<3>::SMEM_BYTES, stream>>>(params);
    CUDA_CHECK(cudaGetLastError());
}

int forward_device_status(bool reset) {
    int status = 0;
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemcpyFromSymbol(&status, forward_status, sizeof(int)));
    if (reset && status != 0) {
        const int zero = 0;
        CUDA_CHECK(cudaMemcpyToSymbol(forward_status, &zero, sizeof(int)));
    }
    return status;
}

}  // namespace internal

void mla_prefill_forward_cuda(__nv_bfloat16* output, float* logsumexp, const __nv_bfloat16* q_nope, const __nv_bfloat16* q_pe,
                              const __nv_bfloat16* k_nope, const __nv_bfloat16* k_pe, const __nv_bfloat16* v, const int* cu_seqlens,
                              int batch_size, int max_sequence_length, int total_tokens, int heads, int nope_size, int rope_size,
                              int value_size, float scale, cudaStream_t stream) {
    internal::check_prefill_shape(cu_seqlens, batch_size, max_sequence_length, total_tokens, heads, nope_size, rope_size, value_size, scale);
    internal::launch_prefill_forward(output, logsumexp, q_nope, q_pe, k_nope, k_pe, v, cu_seqlens, batch_size, max_sequence_length,
                                     total_tokens, heads, scale, stream);
}

void flash_attention_forward_cuda(__nv_bfloat16* output, float* logsumexp, const __nv_bfloat16* query, const __nv_bfloat16* key,
                                  const __nv_bfloat16* value, int batch_size, int sequence_length, int query_heads, int key_value_heads,
                                  int head_size, float scale, cudaStream_t stream) {
    if (head_size != 128) {
        throw std::invalid_argument("flash attention requires head_size 128");
    }
    if (batch_size <= 0 || sequence_length <= 0) {
        throw std::invalid_argument("flash attention requires positive batch and sequence length");
    }
    if (query_heads <= 0 || key_value_heads <= 0 || query_heads % key_value_heads != 0) {
        throw std::invalid_argument("flash attention requires query_heads to be divisible by key_value_heads");
    }
    if (!(scale > 0.0F)) {
        throw std::invalid_argument("flash attention requires a positive softmax scale");
    }
    if (static_cast<long long>(batch_size) * sequence_length > 0x7fffffffLL || query_heads > 65535 || batch_size > 65535) {
        throw std::invalid_argument("flash attention shape exceeds the supported index range");
    }
    check_pointers({output, logsumexp, query, key, value});
    ForwardParams params{};
    const std::uint64_t rows = static_cast<std::uint64_t>(batch_size) * sequence_length;
    const std::uint64_t q_cols = static_cast<std::uint64_t>(query_heads) * 128;
    const std::uint64_t kv_cols = static_cast<std::uint64_t>(key_value_heads) * 128;
    params.q_main = make_bf16_tile_map(query, rows, q_cols, q_cols, 128);
    params.k_main = make_bf16_tile_map(key, rows, kv_cols, kv_cols, 128);
    params.v = make_bf16_tile_map(value, rows, kv_cols, kv_cols, 64);
    params.q_pe = params.q_main;
    params.k_pe = params.k_main;
    params.out = output;
    params.lse = logsumexp;
    params.cu_seqlens = nullptr;
    params.batch = batch_size;
    params.max_seq = sequence_length;
    params.total = static_cast<int>(rows);
    params.heads = query_heads;
    params.group = query_heads / key_value_heads;
    params.scale = scale;
    params.scale_log2 = scale * 1.4426950408889634F;
    configure_forward_kernel<2>();
    const dim3 grid((sequence_length + 255) / 256, query_heads, batch_size);
    attention_forward_kernel<2><<<grid, FORWARD_THREADS, ForwardLayout<2>::SMEM_BYTES, stream>>>(params);
    CUDA_CHECK(cudaGetLastError());
}

}  // namespace dscuda
