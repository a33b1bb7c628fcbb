// Absorbed-latent MLA attention on sm_100a: the paged split-KV decode (mla_decode_forward_cuda and its
// variants) and the causal forward (mla_compressed_attention_forward_cuda).  Both have up to 128 query
// rows sharing every key row of 576 bf16 (512 latent columns that are also the value, 64 rotary
// columns), and both run on one kernel body:
//
//   decode:          rows = the heads of a sequence's one query token; keys = the sequence's cached rows,
//                    found through the block table; split-KV partials merged by decode_combine_kernel;
//   causal forward:  rows = 128 consecutive (token, head) pairs of a batch entry; keys = the rows of
//                    kv_latent / key_rope up to each row's own token (masked per row); row tiles dealt
//                    longest first to the clusters; the output is final.
//
// A 128-head x 512-column fp32 output fills the tensor memory of one SM, so two CTAs of a cluster
// work as one: tcgen05.mma.cta_group::2 with M = 128 gives each CTA 64 heads.  Per 128-key tile
//
//   S = Q K^T   (N = 128 keys, K = 576):  CTA r supplies its 64 heads of Q (A operand) and its own 64
//               keys of the tile (the hardware takes half of the B operand from each CTA), so the
//               scores are computed once and every cached row is fetched from HBM once;
//   O += P V    (N = 256 value columns, twice; K = 128 keys):  CTA r supplies P for its heads (bf16,
//               written to shared memory by the softmax threads) and, for all 128 keys, the value
//               columns [128r, 128r+128) of each 256-column half.
//
// Both products address shared memory at the same offsets in both CTAs.  The eight latent chunks
// of a CTA's own 64 keys sit at offsets SB(0..7); the value operand of key half g and output half a
// is read at SB(4a+2g), SB(4a+2g+1).  For CTA r the chunks {2r, 2r+1, 4+2r, 4+2r+1} of its own
// keys are therefore already in place as value columns; the other four offsets hold chunks only S
// needs, and as soon as the score MMAs have read them they are refilled with the other CTA's keys
// (the same four value columns), from L2.  13 chunk loads of 8 KB per CTA and tile, no copy
// between the CTAs.
//
// Tensor memory per CTA (data-path layout of cta_group::2 with M = 128: lane = head + 64 * half of
// the N range): O as two accumulators of 128 columns (lanes 0-63: value columns 256a + 0..127,
// lanes 64-127: 256a + 128..255), two score buffers of 64 columns (lanes 0-63: keys 0-63 of the
// tile, lanes 64-127: keys 64-127).
//
// Roles per CTA: warps 0-3 softmax / epilogue (thread = head x half of the keys; the two threads of a
// head exchange their maxima and sums through shared memory), warp 4 issues every MMA in the
// leader CTA (whole warp, one elected lane) and in the other CTA relays "loaded" events to the
// leader, warps 5 and 6 load with TMA (5: Q, the tiles' own keys and L2 prefetches; 6: the two small loads
// on the critical path, rotary chunk and refill).  The grid is persistent: one cluster per SM pair, the 128-key tiles
// of all sequences laid end to end and cut into equal ranges; a sequence cut by a range boundary
// yields one normalised partial per range, merged by decode_combine_kernel.  Every wait is bounded.
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

constexpr int RANK = MLA_KV_RANK;               // 512
constexpr int ROPE = MLA_ROPE_SIZE;             // 64
constexpr int WIDTH = RANK + ROPE;              // 576
constexpr int CTA_HEADS = 64;                   // heads per CTA
constexpr int PAIR_HEADS = 128;                 // heads per cluster
constexpr int TILE_KEYS = 128;                  // keys per tile (both CTAs)
constexpr int HALF_KEYS = 64;                   // keys a CTA owns in a tile
constexpr int CHUNK = 64 * 128;                 // 8 KB: [64 rows x 64 bf16]
constexpr int LATENT_CHUNKS = 8;
constexpr int Q_BYTES = 9 * CHUNK;
constexpr int P_BYTES = 2 * CHUNK;
constexpr int STAGES = 2;
constexpr int STAGE_BYTES = LATENT_CHUNKS * CHUNK;
constexpr int MISC_BYTES = 2048;
constexpr int SMEM_BYTES = Q_BYTES + P_BYTES + STAGES * STAGE_BYTES + CHUNK + MISC_BYTES;      // no room to realign
constexpr int THREADS = 224;
constexpr int MMA_WARP = 4;
constexpr int LOAD_WARP = 5;
constexpr int REFILL_WARP = 6;
constexpr int TMEM_COLUMNS = 512;
constexpr uint32_t TMEM_O = 0;                  // 2 x 128 columns
constexpr uint32_t TMEM_S = 256;                // 2 x 64 columns
constexpr float RESCALE_THRESHOLD = 8.0F;
constexpr int PREFETCH_TILES = 3;              // tiles whose cache rows are asked into L2 ahead of their shared-memory load
static_assert(SMEM_BYTES <= 232448, "decode shared memory");

__device__ int decode_status = 0;

// Scratch for mla_decode_forward_static_cuda: room for STATIC_DECODE_RECORDS split partials of
// (log-sum-exp, 1, 512 outputs).  It lives in the image of the library, so every GPU that loads the
// library keeps these 16.1 MiB until the process ends.  The name below is only a host-side handle
// in host code; the device address is looked up once per device with cudaGetSymbolAddress.
constexpr std::size_t STATIC_DECODE_RECORDS = 8192;
static __device__ __align__(256) float decode_static_scratch[STATIC_DECODE_RECORDS * (MLA_KV_RANK + 2)];

struct DecodeParams {
    CUtensorMap q_all;      // [B*H rows][9 chunks][64]: all nine chunks of 64 query rows in one load
    CUtensorMap k_lat8;     // cache rows as [8 latent chunks][row][64], box of 8 chunks x 64 rows: a stage in one load
    CUtensorMap k_lat2;     // the same view, box of 2 chunks x 64 rows: one refilled slot pair
    CUtensorMap k_rope;     // [cache rows, 64] box 64 x 64
    // causal forward only: the queries as two tensors, the outputs, the sequence length
    CUtensorMap q_lat;      // [B*T*H rows][8 chunks][64], box of 8 chunks x 64 rows
    CUtensorMap q_rope;     // [B*T*H rows, 64], box 64 x 64
    __nv_bfloat16* out;     // [B,T,H,512]
    float* lse;             // [B,H,T]
    int sequence;           // T
    const __nv_bfloat16* cache;     // [cache rows, 576]
    const int* block_table; // [B, pages]
    const int* lengths;     // [B]
    float* workspace;       // [B,H,splits,2+512]
    int batch;
    int heads;
    int page_size;
    int pages;
    int splits;
    int cache_blocks;       // physical pages in the cache, or 0 when the caller did not say
    float scale;
    float scale_log2;
};

struct Schedule {
    int chunk;          // 128-key tiles per cluster
    int total;          // tiles of all units
    int first_unit;     // first unit that overlaps this cluster's range
    int first_offset;   // global tile index at which that unit starts
};

struct Shared {
    // completed by TMA transactions of this CTA
    uint64_t q_full;
    uint64_t full_a[STAGES];        // the eight latent chunks of this CTA's own keys
    uint64_t full_r;                // the rotary chunk
    uint64_t full_b[STAGES];        // the four chunks refilled with the other CTA's keys
    // leader only: the same events of the other CTA, forwarded by its relay warp
    uint64_t peer_q_full;
    uint64_t peer_full_a[STAGES];
    uint64_t peer_full_r;
    uint64_t peer_full_b[STAGES];
    // completed by tcgen05.commit of the leader (one commit per CTA)
    uint64_t refill_free[STAGES];   // the score MMAs have read this CTA's four S-only latent chunks
    uint64_t rope_free;             // ... and the rotary chunk
    uint64_t s_full[2];
    uint64_t stage_free[STAGES];    // P V has read the stage
    uint64_t p_free;                // P V has read P (and O is quiescent)
    uint64_t o_final;
    // leader only: one arrival per softmax warp of either CTA (lane 0, after the warp has synchronised): P is
    // stored.  One arrival per thread would be 128 serialised transactions on the link between the two SMs.
    uint64_t p_full;
    // the four softmax warps of this CTA (lane 0, after the warp has synchronised): the two threads of a head have
    // published their maxima / sums
    uint64_t max_ready[2];
    uint64_t sum_ready;
    uint32_t tmem_base;
    int abort_flag;
    Schedule schedule;
    float maxima[2][PAIR_HEADS];    // per tile parity
    float sums[PAIR_HEADS];
};
static_assert(sizeof(Shared) <= MISC_BYTES, "decode barrier block too large");

// ---- cluster / cta_group::2 primitives ------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t result;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(result) : "r"(smem_addr), "r"(rank));
    return result;
}

// One arrival on a barrier of the other CTA.  Default semantics (release at CTA scope), like every
// other arrive here: what the arrival publishes is shared memory of the arriving CTA itself, made
// visible to the tensor core by fence.proxy.async before the arrive; cluster-scope release /
// acquire pairs cost several hundred cycles each on this path and buy nothing.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// Asks for `bytes` (a multiple of 16) of contiguous global memory to be brought into L2; nothing to wait for.
__device__ __forceinline__ void prefetch_l2_bulk(const void* global_address, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(global_address), "r"(bytes) : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(columns) : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}

// D[tmem of both CTAs] (+)= A[smem of each CTA] * B[smem, half of N from each CTA]; elected lane of the leader
// CTA.  Split descriptors: the high words are compile-time constants, the low words advance with 32-bit adds.
__device__ __forceinline__ void mma_pair_ss_split(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                                  uint32_t accumulate, uint32_t leader) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        ".reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "setp.ne.b32 q, %7, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "@q tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}

// One arrival on the barrier at `cluster_addr` (this CTA's or, through map_to_cta, the other's)
// once every MMA issued so far has finished.
__device__ __forceinline__ void commit_pair(uint32_t cluster_addr, uint32_t leader) {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}\n"
        ::"r"(cluster_addr), "r"(leader)
        : "memory");
}

// ---- schedule ---------------------------------------------------------------
// Cached tokens of sequence `b` the kernel will read: the caller's length, held inside
// [0, capacity of the sequence's block-table row].
template <bool CAUSAL>
__device__ __forceinline__ int sequence_length(const DecodeParams& p, int b) {
    if (CAUSAL) {
        return p.sequence;
    }
    return max(0, min(p.lengths[b], p.pages * p.page_size));
}

// Causal forward: the rows of a batch entry are its (token, head) pairs, 128 to a row tile; a row tile
// attends to the keys up to the token of its last row.  Row tiles are dealt longest first.
__device__ __forceinline__ int causal_row_tile(const DecodeParams& p, int unit, int row_tiles) {
    return row_tiles - 1 - unit % row_tiles;
}

template <bool CAUSAL>
__device__ __forceinline__ int unit_tiles(const DecodeParams& p, int unit, int head_tiles) {
    if (CAUSAL) {
        const int last_row = min(causal_row_tile(p, unit, head_tiles) * PAIR_HEADS + PAIR_HEADS - 1, p.sequence * p.heads - 1);
        return (last_row / p.heads) / TILE_KEYS + 1;
    }
    return (sequence_length<false>(p, unit / head_tiles) + TILE_KEYS - 1) / TILE_KEYS;
}

// One piece of work: tiles [tile_begin, tile_end) of sequence `b`, heads [128*row_tile, +128).
struct Segment {
    int b;
    int row_tile;
    int tile_begin;
    int tile_end;
    int slot;            // which partial record of (b, head) this segment fills
    bool last_of_unit;   // the segment that reaches the end of the sequence
};

struct Walker {
    int unit;
    int offset;     // global tile index where `unit` starts
    bool done;
};

// Units are (sequence, 128-head tile) pairs, laid end to end as one long list of 128-key tiles.
// With splits > 1 the list is cut into equal ranges, one per cluster; a unit cut by a range
// boundary produces one partial per range it touches.  The range length is never smaller than
// ceil(longest unit / (splits - 1)), which bounds the partials of a unit by `splits`.  With
// splits == 1 whole units are dealt round-robin.  Every role thread runs its own walker over the
// same schedule, so all roles of both CTAs see the same sequence of segments.
template <bool CAUSAL>
__device__ __forceinline__ bool next_segment(const DecodeParams& p, const Schedule& s, Walker& w, Segment& seg, int cluster, int clusters) {
    if (w.done) {
        return false;
    }
    // decode: 128-head tiles of a sequence; causal forward: 128-row tiles of a batch entry's (token, head) rows
    const int head_tiles = CAUSAL ? static_cast<int>((static_cast<long long>(p.sequence) * p.heads + PAIR_HEADS - 1) / PAIR_HEADS)
                                  : (p.heads + PAIR_HEADS - 1) / PAIR_HEADS;
    const int units = p.batch * head_tiles;
    if (CAUSAL || p.splits == 1) {
        while (w.unit < units && unit_tiles<CAUSAL>(p, w.unit, head_tiles) == 0) {
            w.unit += clusters;
        }
        if (w.unit >= units) {
            w.done = true;
            return false;
        }
        seg.b = w.unit / head_tiles;
        seg.row_tile = CAUSAL ? causal_row_tile(p, w.unit, head_tiles) : w.unit % head_tiles;
        seg.tile_begin = 0;
        seg.tile_end = unit_tiles<CAUSAL>(p, w.unit, head_tiles);
        seg.slot = 0;
        seg.last_of_unit = true;
        w.unit += clusters;
        return true;
    }
    const long long lo = static_cast<long long>(cluster) * s.chunk;
    const long long hi = min(lo + s.chunk, static_cast<long long>(s.total));
    while (w.unit < units && w.offset < hi) {
        const int tiles = unit_tiles<false>(p, w.unit, head_tiles);
        const int begin = static_cast<int>(max(lo, static_cast<long long>(w.offset)) - w.offset);
        const int end = static_cast<int>(min(hi, static_cast<long long>(w.offset) + tiles) - w.offset);
        const int unit = w.unit;
        const int offset = w.offset;
        w.unit += 1;
        w.offset += tiles;
        if (end > begin) {
            seg.b = unit / head_tiles;
            seg.row_tile = unit % head_tiles;
            seg.tile_begin = begin;
            seg.tile_end = end;
            seg.slot = cluster - offset / s.chunk;
            seg.last_of_unit = end == tiles;
            return true;
        }
    }
    w.done = true;
    return false;
}

template <bool CAUSAL>
__device__ __forceinline__ void absorbed_pair_body(const DecodeParams& p) {
    extern __shared__ uint8_t smem_raw[];
    // No early exit on a status left by an earlier launch: the two CTAs of a cluster must take the
    // same path to the cluster barriers below, and they could read different values.
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const uint32_t rank = cluster_cta_rank();           // 0 = leader
    const uint32_t peer = rank ^ 1U;
    const int cluster = blockIdx.x >> 1;
    const int clusters = gridDim.x >> 1;

    // ---- shared memory (the same offsets in both CTAs) -------------------------
    const uint32_t smem_base = smem_u32(smem_raw);
    const uint32_t q_smem = smem_base;                              // 9 chunks: Q of this CTA's 64 heads
    const uint32_t p_smem = q_smem + Q_BYTES;                       // 2 chunks: P [64 heads x 128 keys]
    const uint32_t stage_smem = p_smem + P_BYTES;                   // 2 stages x 8 latent chunks, SB(c) = stage + c * CHUNK
    const uint32_t rope_smem = stage_smem + STAGES * STAGE_BYTES;   // the rotary chunk (one slot)
    uint8_t* p_ptr = smem_raw + Q_BYTES;
    uint8_t* stage_ptr = smem_raw + Q_BYTES + P_BYTES;
    Shared* sh = reinterpret_cast<Shared*>(smem_raw + Q_BYTES + P_BYTES + STAGES * STAGE_BYTES + CHUNK);
    volatile int* abort_flag = &sh->abort_flag;
    // Both CTAs must take the same path here: the alignment is a property of the kernel image.
    if ((smem_base & 1023U) != 0U) {
        if (threadIdx.x == 0) {
            atomicExch(&decode_status, STATUS_SMEM_MISALIGNED);
        }
        return;
    }

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&sh->q_full), 1);
        mbar_init(smem_u32(&sh->full_r), 1);
        mbar_init(smem_u32(&sh->peer_q_full), 1);
        mbar_init(smem_u32(&sh->peer_full_r), 1);
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(smem_u32(&sh->full_a[i]), 1);
            mbar_init(smem_u32(&sh->full_b[i]), 1);
            mbar_init(smem_u32(&sh->peer_full_a[i]), 1);
            mbar_init(smem_u32(&sh->peer_full_b[i]), 1);
            mbar_init(smem_u32(&sh->refill_free[i]), 1);
            mbar_init(smem_u32(&sh->stage_free[i]), 1);
            mbar_init(smem_u32(&sh->s_full[i]), 1);
        }
        mbar_init(smem_u32(&sh->rope_free), 1);
        mbar_init(smem_u32(&sh->p_free), 1);
        mbar_init(smem_u32(&sh->o_final), 1);
        mbar_init(smem_u32(&sh->p_full), 8);
        mbar_init(smem_u32(&sh->max_ready[0]), 4);          // one arrival per softmax warp
        mbar_init(smem_u32(&sh->max_ready[1]), 4);
        mbar_init(smem_u32(&sh->sum_ready), 4);
        sh->abort_flag = 0;
        mbar_init_fence();
        // ---- schedule of this cluster (splits > 1) ----------------------------------
        Schedule schedule = {1, 0, 0, 0};
        if (!CAUSAL && p.splits > 1) {
            const int head_tiles = (p.heads + PAIR_HEADS - 1) / PAIR_HEADS;
            long long total = 0;
            int longest = 0;
            for (int b = 0; b < p.batch; ++b) {
                const int tiles = (sequence_length<false>(p, b) + TILE_KEYS - 1) / TILE_KEYS;
                total += static_cast<long long>(tiles) * head_tiles;
                longest = max(longest, tiles);
            }
            long long chunk = (total + clusters - 1) / clusters;
            chunk = max(chunk, static_cast<long long>((longest + p.splits - 2) / (p.splits - 1)));
            chunk = max(chunk, 1LL);
            schedule.chunk = static_cast<int>(min(chunk, 0x7fffffffLL));
            schedule.total = static_cast<int>(min(total, 0x7fffffffLL));
            const long long lo = static_cast<long long>(cluster) * schedule.chunk;
            int unit = 0;
            long long offset = 0;
            const int units = p.batch * head_tiles;
            while (unit < units) {
                const int tiles = unit_tiles<false>(p, unit, head_tiles);
                if (offset + tiles > lo) {
                    break;
                }
                offset += tiles;
                ++unit;
            }
            schedule.first_unit = unit;
            schedule.first_offset = static_cast<int>(offset);
        }
        sh->schedule = schedule;
    }
    if (warp == MMA_WARP) {
        tmem_alloc_pair(smem_u32(&sh->tmem_base), TMEM_COLUMNS);        // the same warp of both CTAs, together
        tmem_relinquish_pair();
    }
    if (warp == LOAD_WARP && lane == 0) {
        tma_prefetch_descriptor(CAUSAL ? &p.q_lat : &p.q_all);
        tma_prefetch_descriptor(&p.k_lat8);
        tma_prefetch_descriptor(&p.k_lat2);
        tma_prefetch_descriptor(&p.k_rope);
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                 // the other CTA's barriers exist before anything arrives on them
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&sh->tmem_base);
    const Schedule schedule = sh->schedule;

    Walker walker;
    walker.unit = (CAUSAL || p.splits == 1) ? cluster : schedule.first_unit;
    walker.offset = schedule.first_offset;
    walker.done = false;
    Segment seg;
    int segment_index = 0;      // segments this cluster has started (every role counts the same)
    int tile_index = 0;         // tiles this cluster has started, over all segments

    // Chunk c of a tile's own keys lives in slot c of its stage.  CTA r keeps slots {2r, 2r+1, 4+2r, 4+2r+1}
    // (its value columns); the other four are refilled with the other CTA's keys after S.
    if (warp == LOAD_WARP || warp == REFILL_WARP) {
        // =================== TMA producers ==================================
        // Three kinds of load per tile, each free to go as soon as what it overwrites has been read:
        //   A(t): the eight latent chunks of this CTA's own keys   - after P V of tile t-2 (same stage);
        //   R(t): the rotary chunk                                  - after the first four score MMAs of tile t-1;
        //   B(t): refill of the four S-only slots with the other CTA's keys - after this CTA's half of S(t).
        // Warp LOAD_WARP issues Q, A and the L2 prefetches; warp REFILL_WARP issues R and B, which sit on the
        // critical path (S waits for R, P V for B) and must not queue behind an A load and its prefetch.  All 32
        // lanes of a warp walk its loop, because the block-table entries are fetched 32 at a time, one per
        // lane; lane 0 tests and issues.  Each kind is issued in tile order by one thread, so a parity test
        // for tile t always comes after the phase of tile t - STAGES has been seen complete.
        bool alive = true;
        while (alive && next_segment<CAUSAL>(p, schedule, walker, seg, cluster, clusters)) {
            const int tile_count = seg.tile_end - seg.tile_begin;
            const int length = sequence_length<CAUSAL>(p, seg.b);
            const int last_half_start = ((length - 1) / HALF_KEYS) * HALF_KEYS;
            // Physical cache row (page * page_size + offset) of the first key of a 64-key half-tile of this
            // sequence.  Each kind of load walks the half-tiles in order and keeps its own window of 32 rows.
            struct Window {
                int rows;       // lane l: row of half-tile first + l
                int first;
            };
            auto row_of = [&](Window& w, int half_tile) -> int {
                if (CAUSAL) {
                    // not paged: the keys of batch entry b are rows b * T .. of kv_latent / key_rope (a half past the
                    // end reads the next entry's rows or, behind the last one, zeros; those keys are masked)
                    return seg.b * p.sequence + half_tile * HALF_KEYS;
                }
                if (half_tile < w.first || half_tile >= w.first + 32) {
                    w.first = half_tile & ~31;
                    const int token = min((w.first + lane) * HALF_KEYS, last_half_start);     // a half past the end rereads the last one; it is masked
                    int page = __ldg(p.block_table + static_cast<size_t>(seg.b) * p.pages + token / p.page_size);
                    if (p.cache_blocks > 0 && static_cast<unsigned>(page) >= static_cast<unsigned>(p.cache_blocks)) {
                        atomicExch(&decode_status, STATUS_BAD_INDEX);       // a page number outside the cache: read page 0 instead and report it
                        page = 0;
                    }
                    w.rows = page * p.page_size + token % p.page_size;
                }
                return __shfl_sync(0xffffffffU, w.rows, half_tile & 31);
            };
            if (warp == LOAD_WARP) {
                const int q_row0 = (CAUSAL ? seg.b * p.sequence * p.heads : seg.b * p.heads) + seg.row_tile * PAIR_HEADS + static_cast<int>(rank) * CTA_HEADS;
                if (lane == 0) {
                    // Q may be overwritten once every score MMA of the previous segment has finished
                    if (segment_index > 0) {
                        alive = mbar_wait(smem_u32(&sh->o_final), (segment_index - 1) & 1, abort_flag, &decode_status);
                    }
                    if (alive) {
                        const uint32_t bar = smem_u32(&sh->q_full);
                        mbar_arrive_expect_tx(bar, Q_BYTES);
                        if (CAUSAL) {
                            tma_load_3d(q_smem, &p.q_lat, bar, 0, q_row0, 0);
                            tma_load_2d(q_smem + LATENT_CHUNKS * CHUNK, &p.q_rope, bar, 0, q_row0);
                        } else {
                            tma_load_3d(q_smem, &p.q_all, bar, 0, q_row0, 0);
                        }
                    }
                }
                alive = __shfl_sync(0xffffffffU, alive ? 1 : 0, 0) != 0;
                Window win_a = {0, -64}, win_p = {0, -64};
                // A tile load reads 128 bytes from each of 64 cache rows (1152 bytes apart) per chunk.  The 64 rows a
                // CTA owns in a tile are one contiguous piece of a page, so they are asked into L2 with one bulk
                // prefetch a few tiles ahead, and the tile loads then mostly hit L2.
                int next_p = 0;
                auto prefetch_up_to = [&](int limit) {
                    for (; next_p < min(limit, tile_count); ++next_p) {
                        const int row = row_of(win_p, 2 * (seg.tile_begin + next_p) + static_cast<int>(rank));
                        if (lane == 0 && !CAUSAL) {         // the causal forward rereads its keys row tile after row tile: they stay in L2
                            prefetch_l2_bulk(p.cache + static_cast<size_t>(row) * WIDTH, HALF_KEYS * WIDTH * 2);
                        }
                    }
                };
                prefetch_up_to(PREFETCH_TILES);
                for (int next_a = 0; next_a < tile_count && alive; ++next_a) {
                    const int tile = tile_index + next_a;
                    const int stage = tile % STAGES;
                    const int row = row_of(win_a, 2 * (seg.tile_begin + next_a) + static_cast<int>(rank));
                    if (tile >= STAGES) {
                        alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->stage_free[stage]), (tile / STAGES - 1) & 1, abort_flag, &decode_status));
                        if (!alive) {
                            break;
                        }
                    }
                    if (lane == 0) {
                        const uint32_t bar = smem_u32(&sh->full_a[stage]);
                        mbar_arrive_expect_tx(bar, STAGE_BYTES);
                        tma_load_3d(stage_smem + stage * STAGE_BYTES, &p.k_lat8, bar, 0, row, 0);
                    }
                    prefetch_up_to(next_a + 1 + PREFETCH_TILES);
                }
            } else {
                Window win_r = {0, -64}, win_b = {0, -64};
                int next_r = 0, next_b = 0;         // tiles of this segment whose load of that kind is still to be issued
                long long idle_since = clock64();
                while (alive && (next_r < tile_count || next_b < tile_count)) {
                    int action = 0;
                    if (lane == 0) {
                        if (next_r < tile_count) {
                            const int tile = tile_index + next_r;
                            if (tile == 0 || mbar_test_wait(smem_u32(&sh->rope_free), (tile - 1) & 1)) {
                                action = 2;
                            }
                        }
                        if (action == 0 && next_b < tile_count) {
                            const int tile = tile_index + next_b;
                            if (mbar_test_wait(smem_u32(&sh->refill_free[tile % STAGES]), (tile / STAGES) & 1)) {
                                action = 3;
                            }
                        }
                        if (action == 0 && (*abort_flag != 0 || clock64() - idle_since > WAIT_LIMIT_CYCLES)) {
                            *abort_flag = 1;
                            atomicExch(&decode_status, STATUS_WAIT_TIMEOUT);
                            action = -1;
                        }
                    }
                    action = __shfl_sync(0xffffffffU, action, 0);
                    if (action < 0) {
                        alive = false;
                    } else if (action == 2) {
                        const int row = row_of(win_r, 2 * (seg.tile_begin + next_r) + static_cast<int>(rank));
                        if (lane == 0) {
                            const uint32_t bar = smem_u32(&sh->full_r);
                            mbar_arrive_expect_tx(bar, CHUNK);
                            tma_load_2d(rope_smem, &p.k_rope, bar, 0, row);
                        }
                        ++next_r;
                    } else if (action == 3) {
                        const int tile = tile_index + next_b;
                        const int stage = tile % STAGES;
                        const int row = row_of(win_b, 2 * (seg.tile_begin + next_b) + static_cast<int>(peer));
                        if (lane == 0) {
                            const uint32_t bar = smem_u32(&sh->full_b[stage]);
                            mbar_arrive_expect_tx(bar, 4 * CHUNK);
                            for (int a = 0; a < 2; ++a) {
                                // the other CTA's keys, this CTA's value columns -> the two adjacent slots only S needed
                                const int chunk = 4 * a + 2 * static_cast<int>(rank);
                                const int slot = 4 * a + 2 * static_cast<int>(peer);
                                tma_load_3d(stage_smem + stage * STAGE_BYTES + slot * CHUNK, &p.k_lat2, bar, 0, row, chunk);
                            }
                        }
                        ++next_b;
                    }
                    if (action > 0) {
                        idle_since = clock64();
                    }
                }
            }
            tile_index += tile_count;
            segment_index += 1;
        }
    } else if (warp == MMA_WARP && rank != 0) {
        // =================== relay: this CTA's "loaded" events -> the leader =========
        // One thread: each landed load of this CTA is forwarded as one arrival on the leader's matching
        // barrier, in whatever order the loads land (per kind they land in tile order).
        if (lane == 0) {
            bool alive = true;
            const uint32_t leader_q = map_to_cta(smem_u32(&sh->peer_q_full), 0);
            const uint32_t leader_r = map_to_cta(smem_u32(&sh->peer_full_r), 0);
            const uint32_t leader_a0 = map_to_cta(smem_u32(&sh->peer_full_a[0]), 0);
            const uint32_t leader_b0 = map_to_cta(smem_u32(&sh->peer_full_b[0]), 0);
            static_assert(STAGES == 2, "the relay addresses the two stage barriers as base + 8 * stage");
            while (alive && next_segment<CAUSAL>(p, schedule, walker, seg, cluster, clusters)) {
                const int tile_count = seg.tile_end - seg.tile_begin;
                alive = mbar_wait(smem_u32(&sh->q_full), segment_index & 1, abort_flag, &decode_status);
                if (alive) {
                    mbar_arrive_remote(leader_q);
                }
                int next_a = 0, next_r = 0, next_b = 0;
                long long idle_since = clock64();
                while (alive && (next_a < tile_count || next_r < tile_count || next_b < tile_count)) {
                    bool progress = false;
                    if (next_r < tile_count) {
                        const int tile = tile_index + next_r;
                        if (mbar_test_wait(smem_u32(&sh->full_r), tile & 1)) {
                            mbar_arrive_remote(leader_r);
                            ++next_r;
                            progress = true;
                        }
                    }
                    if (next_a < tile_count) {
                        const int tile = tile_index + next_a;
                        if (mbar_test_wait(smem_u32(&sh->full_a[tile % STAGES]), (tile / STAGES) & 1)) {
                            mbar_arrive_remote(leader_a0 + 8 * (tile % STAGES));
                            ++next_a;
                            progress = true;
                        }
                    }
                    if (next_b < tile_count) {
                        const int tile = tile_index + next_b;
                        if (mbar_test_wait(smem_u32(&sh->full_b[tile % STAGES]), (tile / STAGES) & 1)) {
                            mbar_arrive_remote(leader_b0 + 8 * (tile % STAGES));
                            ++next_b;
                            progress = true;
                        }
                    }
                    if (progress) {
                        idle_since = clock64();
                    } else if (*abort_flag != 0 || clock64() - idle_since > WAIT_LIMIT_CYCLES) {
                        *abort_flag = 1;
                        atomicExch(&decode_status, STATUS_WAIT_TIMEOUT);
                        alive = false;
                    }
                }
                tile_index += tile_count;
                segment_index += 1;
            }
        }
    } else if (warp == MMA_WARP) {
        // =================== MMA issuer (leader CTA) ============================
        // Lane 0 watches the barriers and picks what to issue; the whole warp then runs the issue code
        // (uniform control flow) and the elected lane executes the tcgen05 instructions.
        const uint32_t leader = elect_one();
        constexpr uint32_t IDESC_QK = make_idesc_bf16(PAIR_HEADS, TILE_KEYS, false, false);
        constexpr uint32_t IDESC_PV = make_idesc_bf16(PAIR_HEADS, 256, false, true);
        constexpr uint32_t HI = smem_desc_hi(1024);
        const uint32_t q_lo = smem_desc_lo(q_smem, 16);
        const uint32_t rope_lo = smem_desc_lo(rope_smem, 16);
        const uint32_t p_lo = smem_desc_lo(p_smem, 16);
        bool alive = true;
        auto both = [&](uint64_t* bar) {        // one commit for this CTA's barrier, one for the other CTA's
            commit_pair(smem_u32(bar), leader);
            commit_pair(map_to_cta(smem_u32(bar), 1), leader);
        };
        // own keys and rotary chunk of `tile` have landed in both CTAs
        auto s_ready = [&](int tile) -> bool {
            const int stage = tile % STAGES;
            const uint32_t parity = (tile / STAGES) & 1;
            return mbar_test_wait(smem_u32(&sh->full_a[stage]), parity) && mbar_test_wait(smem_u32(&sh->peer_full_a[stage]), parity) &&
                   mbar_test_wait(smem_u32(&sh->full_r), tile & 1) && mbar_test_wait(smem_u32(&sh->peer_full_r), tile & 1);
        };
        // P of `tile` is stored and the refilled slots have landed, in both CTAs
        auto pv_ready = [&](int tile) -> bool {
            const int stage = tile % STAGES;
            const uint32_t parity = (tile / STAGES) & 1;
            return mbar_test_wait(smem_u32(&sh->p_full), tile & 1) && mbar_test_wait(smem_u32(&sh->full_b[stage]), parity) &&
                   mbar_test_wait(smem_u32(&sh->peer_full_b[stage]), parity);
        };
        auto issue_s = [&](int tile) {
            const int stage = tile % STAGES;
            const uint32_t s_tmem = tmem_base + TMEM_S + (tile & 1) * HALF_KEYS;
            const uint32_t stage_lo = smem_desc_lo(stage_smem + stage * STAGE_BYTES, 16);
            // The rotary chunk first: there is one slot for it, and the next tile's chunk can only be loaded once
            // these four MMAs have read it.  Then slots {2,3,6,7} (S-only in the leader), then {0,1,4,5} (S-only in
            // the other CTA); each group's commit lets that CTA refill the slots.
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                mma_pair_ss_split(s_tmem, q_lo + LATENT_CHUNKS * (CHUNK >> 4) + 2 * k, HI, rope_lo + 2 * k, HI, IDESC_QK, k != 0 ? 1U : 0U, leader);
            }
            both(&sh->rope_free);
#pragma unroll
            for (int group = 0; group < 2; ++group) {
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    const int c = (group == 0 ? 2 : 0) + (n & 1) + (n >> 1) * 4;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        mma_pair_ss_split(s_tmem, q_lo + c * (CHUNK >> 4) + 2 * k, HI, stage_lo + c * (CHUNK >> 4) + 2 * k, HI, IDESC_QK, 1U, leader);
                    }
                }
                if (group == 0) {
                    commit_pair(smem_u32(&sh->refill_free[stage]), leader);
                } else {
                    commit_pair(map_to_cta(smem_u32(&sh->refill_free[stage]), 1), leader);
                }
            }
            both(&sh->s_full[tile & 1]);
        };
        auto issue_pv = [&](int tile, bool first_of_segment, bool last_of_segment) {
            const int stage = tile % STAGES;
            const uint32_t v_lo = smem_desc_lo(stage_smem + stage * STAGE_BYTES, CHUNK);      // MN-major: the two 64-column chunks are CHUNK apart
#pragma unroll
            for (int a = 0; a < 2; ++a) {
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const int g = kk >> 2;          // which 64 keys of the tile
                    mma_pair_ss_split(tmem_base + TMEM_O + a * 128, p_lo + g * (CHUNK >> 4) + 2 * (kk & 3), HI,
                                      v_lo + (4 * a + 2 * g) * (CHUNK >> 4) + (kk & 3) * (2048 >> 4), HI, IDESC_PV, (first_of_segment && kk == 0) ? 0U : 1U,
                                      leader);
                }
            }
            both(&sh->stage_free[stage]);
            both(&sh->p_free);
            if (last_of_segment) {
                both(&sh->o_final);
            }
        };
        while (alive && next_segment<CAUSAL>(p, schedule, walker, seg, cluster, clusters)) {
            const int tile_count = seg.tile_end - seg.tile_begin;
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->q_full), segment_index & 1, abort_flag, &decode_status) &&
                                                mbar_wait(smem_u32(&sh->peer_q_full), segment_index & 1, abort_flag, &decode_status));
            // Owed at any time: S of the next tile not yet issued (it runs while the softmax of the tile before
            // it is computed) and P V of the oldest tile not yet done.  Whichever has its inputs first goes
            // first: waiting for cache rows must not hold back a P V whose P is there, and the other way round.
            int next_s = 0, next_pv = 0;
            long long idle_since = clock64();
            while (alive && next_pv < tile_count) {
                int action = 0;
                if (lane == 0) {
                    if (next_s < tile_count && next_s <= next_pv + 1 && s_ready(tile_index + next_s)) {
                        action = 1;
                    } else if (next_pv < next_s && pv_ready(tile_index + next_pv)) {
                        action = 2;
                    } else if (*abort_flag != 0 || clock64() - idle_since > WAIT_LIMIT_CYCLES) {
                        *abort_flag = 1;
                        atomicExch(&decode_status, STATUS_WAIT_TIMEOUT);
                        action = -1;
                    }
                }
                action = __shfl_sync(0xffffffffU, action, 0);
                if (action < 0) {
                    alive = false;
                } else if (action == 1) {
                    tc_fence_after_sync();
                    issue_s(tile_index + next_s);
                    ++next_s;
                    idle_since = clock64();
                } else if (action == 2) {
                    tc_fence_after_sync();
                    issue_pv(tile_index + next_pv, next_pv == 0, next_pv + 1 == tile_count);
                    ++next_pv;
                    idle_since = clock64();
                }
            }
            tile_index += tile_count;
            segment_index += 1;
        }
    } else {
        // =================== softmax + epilogue: thread = (head, half of the tile's keys) ============
        const int r = threadIdx.x;                          // tensor-memory lane
        const int head_in_cta = r & 63;
        const int key_half = r >> 6;
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        const uint32_t p_full_bar = rank == 0 ? smem_u32(&sh->p_full) : map_to_cta(smem_u32(&sh->p_full), 0);
        bool alive = true;

        while (alive && next_segment<CAUSAL>(p, schedule, walker, seg, cluster, clusters)) {
            const int tile_count = seg.tile_end - seg.tile_begin;
            // decode: row = head of the sequence's one query token.  Causal forward: row = (token, head) pair of the batch entry.
            const int row = seg.row_tile * PAIR_HEADS + static_cast<int>(rank) * CTA_HEADS + head_in_cta;
            const int head = CAUSAL ? row % p.heads : row;
            const int token = CAUSAL ? row / p.heads : 0;
            const bool valid = CAUSAL ? token < p.sequence : head < p.heads;
            const int kv_end = min(sequence_length<CAUSAL>(p, seg.b), seg.tile_end * TILE_KEYS);      // keys >= kv_end are not part of this segment
            const int key_limit = CAUSAL ? min(kv_end, token + 1) : kv_end;                          // keys this row may attend to
            float m_ref = 0.0F;
            float l_sum = 0.0F;
            for (int j = 0; j < tile_count && alive; ++j) {
                const int tile = tile_index + j;
                const int stage = tile % STAGES;
                const uint32_t s_tmem = tmem_base + lane_base + TMEM_S + (tile & 1) * HALF_KEYS;
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->s_full[tile & 1]), (tile >> 1) & 1, abort_flag, &decode_status));
                if (!alive) {
                    break;
                }
                tc_fence_after_sync();
                uint32_t sb[HALF_KEYS];
                tmem_ld_x32(s_tmem, sb);
                tmem_ld_x32(s_tmem + 32, sb + 32);
                tmem_wait_ld();
                const int token0 = (seg.tile_begin + j) * TILE_KEYS + key_half * HALF_KEYS;
                const bool ragged = (seg.tile_begin + j + 1) * TILE_KEYS > kv_end;          // warp-uniform: some key of the tile is past the end
                if (token0 + HALF_KEYS > key_limit) {
#pragma unroll
                    for (int n = 0; n < HALF_KEYS; ++n) {
                        sb[n] = token0 + n < key_limit ? sb[n] : 0xff800000U;
                    }
                }
                // three-input maxima, four independent chains
                float mx0 = __uint_as_float(sb[0]), mx1 = __uint_as_float(sb[1]), mx2 = __uint_as_float(sb[2]), mx3 = __uint_as_float(sb[3]);
#pragma unroll
                for (int n = 4; n + 7 < HALF_KEYS; n += 8) {
                    mx0 = max3(mx0, __uint_as_float(sb[n]), __uint_as_float(sb[n + 1]));
                    mx1 = max3(mx1, __uint_as_float(sb[n + 2]), __uint_as_float(sb[n + 3]));
                    mx2 = max3(mx2, __uint_as_float(sb[n + 4]), __uint_as_float(sb[n + 5]));
                    mx3 = max3(mx3, __uint_as_float(sb[n + 6]), __uint_as_float(sb[n + 7]));
                }
                mx0 = max3(mx0, __uint_as_float(sb[HALF_KEYS - 4]), __uint_as_float(sb[HALF_KEYS - 3]));
                mx1 = max3(mx1, __uint_as_float(sb[HALF_KEYS - 2]), __uint_as_float(sb[HALF_KEYS - 1]));
                // The two threads of a head agree on the tile's maximum.  One buffer and one barrier per tile
                // parity: a thread can only be one tile ahead of the slowest, because it needs everyone's
                // arrival on the other parity's barrier in between.
                float tile_max = fmaxf(fmaxf(mx0, mx2), fmaxf(mx1, mx3));
                sh->maxima[tile & 1][r] = tile_max;
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(smem_u32(&sh->max_ready[tile & 1]));
                }
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->max_ready[tile & 1]), (tile >> 1) & 1, abort_flag, &decode_status));
                if (!alive) {
                    break;
                }
                tile_max = fmaxf(tile_max, sh->maxima[tile & 1][r ^ 64]);
                // The first key of a segment is always valid for key half 0 (every row may attend to key 0), so tile_max
                // is finite on the first tile; a later tile may be masked altogether for a row (tile_max = -inf),
                // which leaves m_ref alone and turns into probabilities of exactly 0.
                float alpha = 1.0F;
                bool grow = false;
                if (j == 0) {
                    m_ref = tile_max;
                } else {
                    grow = (tile_max - m_ref) * p.scale_log2 > RESCALE_THRESHOLD;
                    if (grow) {
                        alpha = exp2_approx((m_ref - tile_max) * p.scale_log2);
                        m_ref = tile_max;
                        l_sum *= alpha;
                    }
                }
                const float bias = -m_ref * p.scale_log2;
                float2 sums = make_float2(0.0F, 0.0F);
                const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
                const float2 bias2 = make_float2(bias, bias);
                uint32_t packed[HALF_KEYS / 2];
#pragma unroll
                for (int e = 0; e < HALF_KEYS / 2; ++e) {
                    const float2 x = fma2(make_float2(__uint_as_float(sb[2 * e]), __uint_as_float(sb[2 * e + 1])), scale2, bias2);
                    const float2 pr = make_float2(exp2_approx(x.x), exp2_approx(x.y));
                    sums = add2(sums, pr);
                    packed[e] = pack_bf16x2(pr.x, pr.y);
                }
                l_sum += sums.x + sums.y;
                // P and O belong to the previous tile's P V until it has finished
                if (tile > 0) {
                    alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->p_free), (tile - 1) & 1, abort_flag, &decode_status));
                    if (!alive) {
                        break;
                    }
                    tc_fence_after_sync();
                }
                if (__any_sync(0xffffffffU, grow)) {
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        uint32_t o[32];
                        tmem_ld_x32(tmem_base + lane_base + TMEM_O + c * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                        }
                        tmem_st_x32(tmem_base + lane_base + TMEM_O + c * 32, o);
                    }
                    tmem_wait_st();
                }
                // row head_in_cta of chunk key_half of P: 64 keys = eight 16-byte units, swizzled by the row
                uint8_t* p_row = p_ptr + key_half * CHUNK + head_in_cta * 128;
#pragma unroll
                for (int unit = 0; unit < 8; ++unit) {
                    *reinterpret_cast<uint4*>(p_row + ((unit ^ (head_in_cta & 7)) * 16)) =
                        make_uint4(packed[4 * unit], packed[4 * unit + 1], packed[4 * unit + 2], packed[4 * unit + 3]);
                }
                if (ragged) {
                    // Keys past the end may hold anything (the page is only partly written): zero their rows in
                    // this CTA's value chunks so that 0 * V stays 0.  Key half g of the tile sits in slots
                    // 4a+2g, 4a+2g+1; the refilled ones must have landed first.
                    alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->full_b[stage]), (tile / STAGES) & 1, abort_flag, &decode_status));
                    if (!alive) {
                        break;
                    }
                    uint8_t* stage_rows = stage_ptr + stage * STAGE_BYTES;
                    for (int g = 0; g < 2; ++g) {
                        const int first_bad = max(0, kv_end - ((seg.tile_begin + j) * TILE_KEYS + g * HALF_KEYS));      // rows >= first_bad of this half
                        const int bad_units = (HALF_KEYS - min(first_bad, HALF_KEYS)) * 8;                        // 16-byte units per chunk
                        for (int u = r; u < bad_units * 4; u += PAIR_HEADS) {
                            const int which = u / bad_units;                  // 0..3 -> slots 2g, 2g+1, 4+2g, 4+2g+1
                            const int within = u % bad_units;
                            const int slot = (which >> 1) * 4 + 2 * g + (which & 1);
                            *reinterpret_cast<uint4*>(stage_rows + slot * CHUNK + (first_bad + within / 8) * 128 + (within % 8) * 16) = make_uint4(0, 0, 0, 0);
                        }
                    }
                }
                fence_proxy_async_smem();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (rank == 0) {
                        mbar_arrive(p_full_bar);
                    } else {
                        mbar_arrive_remote(p_full_bar);
                    }
                }
            }

            if (alive) {
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->o_final), segment_index & 1, abort_flag, &decode_status));
            }
            if (!alive) {
                break;
            }
            tc_fence_after_sync();
            // the head's row sum is the sum of its two threads' sums (the buffer is free: every thread has
            // been through the tiles of this segment since it last read it)
            sh->sums[r] = l_sum;
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(&sh->sum_ready));
            }
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->sum_ready), segment_index & 1, abort_flag, &decode_status));
            if (!alive) {
                break;
            }
            const float l_total = l_sum + sh->sums[r ^ 64];
            const float inverse = 1.0F / l_total;
            if (CAUSAL) {
                // the finished rows: bf16 output [B,T,H,512] and the natural-log LSE [B,H,T]
                __nv_bfloat16* out_row = p.out + ((static_cast<size_t>(seg.b) * p.sequence + (valid ? token : 0)) * p.heads + head) * RANK;
                if (valid && key_half == 0) {
                    p.lse[(static_cast<size_t>(seg.b) * p.heads + head) * p.sequence + token] = m_ref * p.scale + logf(l_total);
                }
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    uint32_t o[32];
                    tmem_ld_x32(tmem_base + lane_base + TMEM_O + c * 32, o);
                    tmem_wait_ld();
                    if (valid) {
                        uint4* dst = reinterpret_cast<uint4*>(out_row + (c >> 2) * 256 + key_half * 128 + (c & 3) * 32);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            dst[e] = make_uint4(pack_bf16x2(__uint_as_float(o[8 * e]) * inverse, __uint_as_float(o[8 * e + 1]) * inverse),
                                                pack_bf16x2(__uint_as_float(o[8 * e + 2]) * inverse, __uint_as_float(o[8 * e + 3]) * inverse),
                                                pack_bf16x2(__uint_as_float(o[8 * e + 4]) * inverse, __uint_as_float(o[8 * e + 5]) * inverse),
                                                pack_bf16x2(__uint_as_float(o[8 * e + 6]) * inverse, __uint_as_float(o[8 * e + 7]) * inverse));
                        }
                    }
                }
            } else {
                float* records = p.workspace + (static_cast<size_t>(seg.b) * p.heads + (valid ? head : 0)) * p.splits * (RANK + 2);
                float* record = records + static_cast<size_t>(seg.slot) * (RANK + 2);
                // A record is (log-sum-exp of the partial, 1, normalised output): decode_combine_kernel weights the
                // partials of a (sequence, head) by exp(lse - max lse).
                if (valid && key_half == 0) {
                    record[0] = m_ref * p.scale + logf(l_total);
                    record[1] = 1.0F;
                    if (seg.last_of_unit && seg.slot + 1 < p.splits) {
                        // a sequence fills slots 0..slot in order; the first unused one ends the list (its row sum is 0)
                        records[static_cast<size_t>(seg.slot + 1) * (RANK + 2)] = -INFINITY;
                        records[static_cast<size_t>(seg.slot + 1) * (RANK + 2) + 1] = 0.0F;
                    }
                }
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    uint32_t o[32];
                    tmem_ld_x32(tmem_base + lane_base + TMEM_O + c * 32, o);
                    tmem_wait_ld();
                    if (valid) {
                        // accumulator a = c / 4, lanes 64.. hold its columns 128..255
                        float2* dst = reinterpret_cast<float2*>(record + 2 + (c >> 2) * 256 + key_half * 128 + (c & 3) * 32);
#pragma unroll
                        for (int e = 0; e < 32; e += 2) {
                            dst[e / 2] = make_float2(__uint_as_float(o[e]) * inverse, __uint_as_float(o[e + 1]) * inverse);
                        }
                    }
                }
            }
            // O may be overwritten by the next segment only after every lane has been read out: the next
            // segment's first P V waits for the P arrivals of every softmax thread, which come after this point.
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
    cluster_sync_all();                 // neither CTA frees tensor memory or exits while the other may still signal it
    if (warp == MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, TMEM_COLUMNS);
    }
}

// The two kernels: one body, two schedules (see the file header).
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1) absorbed_decode_kernel(const __grid_constant__ DecodeParams p) {
    absorbed_pair_body<false>(p);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1) absorbed_attention_kernel(const __grid_constant__ DecodeParams p) {
    absorbed_pair_body<true>(p);
}

// Merges the split partials of one (sequence, head).  A record is (log-sum-exp of the
// partial, 1, normalised output); the partials are weighted by exp(lse_s - max lse).
// Writes bf16 output and the natural-log LSE.  A sequence without cached tokens has no
// partial at all: its output is NaN and its LSE -inf, what the softmax of an empty row
// gives in the reference (reference/python/mla.py:36-38).
__global__ void __launch_bounds__(128) decode_combine_kernel(__nv_bfloat16* output, float* logsumexp, const float* workspace,
                                                             const int* lengths, int heads, int splits) {
    const int row = blockIdx.y * heads + blockIdx.x;
    if (lengths[blockIdx.y] <= 0) {
        const uint32_t nan2 = 0x7fc07fc0U;
        *reinterpret_cast<uint2*>(output + static_cast<size_t>(row) * RANK + threadIdx.x * 4) = make_uint2(nan2, nan2);
        if (threadIdx.x == 0) {
            logsumexp[row] = -INFINITY;
        }
        return;
    }
    const float* records = workspace + static_cast<size_t>(row) * splits * (RANK + 2);
    // Slots are filled in order from 0; the first one with a zero row sum ends the list.
    float maximum = -INFINITY;
    int used = 0;
    for (; used < splits; ++used) {
        const float l = records[static_cast<size_t>(used) * (RANK + 2) + 1];
        if (!(l > 0.0F)) {
            break;
        }
        maximum = fmaxf(maximum, records[static_cast<size_t>(used) * (RANK + 2)]);
    }
    float normalizer = 0.0F;
    float acc[4] = {0.0F, 0.0F, 0.0F, 0.0F};
    const int column = threadIdx.x * 4;
    for (int s = 0; s < used; ++s) {
        const float* record = records + static_cast<size_t>(s) * (RANK + 2);
        const float weight = __expf(record[0] - maximum);
        normalizer += weight * record[1];
        const float2 lo = *reinterpret_cast<const float2*>(record + 2 + column);
        const float2 hi = *reinterpret_cast<const float2*>(record + 4 + column);
        acc[0] += weight * lo.x;
        acc[1] += weight * lo.y;
        acc[2] += weight * hi.x;
        acc[3] += weight * hi.y;
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
    CUDA_CHECK(cudaFuncSetAttribute(absorbed_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    CUDA_CHECK(cudaFuncSetAttribute(absorbed_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    if (device < 16) {
        done[device] = true;
    }
}

int multiprocessor_count() {
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
    return count;
}

// Shared by the decode entry points.  `cache_blocks` <= 0: the number of physical pages is
// unknown (the reference's interface does not carry it).
void launch_decode(__nv_bfloat16* output, float* logsumexp, const __nv_bfloat16* query, const __nv_bfloat16* paged_kv_cache,
                   const int* block_table, const int* cache_lengths, float* workspace, int batch_size, int heads, int kv_rank,
                   int rope_size, int page_size, int pages_per_sequence, int cache_blocks, int splits, float scale, cudaStream_t stream) {
    // kernels/attention/mla/sm89.cu:20-24 of the reference: same condition, same message.
    if (kv_rank != MLA_KV_RANK || rope_size != MLA_ROPE_SIZE) {
        throw std::invalid_argument("MLA requires C=512 and RoPE=64");
    }
    if (batch_size <= 0 || heads <= 0 || pages_per_sequence <= 0 || splits <= 0) {
        throw std::invalid_argument("MLA decode requires positive batch, heads, pages and splits");
    }
    if (page_size <= 0 || page_size % HALF_KEYS != 0) {
        throw std::invalid_argument("MLA decode requires page_size to be a positive multiple of 64");
    }
    if (!(scale > 0.0F)) {
        throw std::invalid_argument("MLA decode requires a positive softmax scale");
    }
    if (batch_size > 65535 || splits > 65535 || static_cast<long long>(batch_size) * heads > 0x7fffffffLL ||
        static_cast<long long>(pages_per_sequence) * page_size > 0x7fffffffLL) {
        throw std::invalid_argument("MLA decode shape exceeds the supported index range");
    }
    for (const void* pointer : {static_cast<const void*>(output), static_cast<const void*>(logsumexp), static_cast<const void*>(query),
                                static_cast<const void*>(paged_kv_cache), static_cast<const void*>(workspace)}) {
        if (pointer == nullptr) {
            throw std::invalid_argument("null tensor pointer");
        }
        if ((reinterpret_cast<std::uintptr_t>(pointer) & 15U) != 0) {
            throw std::invalid_argument("tensor pointers must be 16-byte aligned");
        }
    }
    if (block_table == nullptr || cache_lengths == nullptr) {
        throw std::invalid_argument("null tensor pointer");
    }
    DecodeParams params{};
    const std::uint64_t q_rows = static_cast<std::uint64_t>(batch_size) * heads;
    // Without a page count the view is given the largest row count a tensor map can hold and
    // only rows named by the block table are ever touched.  With one, the view ends where the
    // cache ends and a page number outside it is replaced and reported by the kernel.
    const std::uint64_t k_rows = cache_blocks > 0 ? static_cast<std::uint64_t>(cache_blocks) * page_size : 1ULL << 31;
    params.q_all = make_bf16_chunked_map(query, q_rows, 9, WIDTH, CTA_HEADS, 9);
    params.k_lat8 = make_bf16_chunked_map(paged_kv_cache, k_rows, LATENT_CHUNKS, WIDTH, HALF_KEYS, LATENT_CHUNKS);
    params.k_lat2 = make_bf16_chunked_map(paged_kv_cache, k_rows, LATENT_CHUNKS, WIDTH, HALF_KEYS, 2);
    params.k_rope = make_bf16_tile_map(paged_kv_cache + RANK, k_rows, ROPE, WIDTH, HALF_KEYS);
    params.cache = paged_kv_cache;
    params.block_table = block_table;
    params.lengths = cache_lengths;
    params.workspace = workspace;
    params.batch = batch_size;
    params.heads = heads;
    params.page_size = page_size;
    params.pages = pages_per_sequence;
    params.splits = splits;
    params.cache_blocks = cache_blocks > 0 ? cache_blocks : 0;
    params.scale = scale;
    params.scale_log2 = scale * 1.4426950408889634F;
    configure_kernel();
    // one cluster of two CTAs per SM pair
    const int clusters = std::max(1, multiprocessor_count() / 2);
    absorbed_decode_kernel<<<dim3(2 * clusters, 1, 1), THREADS, SMEM_BYTES, stream>>>(params);
    CUDA_CHECK(cudaGetLastError());
    decode_combine_kernel<<<dim3(heads, batch_size), 128, 0, stream>>>(output, logsumexp, workspace, cache_lengths, heads, splits);
    CUDA_CHECK(cudaGetLastError());
}

}  // namespace

namespace internal {

int decode_device_status(bool reset) {
    int status = 0;
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemcpyFromSymbol(&status, decode_status, sizeof(int)));
    if (reset && status != 0) {
        const int zero = 0;
        CUDA_CHECK(cudaMemcpyToSymbol(decode_status, &zero, sizeof(int)));
    }
    return status;
}

}  // namespace internal

// The absorbed causal forward on the same cluster kernel: rows are (token, head) pairs, keys are the rows
// of kv_latent / key_rope up to each row's own token, the output is final (no partials, no combine).
void mla_compressed_attention_forward_cuda(__nv_bfloat16* output, float* logsumexp, const __nv_bfloat16* query_latent,
                                           const __nv_bfloat16* query_rope, const __nv_bfloat16* kv_latent, const __nv_bfloat16* key_rope,
                                           int batch_size, int sequence_length, int heads, int kv_rank, int rope_size, float scale,
                                           cudaStream_t stream) {
    // kernels/attention/mla/sm89.cu:20-24 of the reference: same condition, same message.
    if (kv_rank != MLA_KV_RANK || rope_size != MLA_ROPE_SIZE) {
        throw std::invalid_argument("MLA requires C=512 and RoPE=64");
    }
    if (batch_size <= 0 || sequence_length <= 0 || heads <= 0) {
        throw std::invalid_argument("MLA forward requires positive batch, sequence length and heads");
    }
    if (!(scale > 0.0F)) {
        throw std::invalid_argument("MLA forward requires a positive softmax scale");
    }
    if (static_cast<long long>(sequence_length) * heads * batch_size > 0x7fffffffLL) {
        throw std::invalid_argument("MLA forward shape exceeds the supported index range");
    }
    for (const void* pointer : {static_cast<const void*>(output), static_cast<const void*>(logsumexp), static_cast<const void*>(query_latent),
                                static_cast<const void*>(query_rope), static_cast<const void*>(kv_latent), static_cast<const void*>(key_rope)}) {
        if (pointer == nullptr) {
            throw std::invalid_argument("null tensor pointer");
        }
        if ((reinterpret_cast<std::uintptr_t>(pointer) & 15U) != 0) {
            throw std::invalid_argument("tensor pointers must be 16-byte aligned");
        }
    }
    DecodeParams params{};
    const std::uint64_t q_rows = static_cast<std::uint64_t>(batch_size) * sequence_length * heads;
    const std::uint64_t k_rows = static_cast<std::uint64_t>(batch_size) * sequence_length;
    params.q_lat = make_bf16_chunked_map(query_latent, q_rows, LATENT_CHUNKS, RANK, CTA_HEADS, LATENT_CHUNKS);
    params.q_rope = make_bf16_tile_map(query_rope, q_rows, ROPE, ROPE, CTA_HEADS);
    params.q_all = params.q_lat;
    params.k_lat8 = make_bf16_chunked_map(kv_latent, k_rows, LATENT_CHUNKS, RANK, HALF_KEYS, LATENT_CHUNKS);
    params.k_lat2 = make_bf16_chunked_map(kv_latent, k_rows, LATENT_CHUNKS, RANK, HALF_KEYS, 2);
    params.k_rope = make_bf16_tile_map(key_rope, k_rows, ROPE, ROPE, HALF_KEYS);
    params.out = output;
    params.lse = logsumexp;
    params.sequence = sequence_length;
    params.batch = batch_size;
    params.heads = heads;
    params.splits = 1;
    params.scale = scale;
    params.scale_log2 = scale * 1.4426950408889634F;
    configure_kernel();
    const long long row_tiles = (static_cast<long long>(sequence_length) * heads + PAIR_HEADS - 1) / PAIR_HEADS * batch_size;
    const int clusters = static_cast<int>(std::max(1LL, std::min<long long>(multiprocessor_count() / 2, row_tiles)));
    absorbed_attention_kernel<<<dim3(2 * clusters, 1, 1), THREADS, SMEM_BYTES, stream>>>(params);
    CUDA_CHECK(cudaGetLastError());
}

std::size_t mla_decode_workspace_elements(int batch_size, int heads, int splits, int kv_rank) {
    // kernels/attention/mla/sm89.cu:539-541 of the reference.
    return static_cast<std::size_t>(batch_size) * heads * splits * (kv_rank + 2);
}

void mla_decode_forward_cuda(__nv_bfloat16* output, float* logsumexp, const __nv_bfloat16* query, const __nv_bfloat16* paged_kv_cache,
                             const int* block_table, const int* cache_lengths, float* workspace, int batch_size, int heads, int kv_rank,
                             int rope_size, int page_size, int pages_per_sequence, int splits, float scale, cudaStream_t stream) {
    launch_decode(output, logsumexp, query, paged_kv_cache, block_table, cache_lengths, workspace, batch_size, heads, kv_rank, rope_size,
                  page_size, pages_per_sequence, 0, splits, scale, stream);
}

void mla_decode_forward_checked_cuda(__nv_bfloat16* output, float* logsumexp, const __nv_bfloat16* query,
                                     const __nv_bfloat16* paged_kv_cache, const int* block_table, const int* cache_lengths,
                                     float* workspace, int batch_size, int heads, int kv_rank, int rope_size, int page_size,
                                     int pages_per_sequence, int cache_blocks, int splits, float scale, cudaStream_t stream) {
    if (cache_blocks <= 0) {
        throw std::invalid_argument("checked MLA decode requires the number of cache pages");
    }
    launch_decode(output, logsumexp, query, paged_kv_cache, block_table, cache_lengths, workspace, batch_size, heads, kv_rank, rope_size,
                  page_size, pages_per_sequence, cache_blocks, splits, scale, stream);
}

std::size_t mla_decode_static_capacity() {
    return STATIC_DECODE_RECORDS;
}

void mla_decode_forward_static_cuda(__nv_bfloat16* output, float* logsumexp, const __nv_bfloat16* query,
                                    const __nv_bfloat16* paged_kv_cache, const int* block_table, const int* cache_lengths, int batch_size,
                                    int heads, int kv_rank, int rope_size, int page_size, int pages_per_sequence, int splits, float scale,
                                    cudaStream_t stream) {
    if (kv_rank != MLA_KV_RANK || rope_size != MLA_ROPE_SIZE) {
        throw std::invalid_argument("MLA requires C=512 and RoPE=64");
    }
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
    launch_decode(output, logsumexp, query, paged_kv_cache, block_table, cache_lengths, scratch, batch_size, heads, kv_rank, rope_size,
                  page_size, pages_per_sequence, 0, splits, scale, stream);
}

}  // namespace dscuda
