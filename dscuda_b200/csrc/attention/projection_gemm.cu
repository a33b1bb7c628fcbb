// The dense projections either side of the attention kernels, on the sm_100a tensor cores:
//
//   * up-projection of the cached latent to per-head keys and values for the training / prefill path:
//       k_nope [rows, H*128] = kv_latent [rows, 512] W_UK^T,   v [rows, H*128] = kv_latent W_UV^T
//     with W_UK, W_UV stored [H*128, 512];
//   * absorption for the decode path: W_UK folded into the query,
//       q_latent [rows, h, 512] = q_nope [rows, h, 128] W_UK[h]          (W_UK[h] is [128, 512])
//     and W_UV applied to the latent output,
//       out [rows, h, 128] = o_latent [rows, h, 512] W_UV[h]^T.
//
// All four are one kernel: a batched bf16 GEMM  C_b [M, N] = A_b [M, K] op(B_b)  with fp32 accumulation
// in tensor memory, where a batch entry (a head) is a column offset into A and C and a row offset into
// B, and op(B) is either B^T (B stored [N, K], K-major) or B itself (B stored [K, N], N contiguous: the
// MN-major operand form, no transpose pass).  The reference has none of these (its inputs are drawn
// already projected), so there is no reference kernel to cite.
//
// CTA tile 128 x 128, K in chunks of 64 through a ring of five 32 KB stages (TMA, 128-byte swizzle); the
// CTAs are persistent (one per SM) and walk the tiles with a stride; the accumulator is double-buffered
// in tensor memory (2 x 128 columns), so the MMA warp starts the next tile while the four epilogue warps
// convert the previous one to bf16 in shared memory (two 32 KB output buffers), from where one TMA store
// per 64 columns writes it: whole 128-byte lines, rows past M clipped by the TMA unit.  Warp 4 issues
// MMAs (whole warp, elected lane), warp 5 loads.  Every mbarrier wait is bounded.
#include "mla.h"
#include "cuda_common.h"
#include "attention_internal.h"
#include "sm100_primitives.cuh"
#include "../common/tensor_map.h"

#include <algorithm>
#include <cstdint>
#include <stdexcept>

namespace dscuda {
namespace {

using namespace sm100;

constexpr int TILE_M = 128;
constexpr int TILE_N = 128;
constexpr int TILE_K = 64;
constexpr int A_BYTES = TILE_M * 128;           // 16 KB: [128 rows x 64 bf16]
constexpr int B_BYTES = TILE_N * 128;           // 16 KB: [128 n x 64 k] (K-major) or two [64 k x 64 n] chunks (MN-major)
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGES = 5;
constexpr int OUT_BYTES = TILE_M * TILE_N * 2;   // 32 KB: two [128 rows x 64 bf16] swizzled chunks
constexpr int MISC_BYTES = 1024;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * OUT_BYTES + MISC_BYTES + 1024;
constexpr int THREADS = 192;
constexpr int MMA_WARP = 4;
constexpr int LOAD_WARP = 5;
constexpr int TMEM_COLUMNS = 256;               // two accumulators of 128 columns

__device__ int projection_status = 0;

struct GemmParams {
    CUtensorMap a;          // [M rows, all A columns] box 128 x 64
    CUtensorMap b;          // K-major: [all B rows, K] box 128 x 64; MN-major: [all B rows, N] box 64 x 64
    CUtensorMap c;          // [M rows, all C columns] box 128 x 64 (stores)
    int m, n, k;
    int batch;
    int a_batch_cols;       // batch entry b reads A columns [b * a_batch_cols, +K)
    int b_batch_rows;       // ... B rows from b * b_batch_rows
    int c_batch_cols;       // ... writes C columns [b * c_batch_cols, +N)
    int b_mn_major;         // 0: B is [N, K]; 1: B is [K, N]
};

struct Shared {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[2];       // tensor core -> epilogue
    uint64_t acc_empty[2];      // 128 epilogue threads -> tensor core
    uint64_t out_written[2];    // 128 epilogue threads: the tile is in the output buffer
    uint64_t out_free[2];       // the storing thread: the TMA store has read the buffer
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(Shared) <= MISC_BYTES, "barrier block too large");

__global__ void __launch_bounds__(THREADS, 1) projection_gemm_kernel(const __grid_constant__ GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    if (*reinterpret_cast<volatile int*>(&projection_status) == STATUS_WAIT_TIMEOUT) {
        return;
    }
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023U) & ~1023U;
    uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    Shared* sh = reinterpret_cast<Shared*>(smem_aligned + STAGES * STAGE_BYTES + 2 * OUT_BYTES);
    volatile int* abort_flag = &sh->abort_flag;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(smem_u32(&sh->full[i]), 1);
            mbar_init(smem_u32(&sh->empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&sh->acc_full[i]), 1);
            mbar_init(smem_u32(&sh->acc_empty[i]), TILE_M);
            mbar_init(smem_u32(&sh->out_written[i]), TILE_M);
            mbar_init(smem_u32(&sh->out_free[i]), 1);
        }
        sh->abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&sh->tmem_base), TMEM_COLUMNS);
        tmem_relinquish();
    }
    if (warp == LOAD_WARP && lane == 0) {
        tma_prefetch_descriptor(&p.a);
        tma_prefetch_descriptor(&p.b);
        tma_prefetch_descriptor(&p.c);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&sh->tmem_base);

    const int tiles_m = (p.m + TILE_M - 1) / TILE_M;
    const int tiles_n = p.n / TILE_N;
    const long long tiles = static_cast<long long>(tiles_m) * tiles_n * p.batch;
    const int k_chunks = p.k / TILE_K;
    // tile order: M fastest, so that CTAs running at the same time share the B tile (the weights) in L2
    auto locate = [&](long long tile, int& batch, int& tile_n, int& tile_m) {
        tile_m = static_cast<int>(tile % tiles_m);
        const long long rest = tile / tiles_m;
        tile_n = static_cast<int>(rest % tiles_n);
        batch = static_cast<int>(rest / tiles_n);
    };

    if (warp == LOAD_WARP) {
        if (lane == 0) {
            bool alive = true;
            long long chunk = 0;
            for (long long tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
                int batch, tile_n, tile_m;
                locate(tile, batch, tile_n, tile_m);
                for (int kc = 0; kc < k_chunks && alive; ++kc, ++chunk) {
                    const int stage = static_cast<int>(chunk % STAGES);
                    if (chunk >= STAGES) {
                        alive = mbar_wait(smem_u32(&sh->empty[stage]), static_cast<uint32_t>((chunk / STAGES - 1) & 1), abort_flag, &projection_status);
                        if (!alive) {
                            break;
                        }
                    }
                    const uint32_t bar = smem_u32(&sh->full[stage]);
                    const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
                    const uint32_t b_dst = a_dst + A_BYTES;
                    mbar_arrive_expect_tx(bar, STAGE_BYTES);
                    tma_load_2d(a_dst, &p.a, bar, batch * p.a_batch_cols + kc * TILE_K, tile_m * TILE_M);
                    if (p.b_mn_major == 0) {
                        tma_load_2d(b_dst, &p.b, bar, kc * TILE_K, batch * p.b_batch_rows + tile_n * TILE_N);
                    } else {
                        // two [64 k x 64 n] chunks side by side
                        tma_load_2d(b_dst, &p.b, bar, tile_n * TILE_N, batch * p.b_batch_rows + kc * TILE_K);
                        tma_load_2d(b_dst + B_BYTES / 2, &p.b, bar, tile_n * TILE_N + 64, batch * p.b_batch_rows + kc * TILE_K);
                    }
                }
            }
        }
    } else if (warp == MMA_WARP) {
        const uint32_t leader = elect_one();
        const uint32_t idesc = make_idesc_bf16(TILE_M, TILE_N, false, p.b_mn_major != 0);
        bool alive = true;
        long long chunk = 0;
        int local_tile = 0;
        for (long long tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x, ++local_tile) {
            const int buffer = local_tile & 1;
            if (local_tile >= 2) {
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->acc_empty[buffer]), static_cast<uint32_t>((local_tile / 2 - 1) & 1), abort_flag,
                                                          &projection_status));
                if (!alive) {
                    break;
                }
            }
            tc_fence_after_sync();
            const uint32_t acc = tmem_base + buffer * TILE_N;
            for (int kc = 0; kc < k_chunks && alive; ++kc, ++chunk) {
                const int stage = static_cast<int>(chunk % STAGES);
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->full[stage]), static_cast<uint32_t>((chunk / STAGES) & 1), abort_flag, &projection_status));
                if (!alive) {
                    break;
                }
                tc_fence_after_sync();
                const uint32_t a_smem = smem_base + stage * STAGE_BYTES;
                const uint32_t b_smem = a_smem + A_BYTES;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint64_t b_desc = p.b_mn_major == 0 ? make_kmajor_desc(b_smem + k * 32) : make_smem_desc(b_smem + k * 2048, B_BYTES / 2, 1024);
                    mma_ss_elect(acc, make_kmajor_desc(a_smem + k * 32), b_desc, idesc, (kc | k) != 0 ? 1U : 0U, leader);
                }
                mma_commit_elect(smem_u32(&sh->empty[stage]), leader);
            }
            if (alive) {
                mma_commit_elect(smem_u32(&sh->acc_full[buffer]), leader);
            }
        }
    } else {
        // =================== epilogue: thread = row of the tile ==================
        const int r = threadIdx.x;
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        bool alive = true;
        int local_tile = 0;
        for (long long tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x, ++local_tile) {
            int batch, tile_n, tile_m;
            locate(tile, batch, tile_n, tile_m);
            const int buffer = local_tile & 1;
            alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->acc_full[buffer]), static_cast<uint32_t>((local_tile / 2) & 1), abort_flag, &projection_status));
            if (!alive) {
                break;
            }
            tc_fence_after_sync();
            // the output buffer was last used two tiles ago; its store must have read it
            if (local_tile >= 2) {
                alive = __all_sync(0xffffffffU, mbar_wait(smem_u32(&sh->out_free[buffer]), static_cast<uint32_t>((local_tile / 2 - 1) & 1), abort_flag,
                                                          &projection_status));
                if (!alive) {
                    break;
                }
            }
            uint8_t* out_row = smem_aligned + STAGES * STAGE_BYTES + buffer * OUT_BYTES + r * 128;
#pragma unroll
            for (int c = 0; c < TILE_N / 32; ++c) {
                uint32_t values[32];
                tmem_ld_x32(tmem_base + lane_base + buffer * TILE_N + c * 32, values);
                tmem_wait_ld();
                // columns 32c..32c+31 = 16-byte units 4(c&1)..4(c&1)+3 of row r in chunk c/2, swizzled by the row
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    uint4 vec;
                    vec.x = pack_bf16x2(__uint_as_float(values[8 * u]), __uint_as_float(values[8 * u + 1]));
                    vec.y = pack_bf16x2(__uint_as_float(values[8 * u + 2]), __uint_as_float(values[8 * u + 3]));
                    vec.z = pack_bf16x2(__uint_as_float(values[8 * u + 4]), __uint_as_float(values[8 * u + 5]));
                    vec.w = pack_bf16x2(__uint_as_float(values[8 * u + 6]), __uint_as_float(values[8 * u + 7]));
                    const int unit = (c & 1) * 4 + u;
                    *reinterpret_cast<uint4*>(out_row + (c >> 1) * (OUT_BYTES / 2) + ((unit ^ (r & 7)) * 16)) = vec;
                }
            }
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&sh->acc_empty[buffer]));         // the accumulator is free as soon as it is in registers / shared memory
            fence_proxy_async_smem();
            mbar_arrive(smem_u32(&sh->out_written[buffer]));
            if (r == 0) {
                const bool written = mbar_wait(smem_u32(&sh->out_written[buffer]), static_cast<uint32_t>((local_tile / 2) & 1), abort_flag, &projection_status);
                if (written) {
                    const uint32_t src = smem_base + STAGES * STAGE_BYTES + buffer * OUT_BYTES;
                    const int x = batch * p.c_batch_cols + tile_n * TILE_N;
                    tma_store_2d(&p.c, src, x, tile_m * TILE_M);
                    tma_store_2d(&p.c, src + OUT_BYTES / 2, x + 64, tile_m * TILE_M);
                    tma_store_commit();
                    tma_store_wait_read();
                    mbar_arrive(smem_u32(&sh->out_free[buffer]));
                }
            }
        }
        if (r == 0) {
            tma_store_wait_all();       // the last stores have been written before the CTA exits
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

int sm_count() {
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

void configure_kernel() {
    static bool done[16] = {};
    int device = 0;
    CUDA_CHECK(cudaGetDevice(&device));
    if (device < 16 && done[device]) {
        return;
    }
    CUDA_CHECK(cudaFuncSetAttribute(projection_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    if (device < 16) {
        done[device] = true;
    }
}

// C_b [m, n] = A_b [m, k] op(B_b) for b in [0, batch): see GemmParams for the batch offsets.
void launch_gemm(__nv_bfloat16* c, const __nv_bfloat16* a, const __nv_bfloat16* b, long long m, int n, int k, long long a_cols, long long b_rows,
                 long long b_cols, long long ldc, int batch, int a_batch_cols, int b_batch_rows, int c_batch_cols, bool b_mn_major,
                 cudaStream_t stream) {
    if (m <= 0 || n <= 0 || k <= 0 || batch <= 0) {
        throw std::invalid_argument("MLA projection requires positive sizes");
    }
    if (n % TILE_N != 0 || k % TILE_K != 0) {
        throw std::invalid_argument("MLA projection requires N to be a multiple of 128 and K a multiple of 64");
    }
    if (m > 0x7fffffffLL) {
        throw std::invalid_argument("MLA projection shape exceeds the supported index range");
    }
    for (const void* pointer : {static_cast<const void*>(c), static_cast<const void*>(a), static_cast<const void*>(b)}) {
        if (pointer == nullptr) {
            throw std::invalid_argument("null tensor pointer");
        }
        if ((reinterpret_cast<std::uintptr_t>(pointer) & 15U) != 0) {
            throw std::invalid_argument("tensor pointers must be 16-byte aligned");
        }
    }
    GemmParams params{};
    params.a = make_bf16_tile_map(a, static_cast<std::uint64_t>(m), static_cast<std::uint64_t>(a_cols), static_cast<std::uint64_t>(a_cols), TILE_M);
    params.b = make_bf16_tile_map(b, static_cast<std::uint64_t>(b_rows), static_cast<std::uint64_t>(b_cols), static_cast<std::uint64_t>(b_cols),
                                  b_mn_major ? TILE_K : TILE_N);
    params.c = make_bf16_tile_map(c, static_cast<std::uint64_t>(m), static_cast<std::uint64_t>(ldc), static_cast<std::uint64_t>(ldc), TILE_M);
    params.m = static_cast<int>(m);
    params.n = n;
    params.k = k;
    params.batch = batch;
    params.a_batch_cols = a_batch_cols;
    params.b_batch_rows = b_batch_rows;
    params.c_batch_cols = c_batch_cols;
    params.b_mn_major = b_mn_major ? 1 : 0;
    configure_kernel();
    const long long tiles = ((m + TILE_M - 1) / TILE_M) * (n / TILE_N) * batch;
    const unsigned grid = static_cast<unsigned>(std::min<long long>(tiles, sm_count()));
    projection_gemm_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(params);
    CUDA_CHECK(cudaGetLastError());
}

void check_heads(long long rows, int heads) {
    if (rows <= 0 || heads <= 0) {
        throw std::invalid_argument("MLA projection requires positive rows and heads");
    }
    if (static_cast<long long>(heads) * MLA_KV_RANK > 0x7fffffffLL) {
        throw std::invalid_argument("MLA projection shape exceeds the supported index range");
    }
}

}  // namespace

namespace internal {

int projection_device_status(bool reset) {
    int status = 0;
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemcpyFromSymbol(&status, projection_status, sizeof(int)));
    if (reset && status != 0) {
        const int zero = 0;
        CUDA_CHECK(cudaMemcpyToSymbol(projection_status, &zero, sizeof(int)));
    }
    return status;
}

}  // namespace internal

void mla_up_project_cuda(__nv_bfloat16* k_nope, __nv_bfloat16* v, const __nv_bfloat16* kv_latent, const __nv_bfloat16* w_uk,
                         const __nv_bfloat16* w_uv, long long rows, int heads, cudaStream_t stream) {
    check_heads(rows, heads);
    const int n = heads * MLA_NOPE_SIZE;
    if (k_nope != nullptr) {
        launch_gemm(k_nope, kv_latent, w_uk, rows, n, MLA_KV_RANK, MLA_KV_RANK, n, MLA_KV_RANK, n, 1, 0, 0, 0, false, stream);
    }
    if (v != nullptr) {
        launch_gemm(v, kv_latent, w_uv, rows, n, MLA_KV_RANK, MLA_KV_RANK, n, MLA_KV_RANK, n, 1, 0, 0, 0, false, stream);
    }
    if (k_nope == nullptr && v == nullptr) {
        throw std::invalid_argument("MLA up-projection needs at least one output");
    }
}

void mla_absorb_query_cuda(__nv_bfloat16* q_latent, const __nv_bfloat16* q_nope, const __nv_bfloat16* w_uk, long long rows, int heads,
                           cudaStream_t stream) {
    check_heads(rows, heads);
    // per head: [rows, 128] x W_UK[h] ([128, 512], used as stored: K rows, N contiguous)
    launch_gemm(q_latent, q_nope, w_uk, rows, MLA_KV_RANK, MLA_NOPE_SIZE, static_cast<long long>(heads) * MLA_NOPE_SIZE,
                static_cast<long long>(heads) * MLA_NOPE_SIZE, MLA_KV_RANK, static_cast<long long>(heads) * MLA_KV_RANK, heads, MLA_NOPE_SIZE,
                MLA_NOPE_SIZE, MLA_KV_RANK, true, stream);
}

void mla_unabsorb_output_cuda(__nv_bfloat16* output, const __nv_bfloat16* output_latent, const __nv_bfloat16* w_uv, long long rows, int heads,
                              cudaStream_t stream) {
    check_heads(rows, heads);
    // per head: [rows, 512] x W_UV[h]^T (W_UV[h] is [128, 512]: N rows, K contiguous)
    launch_gemm(output, output_latent, w_uv, rows, MLA_VALUE_SIZE, MLA_KV_RANK, static_cast<long long>(heads) * MLA_KV_RANK,
                static_cast<long long>(heads) * MLA_VALUE_SIZE, MLA_KV_RANK, static_cast<long long>(heads) * MLA_VALUE_SIZE, heads, MLA_KV_RANK,
                MLA_VALUE_SIZE, MLA_VALUE_SIZE, false, stream);
}

}  // namespace dscuda
