// Probe: how fast can every SM add fp32 tiles into one global accumulator?
//
// A fused single-pass backward (one key-stationary kernel that also produces dQ) has to add a
// [query rows x 192] fp32 partial of dQ into a [rows, heads, 192] accumulator for every key tile it
// visits.  This program measures that reduction alone: every CTA adds 64 x 192 fp32 tiles (48 KB) to
// the rows it walks, with the three instructions that can do it (red.global.add.v4.f32 from registers,
// the 1-D bulk reduce and the 2-D tensor reduce from shared memory), for accumulators that stay in L2
// (2 or 4 heads active at a time) and for accumulators that do not (37 or 148 heads).  It prints
// TB/s of added data; nothing else of the backward runs, so the figures are upper bounds.
//
//     build/probe_dq_reduction
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <vector>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("err %s line %d\n", cudaGetErrorString(e), __LINE__); exit(1);} } while (0)

constexpr int ROWS_PER_TILE = 64;
constexpr int COLS = 192;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// mode 0: red.v4 from registers; mode 1: bulk reduce per row (768 B); mode 2: tensor reduce (one op per tile)
template <int MODE>
__global__ void __launch_bounds__(128) red_kernel(float* acc, const __grid_constant__ CUtensorMap map, int rows, int heads, int heads_active, int iters) {
    extern __shared__ __align__(1024) unsigned char smem[];
    float* tile = reinterpret_cast<float*>(smem);
    for (int i = threadIdx.x; i < ROWS_PER_TILE * COLS; i += 128) tile[i] = 1.0f;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    const int per_head = gridDim.x / heads_active;
    const int head = (blockIdx.x / per_head) % heads;
    const int tiles = rows / ROWS_PER_TILE;
    int t = (blockIdx.x % per_head) * (tiles / per_head);
    for (int it = 0; it < iters; ++it) {
        const int row0 = (t % tiles) * ROWS_PER_TILE;
        if (MODE == 0) {
            // thread = (row pair), 48 float4 per row: 64 rows * 48 = 3072 float4 / 128 threads = 24 each
            for (int j = threadIdx.x; j < ROWS_PER_TILE * 48; j += 128) {
                const int r = j / 48, c = j % 48;
                float* dst = acc + (static_cast<size_t>(row0 + r) * heads + head) * COLS + c * 4;
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(1.0f), "f"(1.0f), "f"(1.0f), "f"(1.0f) : "memory");
            }
        } else if (MODE == 1) {
            if (threadIdx.x < ROWS_PER_TILE) {
                const int r = threadIdx.x;
                float* dst = acc + (static_cast<size_t>(row0 + r) * heads + head) * COLS;
                asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(tile + r * COLS)), "r"(COLS * 4) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory");
            }
        } else {
            if (threadIdx.x == 0) {
                asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(&map), "r"(smem_u32(tile)), "r"(head * COLS), "r"(row0) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory");
            }
        }
        ++t;
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

int main(int argc, char** argv) {
    const int rows = 8192;
    const int heads = 160;
    float* acc;
    const size_t bytes = static_cast<size_t>(rows) * heads * COLS * 4;
    CK(cudaMalloc(&acc, bytes));
    CK(cudaMemset(acc, 0, bytes));
    CUtensorMap map;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(heads) * COLS, static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(heads) * COLS * 4};
    cuuint32_t box[2] = {COLS, ROWS_PER_TILE};
    cuuint32_t estr[2] = {1, 1};
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    auto encode = reinterpret_cast<CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill)>(fn);
    CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, acc, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { printf("encode failed %d\n", (int)r); return 1; }
    const int smem = ROWS_PER_TILE * COLS * 4;
    CK(cudaFuncSetAttribute(red_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    CK(cudaFuncSetAttribute(red_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    CK(cudaFuncSetAttribute(red_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaEvent_t a, b;
    CK(cudaEventCreate(&a)); CK(cudaEventCreate(&b));
    const int iters = 256;
    const int grids[2] = {148, 296};
    for (int g = 0; g < 2; ++g)
    for (int mode = 0; mode < 3; ++mode) {
        for (int heads_active : {2, 4, 37, 148}) {
            const int grid = grids[g];
            float best = 1e9f;
            for (int rep = 0; rep < 4; ++rep) {
                CK(cudaEventRecord(a));
                if (mode == 0) red_kernel<0><<<grid, 128, smem>>>(acc, map, rows, heads, heads_active, iters);
                if (mode == 1) red_kernel<1><<<grid, 128, smem>>>(acc, map, rows, heads, heads_active, iters);
                if (mode == 2) red_kernel<2><<<grid, 128, smem>>>(acc, map, rows, heads, heads_active, iters);
                CK(cudaEventRecord(b));
                CK(cudaEventSynchronize(b));
                float ms; CK(cudaEventElapsedTime(&ms, a, b));
                if (rep > 0 && ms < best) best = ms;
            }
            CK(cudaGetLastError());
            const double moved = static_cast<double>(grid) * iters * ROWS_PER_TILE * COLS * 4;
            printf("grid %3d mode %d heads_active %3d : %.3f ms  %.2f TB/s  (%.1f B/clk/SM at 1.9 GHz)\n", grid, mode, heads_active, best, moved / best / 1e9,
                   moved / best / 1e-3 / 148 / 1.9e9);
        }
    }
    // check: total adds
    std::vector<float> host(1024);
    CK(cudaMemcpy(host.data(), acc, 4096, cudaMemcpyDeviceToHost));
    printf("acc[0]=%f\n", host[0]);
    return 0;
}
