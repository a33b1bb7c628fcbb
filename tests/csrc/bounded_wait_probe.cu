// Test-only library (never linked into the product libraries): one small kernel that
// uses the product's own bounded mbarrier wait on a barrier nobody arrives on, with a
// short limit, so that the give-up path can be exercised without any fault: the wait
// returns false, the status word becomes 1, the CTA tears down the way the attention
// kernels do (tensor memory released), and a launch made while the status is set
// leaves at once.  Nothing here traps, spins without a limit or touches bad memory.
#include "sm100_primitives.cuh"

#include <cuda_runtime.h>

namespace {

using namespace dscuda::sm100;

__device__ int probe_status = 0;

// result[0]: 1 when the wait gave up, 0 when it completed; result[1]: 1 when the launch
// left at entry because the status word was already set; result[2]: tensor-memory
// columns the launch allocated and released.
__global__ void __launch_bounds__(64, 1) bounded_wait_probe_kernel(long long limit_cycles, int arrive, int* result) {
    __shared__ uint64_t barrier;
    __shared__ uint32_t tmem_base;
    __shared__ int abort_flag;
    if (*reinterpret_cast<volatile int*>(&probe_status) == STATUS_WAIT_TIMEOUT) {
        if (threadIdx.x == 0) {
            result[1] = 1;
        }
        return;
    }
    const int warp = threadIdx.x / 32;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&barrier), 1);
        abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_base), 32);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == 0 && threadIdx.x == 0 && arrive != 0) {
        mbar_arrive(smem_u32(&barrier));
    }
    bool completed = true;
    if (warp == 1) {
        // the whole warp waits, as the MMA-issue warps of the attention kernels do
        completed = __all_sync(0xffffffffU, mbar_wait_limit(smem_u32(&barrier), 0, &abort_flag, &probe_status, limit_cycles));
        if (threadIdx.x == 32) {
            result[0] = completed ? 0 : 1;
        }
    }
    // teardown, as in the attention kernels
    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (*reinterpret_cast<volatile int*>(&abort_flag) != 0) {
        for (int k = 0; k < 64; ++k) {
            __nanosleep(1000);
        }
    }
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(*reinterpret_cast<volatile uint32_t*>(&tmem_base), 32);
        if (threadIdx.x == 0) {
            result[2] = 32;
        }
    }
}

}  // namespace

// Runs the probe once and waits for it.  `out` (host, 4 ints) receives result[0..2] and the
// status word after the launch.  Returns a cudaError_t value (0 = success).
extern "C" int dscuda_test_bounded_wait(long long limit_cycles, int arrive, int reset_status_first, int* out) {
    int* device_result = nullptr;
    cudaError_t error = cudaMalloc(&device_result, 3 * sizeof(int));
    if (error != cudaSuccess) {
        return static_cast<int>(error);
    }
    const int zero = 0;
    if (reset_status_first != 0) {
        error = cudaMemcpyToSymbol(probe_status, &zero, sizeof(int));
    }
    if (error == cudaSuccess) {
        error = cudaMemset(device_result, 0, 3 * sizeof(int));
    }
    if (error == cudaSuccess) {
        bounded_wait_probe_kernel<<<1, 64>>>(limit_cycles, arrive, device_result);
        error = cudaGetLastError();
    }
    if (error == cudaSuccess) {
        error = cudaDeviceSynchronize();
    }
    if (error == cudaSuccess) {
        error = cudaMemcpy(out, device_result, 3 * sizeof(int), cudaMemcpyDeviceToHost);
    }
    if (error == cudaSuccess) {
        error = cudaMemcpyFromSymbol(out + 3, probe_status, sizeof(int));
    }
    cudaFree(device_result);
    return static_cast<int>(error);
}
