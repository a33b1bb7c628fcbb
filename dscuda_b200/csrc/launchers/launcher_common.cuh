// Shared pieces of the stand-alone C++ launchers: device buffers that free themselves, a seeded
// pseudo-random fill (the profiled kernels should not see constant data), argument parsing.
#pragma once

#include "cuda_common.h"

#include <cuda_bf16.h>
#include <cuda_profiler_api.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <cstdlib>

namespace launcher {

template <class T>
class DeviceBuffer {
public:
    explicit DeviceBuffer(std::size_t elements) : elements_(elements) {
        CUDA_CHECK(cudaMalloc(&pointer_, (elements > 0 ? elements : 1) * sizeof(T)));
    }
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    ~DeviceBuffer() { cudaFree(pointer_); }
    T* get() const { return static_cast<T*>(pointer_); }
    std::size_t size() const { return elements_; }

private:
    void* pointer_ = nullptr;
    std::size_t elements_;
};

__device__ __forceinline__ float hashed_unit(std::uint64_t index, std::uint32_t seed) {
    std::uint64_t x = index * 0x9E3779B97F4A7C15ULL + seed;
    x ^= x >> 31;
    x *= 0xBF58476D1CE4E5B9ULL;
    x ^= x >> 29;
    return static_cast<float>(static_cast<std::uint32_t>(x >> 40)) * (2.0F / 16777216.0F) - 1.0F;     // [-1, 1)
}

// Sum of three uniforms: bell-shaped, variance 1 after scaling by `sigma`.
__global__ void fill_bf16_kernel(__nv_bfloat16* data, std::size_t elements, std::uint32_t seed, float sigma) {
    const std::size_t stride = static_cast<std::size_t>(gridDim.x) * blockDim.x;
    for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < elements; i += stride) {
        const float value = hashed_unit(3 * i, seed) + hashed_unit(3 * i + 1, seed) + hashed_unit(3 * i + 2, seed);
        data[i] = __float2bfloat16(value * sigma);
    }
}

inline void fill(DeviceBuffer<__nv_bfloat16>& buffer, std::uint32_t seed, float sigma) {
    fill_bf16_kernel<<<148 * 8, 256>>>(buffer.get(), buffer.size(), seed, sigma);
    CUDA_CHECK(cudaGetLastError());
}

inline int argument(int argc, char** argv, int index, int fallback) {
    return argc > index ? std::atoi(argv[index]) : fallback;
}

}  // namespace launcher
