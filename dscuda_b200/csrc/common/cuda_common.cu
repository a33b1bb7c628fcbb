// CUDA error-to-exception conversion and the small allocation helpers the C++
// callers of the host API use.  Mirrors the behaviour of the reference's
// kernels/common/cuda_common.cu:24-67: a failed call throws std::runtime_error
// carrying the expression and location.
#include "cuda_common.h"

#include <cstdio>
#include <stdexcept>
#include <string>

namespace dscuda {
namespace {

__global__ void cast_fp32_to_bf16_kernel(__nv_bfloat16* output, const float* input, std::size_t elements) {
    const std::size_t stride = static_cast<std::size_t>(gridDim.x) * blockDim.x;
    for (std::size_t index = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x; index < elements; index += stride) {
        output[index] = __float2bfloat16(input[index]);
    }
}

}  // namespace

void cuda_check(cudaError_t result, const char* expression, const char* file, int line) {
    if (result != cudaSuccess) {
        throw std::runtime_error(std::string("CUDA failure at ") + file + ":" + std::to_string(line) + " while evaluating " +
                                 expression + ": " + cudaGetErrorString(result));
    }
}

void* device_malloc(std::size_t bytes) {
    void* pointer = nullptr;
    CUDA_CHECK(cudaMalloc(&pointer, bytes));
    return pointer;
}

void device_free(void* pointer) {
    CUDA_CHECK(cudaFree(pointer));
}

void synchronize(cudaStream_t stream) {
    CUDA_CHECK(cudaStreamSynchronize(stream));
}

cudaDeviceProp device_properties(int device) {
    cudaDeviceProp properties{};
    CUDA_CHECK(cudaGetDeviceProperties(&properties, device));
    return properties;
}

void print_device_summary(int device) {
    const cudaDeviceProp properties = device_properties(device);
    std::printf("CUDA device %d: %s, sm_%d%d, %d SMs, %.1f GiB\n", device, properties.name, properties.major, properties.minor,
                properties.multiProcessorCount, static_cast<double>(properties.totalGlobalMem) / (1024.0 * 1024.0 * 1024.0));
}

void convert_fp32_to_bf16_cuda(__nv_bfloat16* output, const float* input, std::size_t elements, cudaStream_t stream) {
    if (elements == 0) {
        return;
    }
    const std::size_t wanted = (elements + 255) / 256;
    const int blocks = static_cast<int>(wanted < 148 * 16 ? wanted : 148 * 16);
    cast_fp32_to_bf16_kernel<<<blocks, 256, 0, stream>>>(output, input, elements);
    CUDA_CHECK(cudaGetLastError());
}

}  // namespace dscuda
