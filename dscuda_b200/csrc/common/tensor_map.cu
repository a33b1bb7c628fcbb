#include "tensor_map.h"

#include "cuda_common.h"

#include <cudaTypedefs.h>

#include <mutex>
#include <stdexcept>
#include <string>

namespace dscuda {
namespace {

PFN_cuTensorMapEncodeTiled_v12000 encode_entry_point() {
    static PFN_cuTensorMapEncodeTiled_v12000 function = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* pointer = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &pointer, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess) {
            function = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(pointer);
        }
    });
    if (function == nullptr) {
        throw std::runtime_error("cuTensorMapEncodeTiled is not available from this driver");
    }
    return function;
}

}  // namespace

CUtensorMap make_bf16_tile_map(const void* base, std::uint64_t rows, std::uint64_t cols, std::uint64_t row_stride_elements,
                               std::uint32_t box_rows) {
    if ((reinterpret_cast<std::uintptr_t>(base) & 15U) != 0 || (row_stride_elements * 2) % 16 != 0) {
        throw std::invalid_argument("tensor base and row stride must be 16-byte aligned");
    }
    if (rows == 0 || cols == 0 || box_rows == 0 || box_rows > 256) {
        throw std::invalid_argument("empty tensor or bad tile height");
    }
    CUtensorMap map;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {row_stride_elements * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t element_strides[2] = {1, 1};
    const CUresult result = encode_entry_point()(
        &map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, element_strides,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (result != CUDA_SUCCESS) {
        throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(result)));
    }
    return map;
}

CUtensorMap make_bf16_chunked_map(const void* base, std::uint64_t rows, std::uint32_t chunks, std::uint64_t row_stride_elements,
                                  std::uint32_t box_rows, std::uint32_t box_chunks) {
    if ((reinterpret_cast<std::uintptr_t>(base) & 15U) != 0 || (row_stride_elements * 2) % 16 != 0) {
        throw std::invalid_argument("tensor base and row stride must be 16-byte aligned");
    }
    if (rows == 0 || chunks == 0 || box_rows == 0 || box_rows > 256 || box_chunks == 0 || box_chunks > chunks) {
        throw std::invalid_argument("empty tensor or bad tile shape");
    }
    CUtensorMap map;
    const cuuint64_t dims[3] = {64, rows, chunks};
    const cuuint64_t strides[2] = {row_stride_elements * 2, 128};
    const cuuint32_t box[3] = {64, box_rows, box_chunks};
    const cuuint32_t element_strides[3] = {1, 1, 1};
    const CUresult result = encode_entry_point()(
        &map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, element_strides,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (result != CUDA_SUCCESS) {
        throw std::runtime_error("cuTensorMapEncodeTiled (chunked view) failed with code " + std::to_string(static_cast<int>(result)));
    }
    return map;
}

CUtensorMap make_u64_rows_map(const void* base, std::uint64_t rows, std::uint32_t row_words, std::uint32_t box_words, std::uint32_t box_rows) {
    if ((reinterpret_cast<std::uintptr_t>(base) & 15U) != 0 || (row_words * 8) % 16 != 0 || (box_words * 8) % 16 != 0) {
        throw std::invalid_argument("tensor base, row length and box width must be multiples of 16 bytes");
    }
    if (rows == 0 || row_words == 0 || box_words == 0 || box_words > 256 || box_rows == 0 || box_rows > 256) {
        throw std::invalid_argument("empty tensor or bad box");
    }
    CUtensorMap map;
    const cuuint64_t dims[2] = {row_words, rows};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_words) * 8};
    const cuuint32_t box[2] = {box_words, box_rows};
    const cuuint32_t element_strides[2] = {1, 1};
    const CUresult result = encode_entry_point()(&map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(base), dims, strides, box, element_strides,
                                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (result != CUDA_SUCCESS) {
        throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(result)));
    }
    return map;
}

}  // namespace dscuda
