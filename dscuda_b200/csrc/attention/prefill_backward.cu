// Placeholder translation unit, replaced by the real backward kernels.
#include "mla.h"
#include "attention_internal.h"

#include <stdexcept>

namespace dscuda {
namespace internal {
int backward_device_status(bool) { return 0; }
}  // namespace internal

std::size_t mla_prefill_backward_workspace_bytes(int, int, int total_tokens, int) {
    return static_cast<std::size_t>(total_tokens) * 64 * sizeof(float);
}

void mla_prefill_backward_cuda(__nv_bfloat16*, __nv_bfloat16*, __nv_bfloat16*, __nv_bfloat16*, const __nv_bfloat16*,
                               const __nv_bfloat16*, const float*, const __nv_bfloat16*, const __nv_bfloat16*, const __nv_bfloat16*,
                               const __nv_bfloat16*, const __nv_bfloat16*, const int*, void*, int, int, int, int, int, int, int, float,
                               cudaStream_t) {
    throw std::runtime_error("mla_prefill_backward_cuda: not built yet");
}

void mla_compressed_attention_backward_cuda(__nv_bfloat16*, __nv_bfloat16*, __nv_bfloat16*, __nv_bfloat16*, const __nv_bfloat16*,
                                            const __nv_bfloat16*, const float*, const __nv_bfloat16*, const __nv_bfloat16*,
                                            const __nv_bfloat16*, const __nv_bfloat16*, int, int, int, int, int, float, cudaStream_t) {
    throw std::runtime_error("mla_compressed_attention_backward_cuda: not built yet");
}
}  // namespace dscuda
