// Declarations shared between the attention translation units and the C-ABI
// bridges; not part of the public headers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstddef>

namespace dscuda {
namespace internal {

// Throws std::invalid_argument unless the arguments describe a supported
// non-absorbed prefill problem (128/64/128 head sizes, positive sizes and scale,
// index ranges that fit the kernels).
void check_prefill_shape(const int* cu_seqlens, int batch_size, int max_sequence_length, int total_tokens, int heads,
                         int nope_size, int rope_size, int value_size, float scale);

void launch_prefill_forward(__nv_bfloat16* output, float* logsumexp, const __nv_bfloat16* q_nope, const __nv_bfloat16* q_pe,
                            const __nv_bfloat16* k_nope, const __nv_bfloat16* k_pe, const __nv_bfloat16* v, const int* cu_seqlens,
                            int batch_size, int max_sequence_length, int total_tokens, int heads, float scale,
                            cudaStream_t stream);

// Per-translation-unit sticky status words (0 = fine).  Reading synchronises.
int forward_device_status(bool reset);
int absorbed_backward_device_status(bool reset);
int decode_device_status(bool reset);
int projection_device_status(bool reset);
int backward_device_status(bool reset);
int append_device_status(bool reset);

}  // namespace internal
}  // namespace dscuda
