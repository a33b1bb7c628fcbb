// Causal D=128 grouped-query attention forward.  Drop-in for the reference's
// include/flash_attention.h:12-24 (same name, arguments and layouts).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace dscuda {

// Q/O are BF16 [B,T,Hq,128], K/V are BF16 [B,T,Hkv,128], the natural-log LSE is
// FP32 [B,Hq,T].  Hq must be divisible by Hkv and head_size must be 128.  The
// reference demands T % 64 == 0 (kernels/attention/flash_attention/
// sm89_forward.cu:226-228); this implementation accepts any T >= 1.
// Launch-only on `stream`: no allocation, no synchronisation, capturable in a
// CUDA graph.  Throws std::invalid_argument / std::runtime_error.
void flash_attention_forward_cuda(
    __nv_bfloat16* output,
    float* logsumexp,
    const __nv_bfloat16* query,
    const __nv_bfloat16* key,
    const __nv_bfloat16* value,
    int batch_size,
    int sequence_length,
    int query_heads,
    int key_value_heads,
    int head_size,
    float scale,
    cudaStream_t stream = nullptr);

}  // namespace dscuda
