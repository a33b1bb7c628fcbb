// Test infrastructure: stands in for the reference's sm_90 flash-attention path when its sm_89 path is built
// for sm_100a as a checker (oracle/build_reference_cuda.py).  The reference's dispatcher
// (kernels/attention/flash_attention/dispatch.cu:17-27) only takes this branch on compute capability 9.x, and
// the sm_90 source uses wgmma, which does not exist on sm_100a; the symbol is needed to link, never to run.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <stdexcept>

namespace dscuda {

void flash_attention_forward_sm90_cuda(__nv_bfloat16*, float*, const __nv_bfloat16*, const __nv_bfloat16*, const __nv_bfloat16*, int, int, int, int, int,
                                       float, cudaStream_t) {
    throw std::runtime_error("the sm_90 flash attention path is not part of this checker build");
}

}  // namespace dscuda
