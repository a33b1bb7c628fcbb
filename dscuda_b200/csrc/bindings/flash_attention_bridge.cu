// extern "C" surface of libdscuda_flash_attention_bench.so; same symbols as the
// reference's benchmarks/bindings/flash_attention_bridge.cu:13-30.
#include "flash_attention.h"
#include "../attention/attention_internal.h"

#include <exception>
#include <string>

namespace {
thread_local std::string last_error;
}

extern "C" const char* dscuda_flash_last_error() {
    return last_error.c_str();
}

extern "C" int dscuda_flash_forward(__nv_bfloat16* output, float* logsumexp, const __nv_bfloat16* query, const __nv_bfloat16* key,
                                    const __nv_bfloat16* value, int batch, int sequence, int query_heads, int key_value_heads,
                                    int dimension, float scale, cudaStream_t stream) {
    try {
        dscuda::flash_attention_forward_cuda(output, logsumexp, query, key, value, batch, sequence, query_heads, key_value_heads,
                                             dimension, scale, stream);
        return 0;
    } catch (const std::exception& error) {
        last_error = error.what();
        return 1;
    }
}

extern "C" int dscuda_flash_device_status(int reset) {
    try {
        return dscuda::internal::forward_device_status(reset != 0);
    } catch (const std::exception& error) {
        last_error = error.what();
        return -1;
    }
}
