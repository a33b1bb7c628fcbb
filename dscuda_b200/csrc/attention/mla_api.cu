// Argument validation shared by the MLA entry points, and the device status
// accessor.  Validation happens on the host before any launch, so a rejected
// call leaves the stream untouched (the reference rejects C != 512 or R != 64
// the same way, kernels/attention/mla/sm89.cu:20-24).
#include "mla.h"
#include "attention_internal.h"

#include <stdexcept>

namespace dscuda {
namespace internal {

void check_prefill_shape(const int* cu_seqlens, int batch_size, int max_sequence_length, int total_tokens, int heads,
                         int nope_size, int rope_size, int value_size, float scale) {
    if (nope_size != MLA_NOPE_SIZE || rope_size != MLA_ROPE_SIZE || value_size != MLA_VALUE_SIZE) {
        throw std::invalid_argument("MLA prefill requires nope=128, RoPE=64 and value=128");
    }
    if (batch_size <= 0 || max_sequence_length <= 0 || total_tokens <= 0 || heads <= 0) {
        throw std::invalid_argument("MLA prefill requires positive batch, sequence length, token count and heads");
    }
    if (!(scale > 0.0F)) {
        throw std::invalid_argument("MLA prefill requires a positive softmax scale");
    }
    if (heads > 65535 || batch_size > 65535) {
        throw std::invalid_argument("MLA prefill supports at most 65535 heads and 65535 sequences");
    }
    if (cu_seqlens == nullptr &&
        static_cast<long long>(batch_size) * max_sequence_length != static_cast<long long>(total_tokens)) {
        throw std::invalid_argument("dense MLA prefill requires total_tokens == batch_size * max_sequence_length");
    }
    if (cu_seqlens != nullptr && max_sequence_length > total_tokens) {
        throw std::invalid_argument("packed MLA prefill requires max_sequence_length <= total_tokens");
    }
}

}  // namespace internal

int mla_device_status(bool reset) {
    const int forward = internal::forward_device_status(reset);
    const int absorbed_backward = internal::absorbed_backward_device_status(reset);
    const int decode = internal::decode_device_status(reset);
    const int projection = internal::projection_device_status(reset);
    const int backward = internal::backward_device_status(reset);
    const int append = internal::append_device_status(reset);
    for (const int status : {forward, decode, absorbed_backward, backward, projection}) {
        if (status != 0) {
            return status;
        }
    }
    return append;
}

}  // namespace dscuda
