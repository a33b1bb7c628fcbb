// Rotary position embedding of the 64 rotary columns, in place, for the tensors
// the attention kernels take (q_pe [rows, H, 64], k_pe [rows, 1, 64], bf16).
//
// Rotate-half pairing: element i (0 <= i < 32) is paired with element i + 32,
// angle = position * theta^(-2i/64):
//     out[i]      = x[i] * cos - x[i+32] * sin
//     out[i + 32] = x[i] * sin + x[i+32] * cos
// The angle, its cosine and sine are computed in double precision once per row
// (they are shared by all heads) and rounded to fp32; the two products and the
// sum are separate fp32 operations, not fused, so the result is the same as the
// same expression evaluated with fp32 tensors on the host.
//
// One warp per row; a lane owns two neighbouring frequencies, sixteen lanes
// cover one head, so a warp instruction moves two heads (2 x 64 bytes per
// half).  The kernel is bound by HBM: every element is read once and written
// once.
#include "mla.h"
#include "cuda_common.h"

#include <cstdint>
#include <stdexcept>

namespace dscuda {
namespace {

constexpr int ROPE_THREADS = 256;

__device__ __forceinline__ float2 unpack(uint32_t v) {
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000U));
}

__device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&pair);
}

__device__ __forceinline__ void rotate(uint32_t* row, int slot, float c0, float s0, float c1, float s1) {
    // row points at 64 bf16 = 32 words; words 0..15 are the first halves, 16..31 the second
    const float2 a = unpack(row[slot]);
    const float2 b = unpack(row[16 + slot]);
    const float lo0 = __fsub_rn(__fmul_rn(a.x, c0), __fmul_rn(b.x, s0));
    const float lo1 = __fsub_rn(__fmul_rn(a.y, c1), __fmul_rn(b.y, s1));
    const float hi0 = __fadd_rn(__fmul_rn(a.x, s0), __fmul_rn(b.x, c0));
    const float hi1 = __fadd_rn(__fmul_rn(a.y, s1), __fmul_rn(b.y, c1));
    row[slot] = pack(lo0, lo1);
    row[16 + slot] = pack(hi0, hi1);
}

__global__ void __launch_bounds__(ROPE_THREADS) rope_apply_kernel(uint32_t* q_pe, uint32_t* k_pe, const int* positions, long long rows, int heads,
                                                                  int sequence_length, double log2_theta) {
    const int lane = threadIdx.x % 32;
    const int slot = lane % 16;                    // frequencies 2*slot and 2*slot + 1
    const int side = lane / 16;                    // which of two heads handled together
    const long long warps = static_cast<long long>(gridDim.x) * (ROPE_THREADS / 32);
    const double inv0 = exp2(-log2_theta * (2.0 * (2 * slot)) / 64.0);
    const double inv1 = exp2(-log2_theta * (2.0 * (2 * slot + 1)) / 64.0);
    for (long long row = static_cast<long long>(blockIdx.x) * (ROPE_THREADS / 32) + threadIdx.x / 32; row < rows; row += warps) {
        const int position = positions != nullptr ? positions[row] : static_cast<int>(row % sequence_length);
        double s0d, c0d, s1d, c1d;
        sincos(static_cast<double>(position) * inv0, &s0d, &c0d);
        sincos(static_cast<double>(position) * inv1, &s1d, &c1d);
        const float c0 = static_cast<float>(c0d), s0 = static_cast<float>(s0d), c1 = static_cast<float>(c1d), s1 = static_cast<float>(s1d);
        if (q_pe != nullptr) {
            uint32_t* base = q_pe + row * heads * 32;
            // four head pairs per pass, all loads before the first store, to keep more bytes in flight
            int h = side;
            for (; h + 6 < heads; h += 8) {
                uint32_t a[4], b[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    a[u] = base[(h + 2 * u) * 32 + slot];
                    b[u] = base[(h + 2 * u) * 32 + 16 + slot];
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float2 x = unpack(a[u]);
                    const float2 y = unpack(b[u]);
                    base[(h + 2 * u) * 32 + slot] = pack(__fsub_rn(__fmul_rn(x.x, c0), __fmul_rn(y.x, s0)), __fsub_rn(__fmul_rn(x.y, c1), __fmul_rn(y.y, s1)));
                    base[(h + 2 * u) * 32 + 16 + slot] =
                        pack(__fadd_rn(__fmul_rn(x.x, s0), __fmul_rn(y.x, c0)), __fadd_rn(__fmul_rn(x.y, s1), __fmul_rn(y.y, c1)));
                }
            }
            for (; h < heads; h += 2) {
                rotate(base + h * 32, slot, c0, s0, c1, s1);
            }
        }
        if (k_pe != nullptr && side == 0) {
            rotate(k_pe + row * 32, slot, c0, s0, c1, s1);
        }
    }
}

}  // namespace

void mla_rope_apply_cuda(__nv_bfloat16* q_pe, __nv_bfloat16* k_pe, const int* positions, long long rows, int heads, int sequence_length,
                         int rope_size, float theta, cudaStream_t stream) {
    if (rope_size != MLA_ROPE_SIZE) {
        throw std::invalid_argument("MLA requires RoPE size 64");
    }
    if (rows <= 0 || heads <= 0 || !(theta > 1.0F)) {
        throw std::invalid_argument("RoPE requires positive rows and heads and theta > 1");
    }
    if (positions == nullptr && sequence_length <= 0) {
        throw std::invalid_argument("RoPE needs explicit positions or a positive sequence length");
    }
    if (q_pe == nullptr && k_pe == nullptr) {
        throw std::invalid_argument("null tensor pointer");
    }
    for (const void* pointer : {static_cast<const void*>(q_pe), static_cast<const void*>(k_pe)}) {
        if ((reinterpret_cast<std::uintptr_t>(pointer) & 15U) != 0) {
            throw std::invalid_argument("tensor pointers must be 16-byte aligned");
        }
    }
    const long long wanted = (rows + ROPE_THREADS / 32 - 1) / (ROPE_THREADS / 32);
    const unsigned blocks = static_cast<unsigned>(wanted < 148LL * 8 ? wanted : 148LL * 8);      // 8 resident CTAs on each of 148 SMs
    rope_apply_kernel<<<blocks, ROPE_THREADS, 0, stream>>>(reinterpret_cast<uint32_t*>(q_pe), reinterpret_cast<uint32_t*>(k_pe), positions, rows, heads,
                                                           sequence_length, log2(static_cast<double>(theta)));
    CUDA_CHECK(cudaGetLastError());
}

}  // namespace dscuda
