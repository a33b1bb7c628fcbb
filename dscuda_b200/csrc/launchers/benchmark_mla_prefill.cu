// benchmark_mla_prefill [batch=1] [sequence=4096] [heads=32] [backward=1]
//
// Non-absorbed causal forward (and backward) of the training path, dense layout, once untimed and
// once between cudaProfilerStart/Stop.  The reference has no launcher for this path (it has no
// such kernels); this one follows the pattern of its benchmark_mla.cu.
#include "launcher_common.cuh"
#include "mla.h"

#include <cmath>
#include <cstdio>
#include <exception>

int main(int argc, char** argv) {
    try {
        using launcher::DeviceBuffer;
        const int batch = launcher::argument(argc, argv, 1, 1);
        const int sequence = launcher::argument(argc, argv, 2, 4096);
        const int heads = launcher::argument(argc, argv, 3, 32);
        const bool backward = launcher::argument(argc, argv, 4, 1) != 0;
        const float scale = 1.0F / std::sqrt(192.0F);
        const int total = batch * sequence;
        const std::size_t rows = static_cast<std::size_t>(total) * heads;
        DeviceBuffer<__nv_bfloat16> q_nope(rows * 128), q_pe(rows * 64), k_nope(rows * 128), k_pe(static_cast<std::size_t>(total) * 64), v(rows * 128);
        DeviceBuffer<__nv_bfloat16> output(rows * 128), dout(rows * 128);
        DeviceBuffer<__nv_bfloat16> dq(rows * 192), dk_nope(rows * 128), dk_pe(static_cast<std::size_t>(total) * 64), dv(rows * 128);
        DeviceBuffer<float> lse(rows);
        DeviceBuffer<unsigned char> workspace(dscuda::mla_prefill_backward_workspace_bytes(batch, sequence, total, heads));
        launcher::fill(q_nope, 1, 1.0F);
        launcher::fill(q_pe, 2, 1.0F);
        launcher::fill(k_nope, 3, 1.0F);
        launcher::fill(k_pe, 4, 1.0F);
        launcher::fill(v, 5, 1.0F);
        launcher::fill(dout, 6, 0.1F);
        auto run = [&]() {
            dscuda::mla_prefill_forward_cuda(output.get(), lse.get(), q_nope.get(), q_pe.get(), k_nope.get(), k_pe.get(), v.get(), nullptr, batch,
                                             sequence, total, heads, 128, 64, 128, scale);
            if (backward) {
                dscuda::mla_prefill_backward_cuda(dq.get(), dk_nope.get(), dk_pe.get(), dv.get(), dout.get(), output.get(), lse.get(), q_nope.get(),
                                                  q_pe.get(), k_nope.get(), k_pe.get(), v.get(), nullptr, workspace.get(), batch, sequence, total,
                                                  heads, 128, 64, 128, scale);
            }
        };
        run();
        dscuda::synchronize();
        std::printf("MLA prefill workload: batch=%d sequence=%d heads=%d backward=%d\n", batch, sequence, heads, backward ? 1 : 0);
        CUDA_CHECK(cudaProfilerStart());
        run();
        dscuda::synchronize();
        CUDA_CHECK(cudaProfilerStop());
        const int status = dscuda::mla_device_status(false);
        if (status != 0) {
            std::fprintf(stderr, "MLA prefill benchmark: device status %d\n", status);
            return 1;
        }
        return 0;
    } catch (const std::exception& error) {
        std::fprintf(stderr, "MLA prefill benchmark failed: %s\n", error.what());
        return 1;
    }
}
