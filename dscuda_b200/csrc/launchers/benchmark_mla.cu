// benchmark_mla [batch=1] [sequence=128] [heads=8] [kv_rank=512] [rope=64]
//
// Runs the absorbed causal forward and backward once untimed and once between
// cudaProfilerStart/Stop, for Nsight Compute (`--profile-from-start off`).  Counterpart of the
// reference's benchmarks/attention/benchmark_mla.cu (same arguments, same profiled region).
#include "launcher_common.cuh"
#include "mla.h"

#include <cmath>
#include <cstdio>
#include <exception>

int main(int argc, char** argv) {
    try {
        using launcher::DeviceBuffer;
        const int batch = launcher::argument(argc, argv, 1, 1);
        const int sequence = launcher::argument(argc, argv, 2, 128);
        const int heads = launcher::argument(argc, argv, 3, 8);
        const int rank = launcher::argument(argc, argv, 4, 512);
        const int rope = launcher::argument(argc, argv, 5, 64);
        const float scale = 1.0F / std::sqrt(static_cast<float>(rank + rope));
        const std::size_t rows = static_cast<std::size_t>(batch) * sequence * heads;
        const std::size_t keys = static_cast<std::size_t>(batch) * sequence;
        DeviceBuffer<__nv_bfloat16> query(rows * rank), query_rope(rows * rope), latent(keys * rank), key_rope(keys * rope);
        DeviceBuffer<__nv_bfloat16> output(rows * rank), dout(rows * rank);
        DeviceBuffer<__nv_bfloat16> dquery(rows * rank), dquery_rope(rows * rope), dlatent(keys * rank), dkey_rope(keys * rope);
        DeviceBuffer<float> lse(rows);
        launcher::fill(query, 1, 0.25F);
        launcher::fill(query_rope, 2, 0.25F);
        launcher::fill(latent, 3, 0.25F);
        launcher::fill(key_rope, 4, 0.25F);
        launcher::fill(dout, 5, 0.2F);
        auto run = [&]() {
            dscuda::mla_compressed_attention_forward_cuda(output.get(), lse.get(), query.get(), query_rope.get(), latent.get(), key_rope.get(),
                                                          batch, sequence, heads, rank, rope, scale);
            dscuda::mla_compressed_attention_backward_cuda(dquery.get(), dquery_rope.get(), dlatent.get(), dkey_rope.get(), dout.get(), output.get(),
                                                           lse.get(), query.get(), query_rope.get(), latent.get(), key_rope.get(), batch, sequence,
                                                           heads, rank, rope, scale);
        };
        run();
        dscuda::synchronize();
        std::printf("MLA workload: batch=%d sequence=%d heads=%d kv_rank=%d rope=%d\n", batch, sequence, heads, rank, rope);
        CUDA_CHECK(cudaProfilerStart());
        run();
        dscuda::synchronize();
        CUDA_CHECK(cudaProfilerStop());
        const int status = dscuda::mla_device_status(false);
        if (status != 0) {
            std::fprintf(stderr, "MLA benchmark: device status %d\n", status);
            return 1;
        }
        return 0;
    } catch (const std::exception& error) {
        std::fprintf(stderr, "MLA benchmark failed: %s\n", error.what());
        return 1;
    }
}
