// benchmark_mla_decode [batch=2] [context=128] [heads=16] [kv_rank=512] [rope=64] [splits=8]
//
// Paged split-KV decode over `context` cached tokens per sequence (64-token pages, pages of the
// sequences interleaved in the cache), once untimed and once between cudaProfilerStart/Stop.
// Counterpart of the reference's benchmarks/attention/benchmark_mla_decode.cu.
#include "launcher_common.cuh"
#include "mla.h"

#include <cmath>
#include <cstdio>
#include <exception>
#include <vector>

int main(int argc, char** argv) {
    try {
        using launcher::DeviceBuffer;
        const int batch = launcher::argument(argc, argv, 1, 2);
        const int context = launcher::argument(argc, argv, 2, 128);
        const int heads = launcher::argument(argc, argv, 3, 16);
        const int rank = launcher::argument(argc, argv, 4, 512);
        const int rope = launcher::argument(argc, argv, 5, 64);
        const int splits = launcher::argument(argc, argv, 6, 8);
        const int page_size = 64;
        const int pages = (context + page_size - 1) / page_size;
        const float scale = 1.0F / std::sqrt(static_cast<float>(rank + rope));
        const std::size_t width = static_cast<std::size_t>(rank) + rope;
        DeviceBuffer<__nv_bfloat16> query(static_cast<std::size_t>(batch) * heads * width);
        DeviceBuffer<__nv_bfloat16> cache(static_cast<std::size_t>(batch) * pages * page_size * width);
        DeviceBuffer<__nv_bfloat16> output(static_cast<std::size_t>(batch) * heads * rank);
        DeviceBuffer<float> lse(static_cast<std::size_t>(batch) * heads);
        DeviceBuffer<float> workspace(dscuda::mla_decode_workspace_elements(batch, heads, splits, rank));
        DeviceBuffer<int> table(static_cast<std::size_t>(batch) * pages), lengths(batch);
        std::vector<int> host_table(static_cast<std::size_t>(batch) * pages), host_lengths(batch, context);
        for (int b = 0; b < batch; ++b) {
            for (int page = 0; page < pages; ++page) {
                host_table[static_cast<std::size_t>(b) * pages + page] = page * batch + b;      // neighbouring pages belong to different sequences
            }
        }
        CUDA_CHECK(cudaMemcpy(table.get(), host_table.data(), host_table.size() * sizeof(int), cudaMemcpyHostToDevice));
        CUDA_CHECK(cudaMemcpy(lengths.get(), host_lengths.data(), host_lengths.size() * sizeof(int), cudaMemcpyHostToDevice));
        launcher::fill(query, 1, 1.0F);
        launcher::fill(cache, 2, 1.0F);
        auto run = [&]() {
            dscuda::mla_decode_forward_cuda(output.get(), lse.get(), query.get(), cache.get(), table.get(), lengths.get(), workspace.get(), batch,
                                            heads, rank, rope, page_size, pages, splits, scale);
        };
        run();
        dscuda::synchronize();
        std::printf("MLA decode workload: batch=%d context=%d heads=%d kv_rank=%d rope=%d page=%d splits=%d\n", batch, context, heads, rank, rope,
                    page_size, splits);
        CUDA_CHECK(cudaProfilerStart());
        run();
        dscuda::synchronize();
        CUDA_CHECK(cudaProfilerStop());
        const int status = dscuda::mla_device_status(false);
        if (status != 0) {
            std::fprintf(stderr, "MLA decode benchmark: device status %d\n", status);
            return 1;
        }
        return 0;
    } catch (const std::exception& error) {
        std::fprintf(stderr, "MLA decode benchmark failed: %s\n", error.what());
        return 1;
    }
}
