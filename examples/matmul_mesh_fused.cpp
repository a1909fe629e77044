// Sharded matmul on a 1 x g mesh of GPUs driven by one process, in the style of the reference's
// bench/metal/matmul_tensor_parallel.cpp (A replicated, B sharded on its columns, ttnn::matmul, ttnn::all_gather), with
// the two things that program does not have:
//   * the fused form of the same product — ttnn::experimental::matmul_all_gather, whose GEMM epilogue stores every
//     finished tile into all devices' C — checked bit for bit against matmul + all_gather and timed beside it;
//   * the K-split variant — A sharded on its columns, B on its rows — as ttnn::matmul + ttnn::reduce_scatter and as the
//     fused ttnn::experimental::matmul_reduce_scatter, both checked against a host product.
//
//   matmul_mesh_fused [g] [size]      g GPUs (default 2), square size (default 2048; a multiple of 128 * g)
// Prints "PARITY OK" and one CSV line per variant: variant,size,devices,mean_us,tflops. Exit code 1 on a mismatch.
#include <ttnn/device.hpp>
#include <ttnn/distributed/api.hpp>
#include <ttnn/operations/matmul/matmul.hpp>
#include <ttnn/tensor/tensor.hpp>
#include <tt-metalium/distributed.hpp>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <random>
#include <vector>

using namespace ttnn;
using namespace tt::tt_metal::distributed;

static std::vector<float> shard_to_host(const tt::tt_metal::Tensor& t, size_t i) {
    auto v = t.shard(i).cpu().to_vector<bfloat16>();
    return std::vector<float>(v.begin(), v.end());
}

template <typename Fn>
static double mean_us(MeshDevice& mesh, Fn&& fn, int warmup = 3, int iters = 10) {
    auto& cq = mesh.mesh_command_queue();
    for (int i = 0; i < warmup; ++i) fn();
    Finish(cq);
    const auto t0 = std::chrono::high_resolution_clock::now();
    for (int i = 0; i < iters; ++i) fn();
    Finish(cq);
    return std::chrono::duration<double, std::micro>(std::chrono::high_resolution_clock::now() - t0).count() / iters;
}

int main(int argc, char** argv) {
    const uint32_t g = argc > 1 ? static_cast<uint32_t>(std::atoi(argv[1])) : 2;
    const uint32_t size = argc > 2 ? static_cast<uint32_t>(std::atoi(argv[2])) : 2048;
    if (g < 2 || size % (128 * g) != 0) {
        std::fprintf(stderr, "usage: matmul_mesh_fused [g >= 2] [size, a multiple of 128 * g]\n");
        return 2;
    }
    auto mesh = ttnn::distributed::open_mesh_device(MeshShape(1, g));
    tt::tt_metal::TensorSpec spec(ttnn::Shape({size, size}),
                                  tt::tt_metal::TensorLayout(DataType::BFLOAT16, tt::tt_metal::PageConfig(Layout::TILE),
                                                             tt::tt_metal::MemoryConfig{}));
    std::mt19937 gen(42);
    std::normal_distribution<float> nd(0.0f, 1.0f);
    const size_t n = static_cast<size_t>(size) * size;
    std::vector<bfloat16> a_data(n), b_data(n);
    for (auto& v : a_data) v = bfloat16(nd(gen));
    for (auto& v : b_data) v = bfloat16(nd(gen));
    auto a_host = tt::tt_metal::Tensor::from_vector(a_data, spec);
    auto b_host = tt::tt_metal::Tensor::from_vector(b_data, spec);
    auto replicate = ttnn::distributed::replicate_tensor_to_mesh_mapper(*mesh);
    auto shard_cols = ttnn::distributed::shard_tensor_to_mesh_mapper(*mesh, 1);
    auto shard_rows = ttnn::distributed::shard_tensor_to_mesh_mapper(*mesh, 0);

    // host product of a row sample (fp32 accumulation of the bf16 values)
    const std::vector<uint32_t> rows = {0, size / 3, size / 2 + 1, size - 1};
    std::vector<std::vector<float>> ref(rows.size(), std::vector<float>(size, 0.0f));
    for (size_t r = 0; r < rows.size(); ++r)
        for (uint32_t k = 0; k < size; ++k) {
            const float av = static_cast<float>(a_data[static_cast<size_t>(rows[r]) * size + k]);
            for (uint32_t j = 0; j < size; ++j) ref[r][j] += av * static_cast<float>(b_data[static_cast<size_t>(k) * size + j]);
        }
    auto rel_err_rows = [&](const std::function<float(uint32_t, uint32_t)>& at) {
        double num = 0, den = 0;
        for (size_t r = 0; r < rows.size(); ++r)
            for (uint32_t j = 0; j < size; ++j) {
                const double d = at(rows[r], j) - ref[r][j];
                num += d * d;
                den += static_cast<double>(ref[r][j]) * ref[r][j];
            }
        return std::sqrt(num / den);
    };
    bool ok = true;

    // ---- N split: A replicated, B sharded on columns -----------------------------------------------------------
    auto a = ttnn::distributed::distribute_tensor(a_host, *replicate, std::ref(*mesh));
    auto b = ttnn::distributed::distribute_tensor(b_host, *shard_cols, std::ref(*mesh));
    auto c_unfused = ttnn::all_gather(ttnn::matmul(a, b), 1);
    auto c_fused = ttnn::experimental::matmul_all_gather(a, b);
    Finish(mesh->mesh_command_queue());
    for (uint32_t d = 0; d < g; ++d) {
        const auto u = shard_to_host(c_unfused, d), f = shard_to_host(c_fused, d);
        if (u != f) {
            std::printf("MISMATCH: fused all-gather differs from matmul + all_gather on device %u\n", d);
            ok = false;
        }
        const double e = rel_err_rows([&](uint32_t i, uint32_t j) { return f[static_cast<size_t>(i) * size + j]; });
        if (!(e <= 1e-2)) {
            std::printf("MISMATCH: all-gathered C on device %u is off by %.3e\n", d, e);
            ok = false;
        }
    }
    const double flops = 2.0 * std::pow(static_cast<double>(size), 3);
    const double t_u = mean_us(*mesh, [&] { auto c = ttnn::all_gather(ttnn::matmul(a, b), 1); });
    const double t_f = mean_us(*mesh, [&] { auto c = ttnn::experimental::matmul_all_gather(a, b); });

    // ---- K split: A sharded on columns, B on rows ----------------------------------------------------------------
    auto ak = ttnn::distributed::distribute_tensor(a_host, *shard_cols, std::ref(*mesh));
    auto bk = ttnn::distributed::distribute_tensor(b_host, *shard_rows, std::ref(*mesh));
    auto r_unfused = ttnn::reduce_scatter(ttnn::matmul(ak, bk), 0);
    auto r_fused = ttnn::experimental::matmul_reduce_scatter(ak, bk);
    Finish(mesh->mesh_command_queue());
    const uint32_t block = size / g;
    for (int fused = 0; fused < 2; ++fused) {
        std::vector<std::vector<float>> parts;
        for (uint32_t d = 0; d < g; ++d) parts.push_back(shard_to_host(fused ? r_fused : r_unfused, d));
        const double e = rel_err_rows([&](uint32_t i, uint32_t j) { return parts[i / block][static_cast<size_t>(i % block) * size + j]; });
        if (!(e <= 1e-2)) {
            std::printf("MISMATCH: %s reduce-scatter is off by %.3e\n", fused ? "fused" : "unfused", e);
            ok = false;
        }
    }
    const double t_ru = mean_us(*mesh, [&] { auto c = ttnn::reduce_scatter(ttnn::matmul(ak, bk), 0); });
    const double t_rf = mean_us(*mesh, [&] { auto c = ttnn::experimental::matmul_reduce_scatter(ak, bk); });

    std::printf(ok ? "PARITY OK\n" : "PARITY FAILED\n");
    std::printf("variant,size,devices,mean_us,tflops\n");
    std::printf("matmul+all_gather,%u,%u,%.1f,%.2f\n", size, g, t_u, flops / t_u / 1e6);
    std::printf("matmul_all_gather (fused),%u,%u,%.1f,%.2f\n", size, g, t_f, flops / t_f / 1e6);
    std::printf("matmul+reduce_scatter,%u,%u,%.1f,%.2f\n", size, g, t_ru, flops / t_ru / 1e6);
    std::printf("matmul_reduce_scatter (fused),%u,%u,%.1f,%.2f\n", size, g, t_rf, flops / t_rf / 1e6);
    ttnn::distributed::close_mesh_device(mesh);
    return ok ? 0 : 1;
}
