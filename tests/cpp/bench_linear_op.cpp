// Operator-level timing of the int8 Linear through the nnops API, the way an embedding
// application calls it: Linear::create(attrs, Backend::CUDA) -> compute(), pitched TensorViews
// over device memory, and the weight's per-channel QuantParams given as HOST arrays -- the
// reference contract (src/backend/cuda/matmul/matmul_i8.cuh:323-376), under which the backend
// stages those arrays to the device on every call.  Method after the reference's own operator
// bench (tests/bench_linear.cpp:127-163): warm-ups, then a timed loop, one synchronisation per
// step.
//
//   bench_linear_op [M N K [steps [warmup]]]      (default: 4096 28672 8192, 10 steps, 3 warm-ups)
//
// Two figures, one JSON line on stdout:
//   * "op_ms":  compute() alone, activations and output resident on the device;
//   * "e2e_ms": every step uploads the activations from pinned host memory, runs compute() and
//               reads the whole result back to pinned host memory.
// Built by nnops_b200/host/build.py against the real nnops headers and front end where the
// nnops source tree is present (NNB200_USE_NNOPS_HEADERS), else against the stand-alone mirror.

#ifdef NNB200_USE_NNOPS_HEADERS
#include "nnops/ops/linear.hpp"
#else
#include "nnops_b200/nnops_api.hpp"
#endif

#include <cuda_runtime_api.h>

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <span>
#include <vector>

using namespace nnops;

#define CUDA_OK(x)                                                             \
    do {                                                                       \
        if ((x) != cudaSuccess) {                                              \
            std::printf("{\"error\": \"CUDA call failed at line %d\"}\n", __LINE__); \
            return 2;                                                          \
        }                                                                      \
    } while (0)

int main(int argc, char** argv)
{
    int dev_count = 0;
    if (cudaGetDeviceCount(&dev_count) != cudaSuccess || dev_count == 0) {
        std::printf("{\"skipped\": \"no CUDA device\"}\n");
        return 77;
    }
    const int64_t m = argc > 3 ? std::atoll(argv[1]) : 4096;
    const int64_t n = argc > 3 ? std::atoll(argv[2]) : 28672;
    const int64_t k = argc > 3 ? std::atoll(argv[3]) : 8192;
    const int steps = argc > 4 ? std::atoi(argv[4]) : 10;
    const int warmup = argc > 5 ? std::atoi(argv[5]) : 3;

    // Seeded synthetic tensors with the benchmark's distributions (values do not affect timing).
    std::mt19937_64 rng(5);
    int8_t *a_host = nullptr, *out_host = nullptr;
    CUDA_OK(cudaMallocHost(reinterpret_cast<void**>(&a_host), static_cast<size_t>(m * k)));
    CUDA_OK(cudaMallocHost(reinterpret_cast<void**>(&out_host), static_cast<size_t>(m * n)));
    for (int64_t i = 0; i < m * k; ++i) a_host[i] = static_cast<int8_t>(static_cast<int>(rng() % 255) - 127);
    std::vector<int8_t> w(static_cast<size_t>(n * k));
    for (auto& v : w) v = static_cast<int8_t>(static_cast<int>(rng() % 255) - 127);
    std::vector<int32_t> bias(static_cast<size_t>(n));
    for (auto& v : bias) v = static_cast<int32_t>(rng() % 2001) - 1000;
    std::vector<float> sw(static_cast<size_t>(n));   // per-channel weight scales: a plain HOST array
    std::uniform_real_distribution<float> us(0.001f, 0.02f);
    for (auto& v : sw) v = us(rng);

    void *da = nullptr, *dw = nullptr, *dbias = nullptr, *dout = nullptr;
    CUDA_OK(cudaMalloc(&da, static_cast<size_t>(m * k)));
    CUDA_OK(cudaMalloc(&dw, static_cast<size_t>(n * k)));
    CUDA_OK(cudaMalloc(&dbias, static_cast<size_t>(n) * 4));
    CUDA_OK(cudaMalloc(&dout, static_cast<size_t>(m * n)));
    CUDA_OK(cudaMemcpy(da, a_host, static_cast<size_t>(m * k), cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(dw, w.data(), w.size(), cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(dbias, bias.data(), bias.size() * 4, cudaMemcpyHostToDevice));
    cudaStream_t stream;
    CUDA_OK(cudaStreamCreate(&stream));

    QuantParams qa, qw, qo;
    qa.scale = 0.02f;
    qw.granularity = QuantGranularity::PerChannel;
    qw.scale_data = sw.data();
    qw.num_scales = n;
    qo.scale = 0.05f;
    const int64_t xs[] = {m, k}, ws[] = {n, k}, bs[] = {n}, os[] = {m, n};
    TensorView x(std::span<const int64_t>(xs, 2), DataType::s8, da, TensorLayout::Dense, qa);
    TensorView wv(std::span<const int64_t>(ws, 2), DataType::s8, dw, TensorLayout::Dense, qw);
    TensorView bv(std::span<const int64_t>(bs, 1), DataType::s32, dbias, TensorLayout::Dense, QuantParams{});
    TensorView out(std::span<const int64_t>(os, 2), DataType::s8, dout, TensorLayout::Dense, qo);

    LinearAttributes attrs;
    attrs.output_dtype = DataType::s8;
    attrs.epilogue.type = EpilogueActivateType::Relu;
    auto op = Linear::create(attrs, Backend::CUDA);
    const TensorDesc in_d[] = {x.desc(), wv.desc(), bv.desc()};
    const TensorDesc out_d[] = {out.desc()};
    if (op->validate(in_d, out_d) != Status::ok) {
        std::printf("{\"error\": \"validate refused the views\"}\n");
        return 1;
    }
    const size_t ws_bytes = op->getWorkspaceSize(in_d, out_d);
    void* workspace = nullptr;
    if (ws_bytes > 0) {
        CUDA_OK(cudaMalloc(&workspace, ws_bytes));
    }
    ComputeContext ctx;
    ctx.expected_backend = Backend::CUDA;
    ctx.cuda_stream = stream;
    const TensorView ins[] = {x, wv, bv};

    const auto run = [&](bool with_copies, int count, double* ms_out) -> int {
        const auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < count; ++i) {
            if (with_copies) {
                CUDA_OK(cudaMemcpyAsync(da, a_host, static_cast<size_t>(m * k), cudaMemcpyHostToDevice, stream));
            }
            if (op->compute(out, ins, ctx, workspace) != Status::ok) {
                std::printf("{\"error\": \"compute returned an error status\"}\n");
                return 1;
            }
            if (with_copies) {
                CUDA_OK(cudaMemcpyAsync(out_host, dout, static_cast<size_t>(m * n), cudaMemcpyDeviceToHost, stream));
            }
            CUDA_OK(cudaStreamSynchronize(stream));
        }
        const auto t1 = std::chrono::steady_clock::now();
        *ms_out = std::chrono::duration<double, std::milli>(t1 - t0).count() / (count > 0 ? count : 1);
        return 0;
    };

    double op_ms = 0.0, e2e_ms = 0.0, unused = 0.0;
    if (int rc = run(false, warmup, &unused)) return rc;
    if (int rc = run(false, steps, &op_ms)) return rc;
    if (int rc = run(true, warmup, &unused)) return rc;
    if (int rc = run(true, steps, &e2e_ms)) return rc;

    const double ops = 2.0 * static_cast<double>(m) * static_cast<double>(n) * static_cast<double>(k);
    long checksum = 0;
    for (int64_t i = 0; i < m * n; i += 4097) checksum += out_host[i];
    std::printf("{\"m\": %lld, \"n\": %lld, \"k\": %lld, \"steps\": %d, \"warmup\": %d, \"op_ms\": %.4f, \"op_tops\": %.1f, "
                "\"e2e_ms\": %.4f, \"e2e_tops\": %.1f, \"h2d_bytes_per_step\": %lld, \"d2h_bytes_per_step\": %lld, "
                "\"scale_arrays\": \"host pointers, staged by the backend on every call\", \"front_end\": \"%s\", "
                "\"timer\": \"host steady_clock around the loop, one stream synchronisation per step\", \"checksum\": %ld}\n",
                static_cast<long long>(m), static_cast<long long>(n), static_cast<long long>(k), steps, warmup, op_ms,
                ops / (op_ms * 1e-3) / 1e12, e2e_ms, ops / (e2e_ms * 1e-3) / 1e12, static_cast<long long>(m * k),
                static_cast<long long>(m * n),
#ifdef NNB200_USE_NNOPS_HEADERS
                "nnops src/ops/linear.cpp (drop-in build)",
#else
                "stand-alone mirror",
#endif
                checksum);
    return 0;
}
