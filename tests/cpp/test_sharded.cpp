// The C++ sharded layer (include/nnops_b200/sharded_linear.hpp), as forked processes:
//
//   test_sharded --exchange     CPU only.  LocalExchange among 4 ranks; a rank that announces its
//                               leaving (the others fail at once, naming it); a rank that never
//                               joins (the others fail at the deadline, naming it).
//   test_sharded --gpus N       N ranks, rank r on GPU r (N = 1: the degenerate layer).  Every
//                               rank's full output must equal, byte for byte, the single-GPU GEMM
//                               over the whole weight computed on that rank's own GPU.
//
// The parent never touches CUDA (it forks).  A lost rank is only ever produced on the host.
#include <cuda_runtime_api.h>
#include <sys/wait.h>
#include <unistd.h>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <string>
#include <vector>

#include "nnops_b200/sharded_linear.hpp"

using nnops::b200::LocalExchange;
using nnops::b200::ShardedLinearI8;

namespace {

std::string segment_name(const char* tag)
{
    return "/nnb200_test_" + std::to_string(getpid()) + "_" + tag;
}

// Fork one child per entry of `ranks`; each runs body(rank) and exits with its result.
// Returns the number of children that did not exit 0.
int run_ranks(const std::vector<int>& ranks, const std::function<int(int)>& body)
{
    std::vector<pid_t> pids;
    for (int r : ranks) {
        const pid_t pid = fork();
        if (pid == 0) {
            _exit(body(r));
        }
        pids.push_back(pid);
    }
    int bad = 0;
    for (pid_t pid : pids) {
        int status = 0;
        waitpid(pid, &status, 0);
        bad += (WIFEXITED(status) && WEXITSTATUS(status) == 0) ? 0 : 1;
    }
    return bad;
}

double seconds_since(std::chrono::steady_clock::time_point t0)
{
    return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
}

int exchange_tests()
{
    int failed = 0;
    {   // every rank sees every rank's payload, step after step
        const std::string name = segment_name("gather");
        const int world = 4;
        failed += run_ranks({0, 1, 2, 3}, [&](int rank) {
            LocalExchange ex(name, rank, world, 20.0);
            if (!ex.ok()) {
                return 2;
            }
            for (uint32_t step = 0; step < 300; ++step) {
                uint32_t mine[16], all[4 * 16];
                for (uint32_t i = 0; i < 16; ++i) {
                    mine[i] = (static_cast<uint32_t>(rank) << 24) ^ (step * 2654435761u) ^ i;
                }
                if (!ex.all_gather(mine, all, sizeof(mine))) {
                    return 3;
                }
                for (uint32_t r = 0; r < 4; ++r) {
                    for (uint32_t i = 0; i < 16; ++i) {
                        if (all[r * 16 + i] != ((r << 24) ^ (step * 2654435761u) ^ i)) {
                            return 4;
                        }
                    }
                }
            }
            return ex.barrier() ? 0 : 5;
        });
        shm_unlink(name.c_str());
        std::printf("exchange: 4 ranks x 300 steps: %s\n", failed == 0 ? "ok" : "FAILED");
    }
    {   // a rank that says it is leaving: the others' next exchange fails at once and names it
        const std::string name = segment_name("leave");
        const int before = failed;
        failed += run_ranks({0, 1, 2}, [&](int rank) {
            LocalExchange ex(name, rank, 3, 20.0);
            if (!ex.ok()) {
                return 2;
            }
            for (int step = 0; step < 5; ++step) {
                if (!ex.barrier()) {
                    return 3;
                }
            }
            if (rank == 1) {
                ex.leave();
                return 0;
            }
            const auto t0 = std::chrono::steady_clock::now();
            if (ex.barrier()) {
                return 4;   // must not succeed
            }
            if (ex.lost_rank() != 1 || seconds_since(t0) > 5.0) {
                return 5;
            }
            return ex.barrier() ? 6 : 0;   // and it stays failed
        });
        shm_unlink(name.c_str());
        std::printf("exchange: a rank leaves between steps: %s\n", failed == before ? "ok" : "FAILED");
    }
    {   // a rank that never joins: the deadline, and its number
        const std::string name = segment_name("absent");
        const int before = failed;
        failed += run_ranks({0, 1}, [&](int rank) {
            LocalExchange ex(name, rank, 3, 0.4);
            if (!ex.ok()) {
                return 2;
            }
            const auto t0 = std::chrono::steady_clock::now();
            if (ex.barrier()) {
                return 3;
            }
            const double dt = seconds_since(t0);
            return (ex.lost_rank() == 2 && dt >= 0.39 && dt < 5.0) ? 0 : 4;
        });
        shm_unlink(name.c_str());
        std::printf("exchange: a rank never joins: %s\n", failed == before ? "ok" : "FAILED");
    }
    {   // arguments
        LocalExchange bad_rank(segment_name("args"), 3, 3);
        LocalExchange bad_world(segment_name("args"), 0, 9);
        uint8_t b[8] = {};
        const bool ok = !bad_rank.ok() && !bad_world.ok() && !bad_rank.all_gather(b, b, 1);
        failed += ok ? 0 : 1;
        shm_unlink(segment_name("args").c_str());
        std::printf("exchange: bad rank / world refused: %s\n", ok ? "ok" : "FAILED");
    }
    return failed;
}

#define CUDA_OK(x)                                                                        \
    do {                                                                                  \
        const cudaError_t e_ = (x);                                                       \
        if (e_ != cudaSuccess) {                                                          \
            std::fprintf(stderr, "rank %d: %s -> %s\n", rank, #x, cudaGetErrorString(e_)); \
            return 10;                                                                    \
        }                                                                                 \
    } while (0)
#define NNB_OK(x)                                                                \
    do {                                                                         \
        const int s_ = (x);                                                      \
        if (s_ != NNB200_OK) {                                                   \
            std::fprintf(stderr, "rank %d: %s -> status %d\n", rank, #x, s_);     \
            return 11;                                                           \
        }                                                                        \
    } while (0)

int gpu_rank(int rank, int world, const std::string& name)
{
    // m >= 512 and k >= 2048: at two ranks the ordinary CTA-pair kernel with second stores into
    // the peer's copy, at more ranks the bulk-store form.
    const int64_t m = 640, k = 2048, n_per = 384, n = n_per * world;
    CUDA_OK(cudaSetDevice(rank));
    LocalExchange ex(name, rank, world, 120.0);
    if (!ex.ok()) {
        return 2;
    }
    // The same seeded inputs on every rank.
    std::vector<int8_t> a(static_cast<size_t>(m * k)), w(static_cast<size_t>(n * k));
    std::vector<float> scale(static_cast<size_t>(n));
    std::vector<int32_t> bias(static_cast<size_t>(n));
    uint32_t x = 12345u;
    const auto next = [&]() {
        x = x * 1664525u + 1013904223u;
        return x >> 8;
    };
    for (auto& v : a) v = static_cast<int8_t>(static_cast<int>(next() % 255u) - 127);
    for (auto& v : w) v = static_cast<int8_t>(static_cast<int>(next() % 255u) - 127);
    for (int64_t i = 0; i < n; ++i) {
        scale[static_cast<size_t>(i)] = 0.002f + 0.0001f * static_cast<float>(next() % 50u);
        bias[static_cast<size_t>(i)] = static_cast<int32_t>(next() % 2001u) - 1000;
    }
    int8_t *d_a = nullptr, *d_w = nullptr, *d_ref = nullptr;
    float* d_scale = nullptr;
    int32_t* d_bias = nullptr;
    CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&d_a), a.size()));
    CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&d_w), w.size()));
    CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&d_ref), static_cast<size_t>(m * n)));
    CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&d_scale), scale.size() * 4));
    CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&d_bias), bias.size() * 4));
    CUDA_OK(cudaMemcpy(d_a, a.data(), a.size(), cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(d_w, w.data(), w.size(), cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(d_scale, scale.data(), scale.size() * 4, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(d_bias, bias.data(), bias.size() * 4, cudaMemcpyHostToDevice));

    // Per-channel weight zero points for the second variant.
    std::vector<int32_t> zpw(static_cast<size_t>(n));
    for (auto& v : zpw) v = static_cast<int32_t>(next() % 9u) - 4;
    int32_t* d_zpw = nullptr;
    CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&d_zpw), zpw.size() * 4));
    CUDA_OK(cudaMemcpy(d_zpw, zpw.data(), zpw.size() * 4, cudaMemcpyHostToDevice));

    int mismatches = 0;
    // Variant 0: symmetric, s8 destination, ReLU (the benchmark's epilogue).  Variant 1: zero points
    // on both sides (compensation live in the sharded epilogue), u8 destination with a zero point.
    for (int variant = 0; variant < 2; ++variant) {
        nnb200_gemm_i8_args full;
        std::memset(&full, 0, sizeof(full));
        full.a = d_a; full.w = d_w; full.out = d_ref;
        full.m = m; full.n = n; full.k = k;
        full.a_stride_m = k; full.a_stride_k = 1; full.w_stride_n = k; full.w_stride_k = 1;
        full.ldc = n; full.batch = 1;
        full.out_kind = variant == 0 ? NNB200_OUT_S8 : NNB200_OUT_U8;
        full.bias = d_bias; full.relu = variant == 0 ? 1 : 0;
        full.scale_w = d_scale; full.scale_a_scalar = 0.02f; full.scale_w_scalar = 1.0f;
        full.out_scale = 0.9f;
        full.min_clip = -INFINITY; full.max_clip = INFINITY;
        if (variant == 1) {
            full.zp_a_scalar = 5;
            full.zp_w = d_zpw;
            full.zp_w_nonzero = 1;
            full.out_zp = 117;
        }
        void *ws_full = nullptr, *ws_shard = nullptr;
        full.workspace_bytes = nnb200_gemm_i8_workspace_bytes(&full);
        if (full.workspace_bytes > 0) {
            CUDA_OK(cudaMalloc(&ws_full, full.workspace_bytes));
            full.workspace = ws_full;
        }
        NNB_OK(nnb200_gemm_i8(&full, nullptr));

        nnb200_gemm_i8_args shard = full;
        shard.w = d_w + static_cast<int64_t>(rank) * n_per * k;
        shard.bias = d_bias + static_cast<int64_t>(rank) * n_per;
        shard.scale_w = d_scale + static_cast<int64_t>(rank) * n_per;
        shard.zp_w = variant == 1 ? d_zpw + static_cast<int64_t>(rank) * n_per : nullptr;
        shard.n = n_per;
        shard.workspace = nullptr;
        shard.workspace_bytes = nnb200_gemm_i8_workspace_bytes(&shard);   // asked with a valid destination in place
        shard.out = nullptr;
        if (shard.workspace_bytes > 0) {
            CUDA_OK(cudaMalloc(&ws_shard, shard.workspace_bytes));
            shard.workspace = ws_shard;
        }

        ShardedLinearI8 layer(ex, shard, n);
        NNB_OK(layer.alloc_outputs(m, 2));
        if (layer.alloc_outputs(m, 1) != NNB200_INVALID_ARGUMENT) {   // one allocation per layer
            return 14;
        }
        std::vector<int8_t> want(static_cast<size_t>(m * n)), got(want.size());
        CUDA_OK(cudaDeviceSynchronize());
        CUDA_OK(cudaMemcpy(want.data(), d_ref, want.size(), cudaMemcpyDeviceToHost));
        for (int round = 0; round < 3; ++round) {
            const int oi = round & 1;
            NNB_OK(layer.begin_step());
            CUDA_OK(cudaMemset(layer.output(oi), 0x55, want.size()));
            CUDA_OK(cudaDeviceSynchronize());
            if (!ex.barrier()) {   // nobody's stores arrive before everybody's fill is done
                return 12;
            }
            NNB_OK(layer.forward(d_a, k, oi, nullptr, round == 2));
            NNB_OK(layer.check());
            CUDA_OK(cudaMemcpy(got.data(), layer.output(oi), got.size(), cudaMemcpyDeviceToHost));
            if (std::memcmp(got.data(), want.data(), got.size()) != 0) {
                ++mismatches;
                std::fprintf(stderr, "rank %d variant %d round %d: output differs from the single-GPU result\n", rank,
                             variant, round);
            }
            if (!ex.barrier()) {   // everyone has read its copy before the next round overwrites it
                return 13;
            }
        }
        NNB_OK(layer.close());
        cudaFree(ws_full);
        cudaFree(ws_shard);
    }
    cudaFree(d_zpw);
    cudaFree(d_a); cudaFree(d_w); cudaFree(d_ref); cudaFree(d_scale); cudaFree(d_bias);
    return mismatches == 0 ? 0 : 1;
}

}  // namespace

int main(int argc, char** argv)
{
    if (argc >= 2 && std::strcmp(argv[1], "--exchange") == 0) {
        const int failed = exchange_tests();
        std::printf("%s: exchange, %d failed\n", failed == 0 ? "PASS" : "FAIL", failed);
        return failed == 0 ? 0 : 1;
    }
    if (argc >= 3 && std::strcmp(argv[1], "--gpus") == 0) {
        const int world = std::atoi(argv[2]);
        if (world < 1 || world > nnops::b200::kMaxShardRanks) {
            std::fprintf(stderr, "--gpus takes 1..8\n");
            return 2;
        }
        const std::string name = segment_name("gpus");
        std::vector<int> ranks;
        for (int r = 0; r < world; ++r) {
            ranks.push_back(r);
        }
        const int failed = run_ranks(ranks, [&](int rank) { return gpu_rank(rank, world, name); });
        shm_unlink(name.c_str());
        std::printf("%s: %d ranks, %d failed\n", failed == 0 ? "PASS" : "FAIL", world, failed);
        return failed == 0 ? 0 : 1;
    }
    std::fprintf(stderr, "usage: %s --exchange | --gpus N\n", argv[0]);
    return 2;
}
