// int8 GEMM for a handful of activation rows (17 <= M <= 128: batched decode, short prefills).
//
// With so few rows the whole cost is streaming W once, and the square-tile engine
// (gemm_i8_umma.cu) is a poor fit: it pads the activations to a 128-row MMA operand, re-reads
// that mostly empty tile for every 256 channels and, on mid-sized layers, has fewer tiles than
// the GPU has SMs.  Here the roles of the operands are swapped:
//
//   * the WEIGHTS are the 128-row operand of tcgen05.mma (M = 128 channels per tile), the
//     activations its N operand, padded only to MP = 32 / 64 / 128 rows;
//   * one tile = 128 channels x all activation rows: a stage is 16 KB of weights plus MP x 128
//     bytes of activations, so nearly all ring traffic is the weight stream itself, and N / 128
//     tiles keep more SMs busy than N / 256;
//   * the accumulator comes out transposed (TMEM lane = channel, column = activation row):
//     a thread owns ONE channel, loads that channel's scale / bias / zero point / row sum once
//     per tile into registers, and for each activation row the warp stores 32 consecutive
//     channels of that output row.
//
// Same pipeline skeleton as the square engine (TMA warp, MMA warp, four epilogue warps, two
// TMEM accumulators, bounded waits), same epilogue arithmetic (epilogue.cuh): results are
// bit-identical to every other int8 engine.

#include <mutex>

#include "internal.cuh"
#include "ptx.cuh"

namespace nnb200 {

namespace {

constexpr int kBlockN = 128;       // channels per tile = rows of the MMA's 128-row operand
constexpr int kBlockKBytes = 128;  // one 128-byte swizzle row of K per stage
constexpr int kUmmaK = 32;
constexpr int kNumThreads = 192;   // TMA warp, MMA warp, 4 epilogue warps
constexpr int kEpilogueThreads = 128;

template <int MP>
struct SkinnyConfig {
    static constexpr int kWTileBytes = kBlockN * kBlockKBytes;  // 16 KB
    static constexpr int kATileBytes = MP * kBlockKBytes;       // 4 / 8 / 16 KB
    static constexpr int kStageBytes = kWTileBytes + kATileBytes;
    static constexpr int kStages = (192 * 1024) / kStageBytes > 10 ? 10 : (192 * 1024) / kStageBytes;
    static constexpr int kTmemCols = 2 * MP < 32 ? 32 : 2 * MP;  // two accumulators of MP columns
    static constexpr int kRowTermBytes = 128 * 16;                // I8RowTerms of up to 128 activation rows
    static constexpr int kBarrierBytes = (2 * kStages + 4) * 8 + 16;
    static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kRowTermBytes + kBarrierBytes;
};

template <int MP, int KIND>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_i8_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                      const I8Epilogue ep, const int m_total, const int n_total, const int k_total,
                      const uint32_t idesc, int32_t* error_word)
{
    using Cfg = SkinnyConfig<MP>;
    constexpr int kStages = Cfg::kStages;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stage_base = smem;
    I8RowTerms* row_terms = reinterpret_cast<I8RowTerms*>(smem + kStages * Cfg::kStageBytes);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(row_terms) + Cfg::kRowTermBytes);
    uint64_t* empty_bar = full_bar + kStages;
    uint64_t* acc_full_bar = empty_bar + kStages;
    uint64_t* acc_empty_bar = acc_full_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_tiles = (n_total + kBlockN - 1) / kBlockN;
    const int num_kb = (k_total + kBlockKBytes - 1) / kBlockKBytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full_bar[a], 1);
            mbar_init(&acc_empty_bar[a], kEpilogueThreads / 32);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&map_w);
        tma_prefetch_desc(&map_a);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    // Per-row epilogue terms of every activation row, once per CTA (the rows are the same for all tiles).
    if (warp >= 2) {
        const int t = threadIdx.x - 64;
        if (t < m_total) {
            row_terms[t] = i8_row_terms(ep, t);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t armed = 0;
            uint32_t armed_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
                        atomicCAS(error_word, 0, kErrProducerWait);
                        ok = false;
                        break;
                    }
                    uint8_t* w_dst = stage_base + stage * Cfg::kStageBytes;
                    uint8_t* a_dst = w_dst + Cfg::kWTileBytes;
                    mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
                    tma_load_2d(w_dst, &map_w, &full_bar[stage], kb * kBlockKBytes, tile * kBlockN);
                    tma_load_2d(a_dst, &map_a, &full_bar[stage], kb * kBlockKBytes, 0);
                    armed |= 1u << stage;
                    armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                // Copies already issued still land in shared memory: wait (bounded) for the armed slots.
                const long long t0 = clock64();
                for (int s = 0; s < kStages; ++s) {
                    if ((armed >> s) & 1u) {
                        while (!mbar_try_wait(&full_bar[s], (armed_phase >> s) & 1u)) {
                            if (clock64() - t0 > kWaitLimitCycles) {
                                atomicCAS(error_word, 0, kErrDrainWait);
                                break;
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int local_tile = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local_tile) {
                const int acc = local_tile & 1;
                const uint32_t acc_phase = (local_tile >> 1) & 1u;
                if (!mbar_wait(&acc_empty_bar[acc], acc_phase ^ 1u, abort_flag)) {
                    atomicCAS(error_word, 0, kErrAccumWait);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * MP);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
                        atomicCAS(error_word, 0, kErrMmaWait);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t w_addr = smem_u32(stage_base + stage * Cfg::kStageBytes);
                    const uint32_t a_addr = w_addr + Cfg::kWTileBytes;
                    const uint64_t w_desc = umma_desc_sw128_kmajor(w_addr);  // the MMA's 128-row operand
                    const uint64_t a_desc = umma_desc_sw128_kmajor(a_addr);  // its N operand: MP activation rows
#pragma unroll
                    for (int ks = 0; ks < kBlockKBytes / kUmmaK; ++ks) {
                        umma_i8(d_tmem, w_desc + static_cast<uint64_t>(ks * 2), a_desc + static_cast<uint64_t>(ks * 2),
                                idesc, (kb > 0 || ks > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[stage]);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) {
                    umma_commit(&acc_full_bar[acc]);
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue warps: one channel per thread ----------------
        const int quarter = warp & 3;
        const float zpf = static_cast<float>(ep.out_zp);
        const float lo = (KIND == NNB200_OUT_S8 ? -128.0f : 0.0f) - zpf;
        const float hi = (KIND == NNB200_OUT_S8 ? 127.0f : 255.0f) - zpf;
        int local_tile = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local_tile) {
            const int acc = local_tile & 1;
            const uint32_t acc_phase = (local_tile >> 1) & 1u;
            const int64_t n = static_cast<int64_t>(tile) * kBlockN + quarter * 32 + lane;
            const bool n_ok = n < n_total;
            // This channel's terms, in registers for the whole tile.
            const int32_t zpw = (n_ok && ep.zp_w != nullptr) ? ep.zp_w[n] : ep.zp_w_scalar;
            const int32_t rw = (n_ok && ep.compensate) ? ep.r_w[n] : 0;
            const float s_w = (n_ok && ep.scale_w != nullptr) ? ep.scale_w[n] : ep.scale_w_scalar;
            int32_t bias_i = 0;
            float bias_f = 0.0f;
            if (n_ok && ep.bias != nullptr) {
                if constexpr (KIND <= NNB200_OUT_U8) {
                    bias_i = static_cast<const int32_t*>(ep.bias)[n];
                } else if constexpr (KIND == NNB200_OUT_F32) {
                    bias_f = static_cast<const float*>(ep.bias)[n];
                } else {
                    bias_f = __half2float(static_cast<const __half*>(ep.bias)[n]);
                }
            }

            if (!mbar_wait_warp(&acc_full_bar[acc], acc_phase, abort_flag)) {
                atomicCAS(error_word, 0, kErrEpilogueWait);
                break;
            }
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(acc * MP);
#pragma unroll 1
            for (int c = 0; c < MP / 32; ++c) {
                if (c * 32 >= m_total) {
                    break;  // uniform
                }
                uint32_t v[32];
                tmem_ld_32x32(t_row + static_cast<uint32_t>(c * 32), v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int m = c * 32 + j;
                    if (m < m_total && n_ok) {
                        const I8RowTerms t = row_terms[m];
                        const int64_t idx = static_cast<int64_t>(m) * ep.ldc + n;
                        const int32_t raw = static_cast<int32_t>(v[j]);
                        if constexpr (KIND == NNB200_OUT_S32) {
                            static_cast<int32_t*>(ep.out)[idx] = i8_int_value(ep, t, raw, zpw, rw, bias_i);
                        } else if constexpr (KIND == NNB200_OUT_S8) {
                            const int32_t val = i8_int_value(ep, t, raw, zpw, rw, bias_i);
                            static_cast<int8_t*>(ep.out)[idx] =
                                static_cast<int8_t>(i8_requant(val, __fmul_rn(t.row_k, s_w), lo, hi, ep.out_zp));
                        } else if constexpr (KIND == NNB200_OUT_U8) {
                            const int32_t val = i8_int_value(ep, t, raw, zpw, rw, bias_i);
                            static_cast<uint8_t*>(ep.out)[idx] =
                                static_cast<uint8_t>(i8_requant(val, __fmul_rn(t.row_k, s_w), lo, hi, ep.out_zp));
                        } else if constexpr (KIND == NNB200_OUT_F32) {
                            static_cast<float*>(ep.out)[idx] = i8_fp_value(ep, t, raw, zpw, rw, s_w, bias_f);
                        } else {
                            static_cast<__half*>(ep.out)[idx] =
                                __float2half_rn(i8_fp_value(ep, t, raw, zpw, rw, s_w, bias_f));
                        }
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&acc_empty_bar[acc]);
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

template <int MP, int KIND>
int launch_skinny_variant(const I8Problem& p, const I8Epilogue& ep, const DeviceInfo& dev, cudaStream_t stream)
{
    using Cfg = SkinnyConfig<MP>;
    auto kernel = gemm_i8_skinny_kernel<MP, KIND>;
    static std::once_flag once[kMaxDevices];
    static cudaError_t attr_err[kMaxDevices];
    std::call_once(once[dev.device], [&] {
        attr_err[dev.device] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    });
    if (attr_err[dev.device] != cudaSuccess) {
        return NNB200_INTERNAL;
    }
    const int m = static_cast<int>(p.m), n = static_cast<int>(p.n), k = static_cast<int>(p.k);
    CUtensorMap map_w, map_a;
    if (!make_tma_2d(&map_w, p.w, 1, static_cast<uint64_t>(k), static_cast<uint64_t>(n),
                     static_cast<uint64_t>(p.w_stride_n), kBlockKBytes, kBlockN) ||
        !make_tma_2d(&map_a, p.a, 1, static_cast<uint64_t>(k), static_cast<uint64_t>(m),
                     static_cast<uint64_t>(p.a_stride_m), kBlockKBytes, MP)) {
        return NNB200_INTERNAL;
    }
    const int num_tiles = (n + kBlockN - 1) / kBlockN;
    const int grid = num_tiles < dev.sm_count ? num_tiles : dev.sm_count;
    // 128-row operand = weights (s8), N operand = activations (s8 or u8).
    const uint32_t idesc = umma_idesc(2, 1, p.a_unsigned ? 0u : 1u, kBlockN, MP);
    kernel<<<grid, kNumThreads, Cfg::kSmemBytes, stream>>>(map_w, map_a, ep, m, n, k, idesc, dev.error_word);
    note_launch();
    return cuda_status(cudaGetLastError());
}

template <int MP>
int launch_skinny_mp(const I8Problem& p, const I8Epilogue& ep, const DeviceInfo& dev, cudaStream_t stream)
{
    switch (ep.out_kind) {
    case NNB200_OUT_S32: return launch_skinny_variant<MP, NNB200_OUT_S32>(p, ep, dev, stream);
    case NNB200_OUT_S8: return launch_skinny_variant<MP, NNB200_OUT_S8>(p, ep, dev, stream);
    case NNB200_OUT_U8: return launch_skinny_variant<MP, NNB200_OUT_U8>(p, ep, dev, stream);
    case NNB200_OUT_F32: return launch_skinny_variant<MP, NNB200_OUT_F32>(p, ep, dev, stream);
    case NNB200_OUT_F16: return launch_skinny_variant<MP, NNB200_OUT_F16>(p, ep, dev, stream);
    default: return NNB200_UNSUPPORTED;
    }
}

}  // namespace

// Same operand rules as the square tensor-core engine, at most 128 activation rows.
bool skinny_i8_supported(const I8Problem& p)
{
    return p.m >= 1 && p.m <= 128 && umma_i8_supported(p);
}

int launch_gemm_i8_skinny(const I8Problem& p, const I8Epilogue& ep, const DeviceInfo& dev, cudaStream_t stream)
{
    if (p.m <= 32) {
        return launch_skinny_mp<32>(p, ep, dev, stream);
    }
    if (p.m <= 64) {
        return launch_skinny_mp<64>(p, ep, dev, stream);
    }
    return launch_skinny_mp<128>(p, ep, dev, stream);
}

}  // namespace nnb200
