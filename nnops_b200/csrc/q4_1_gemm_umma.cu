// Q4_1 weight-decode GEMM for prefill-sized M on sm_100a:
//   out[M,N] = act(alpha * A[M,K] (f16) * dequant(W)[N,K]^T + bias), f32 accumulation.
//
// The reference only has a CPU route for this (decode W into dense f16 panels, then a dense
// MMA: FpRoute::pack_b -> pack_q4_1_rhs, src/backend/cpu/matmul/matmul.cpp:137-156,
// src/backend/cpu/x86_64/pack_q4_1.hpp:225-254).  Here the decode is fused into the operand
// staging of a tcgen05 pipeline, so the 4.5-bit weight stream is all that ever leaves HBM:
//
//   * warp 0 TMA-loads 128 x 64 f16 activation tiles (128-byte swizzle) into a ring;
//   * the same warp TMA-loads the RAW Q4_1 stream -- W viewed as rows of 32-bit words, one box
//     of 20 words (4 blocks = 128 k) x BN rows per two k-steps -- into a small ring; rows that
//     TMA cannot address (pitch or base not 16-byte aligned) are read with plain loads instead;
//   * BN/32 dequant warps (one thread per weight row) pull their row's 80 bytes from that ring
//     with conflict-free 16-byte shared loads, expand the nibbles to f16 with integer tricks
//     (nibble | 0x6400 = 1024 + q exactly, minus 1024, then one hfma2 q*d + m -- a single f16
//     rounding per weight, which is what the reference's f16 route stores), and write them
//     into the ring in the same K-major 128-byte-swizzled layout TMA would have produced;
//   * warp 1 issues tcgen05.mma kind::f16 (M128 x N=BN x K16) into one of two TMEM
//     accumulators; warps 2-5 drain the other one and apply alpha / bias / clip / activation.
//
// Every wait is bounded (see ptx.cuh).

#include <cstring>
#include <mutex>

#include "internal.cuh"
#include "ptx.cuh"
#include "q4_1_common.cuh"

namespace nnb200 {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;  // halves per stage = one 128-byte swizzle row = two Q4_1 blocks
constexpr int kUmmaKBytes = 32;
constexpr int kGroupM = 8;

constexpr int kRawSlots = 3;             // raw-block ring depth (each slot = 128 k of BN rows)
constexpr int kRawRowBytes = 4 * kQ4BlockBytes;  // 80 B: four blocks

template <int BN, bool RAW_TMA>
struct Q4Config {
    static constexpr int kATileBytes = kBlockM * kBlockK * 2;
    static constexpr int kBTileBytes = BN * kBlockK * 2;
    static constexpr int kStageBytes = kATileBytes + kBTileBytes;
    static constexpr int kRawSlotBytes = BN * kRawRowBytes;
    static constexpr int kRawBytes = RAW_TMA ? kRawSlots * kRawSlotBytes : 0;
    static constexpr int kStages = RAW_TMA ? ((BN == 256) ? 3 : 5) : ((BN == 256) ? 4 : 6);
    static constexpr int kDequantWarps = BN / 32;
    static constexpr int kNumThreads = (6 + kDequantWarps) * 32;
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kBarrierBytes = (3 * kStages + 4 + 2 * kRawSlots) * 8 + 16;
    static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kRawBytes + kBarrierBytes;
};

struct TileCoord {
    int m_blk;
    int n_blk;
};

__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m, int num_n)
{
    const int group_size = kGroupM * num_n;
    const int group = tile / group_size;
    const int first_m = group * kGroupM;
    const int gm = min(num_m - first_m, kGroupM);
    const int in_group = tile - group * group_size;
    TileCoord c;
    c.m_blk = first_m + in_group % gm;
    c.n_blk = in_group / gm;
    return c;
}

// Two nibble-carrying words (8 bytes of qs) -> 8 consecutive f16 weights of the low nibbles
// and 8 of the high nibbles, each as a uint4 of four half2.
__device__ __forceinline__ void dequant_word_pair(uint32_t w0, uint32_t w1, __half2 d2, __half2 m2, uint4& lo,
                                                  uint4& hi)
{
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
    const uint32_t magic = 0x64646464u;
    uint32_t lo_out[4], hi_out[4];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const uint32_t w = i == 0 ? w0 : w1;
        const uint32_t x = w & 0x0F0F0F0Fu;
        const uint32_t y = (w >> 4) & 0x0F0F0F0Fu;
        // bytes (n0, 0x64, n1, 0x64) = half2(1024 + n0, 1024 + n1)
        const uint32_t x01 = __byte_perm(x, magic, 0x4140);
        const uint32_t x23 = __byte_perm(x, magic, 0x4342);
        const uint32_t y01 = __byte_perm(y, magic, 0x4140);
        const uint32_t y23 = __byte_perm(y, magic, 0x4342);
        const __half2 q0 = __hsub2(*reinterpret_cast<const __half2*>(&x01), k1024);
        const __half2 q1 = __hsub2(*reinterpret_cast<const __half2*>(&x23), k1024);
        const __half2 q2 = __hsub2(*reinterpret_cast<const __half2*>(&y01), k1024);
        const __half2 q3 = __hsub2(*reinterpret_cast<const __half2*>(&y23), k1024);
        const __half2 r0 = __hfma2(q0, d2, m2);
        const __half2 r1 = __hfma2(q1, d2, m2);
        const __half2 r2 = __hfma2(q2, d2, m2);
        const __half2 r3 = __hfma2(q3, d2, m2);
        lo_out[2 * i] = *reinterpret_cast<const uint32_t*>(&r0);
        lo_out[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&r1);
        hi_out[2 * i] = *reinterpret_cast<const uint32_t*>(&r2);
        hi_out[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&r3);
    }
    lo = make_uint4(lo_out[0], lo_out[1], lo_out[2], lo_out[3]);
    hi = make_uint4(hi_out[0], hi_out[1], hi_out[2], hi_out[3]);
}

template <int BN, bool OUT_F16, bool RAW_TMA>
__global__ void __launch_bounds__(Q4Config<BN, RAW_TMA>::kNumThreads, 1)
q4_1_gemm_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                      const uint8_t* __restrict__ w,
                      const int64_t ldw_blocks, void* __restrict__ out, const int64_t ldc, const int m_total,
                      const int n_total, const int k_total, const FpEpilogue ep, const uint32_t idesc,
                      const int vec_ok, int32_t* error_word)
{
    using Cfg = Q4Config<BN, RAW_TMA>;
    constexpr int kStages = Cfg::kStages;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stage_base = smem;
    uint8_t* raw_base = smem + kStages * Cfg::kStageBytes;  // raw-block ring (RAW_TMA only)
    uint64_t* a_full_bar = reinterpret_cast<uint64_t*>(raw_base + Cfg::kRawBytes);
    uint64_t* b_full_bar = a_full_bar + kStages;
    uint64_t* empty_bar = b_full_bar + kStages;
    uint64_t* acc_full_bar = empty_bar + kStages;
    uint64_t* acc_empty_bar = acc_full_bar + 2;
    uint64_t* raw_full_bar = acc_empty_bar + 2;
    uint64_t* raw_empty_bar = raw_full_bar + kRawSlots;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(raw_empty_bar + kRawSlots);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int num_m = (m_total + kBlockM - 1) / kBlockM;
    const int num_n = (n_total + BN - 1) / BN;
    const int num_tiles = num_m * num_n;
    const int num_kb = (k_total + kBlockK - 1) / kBlockK;
    const int nblk = (k_total + kQ4BlockElems - 1) / kQ4BlockElems;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&a_full_bar[s], 1);
            mbar_init(&b_full_bar[s], Cfg::kDequantWarps);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full_bar[a], 1);
            mbar_init(&acc_empty_bar[a], 4);
        }
        for (int rs = 0; rs < kRawSlots; ++rs) {
            mbar_init(&raw_full_bar[rs], 1);
            mbar_init(&raw_empty_bar[rs], Cfg::kDequantWarps);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&map_a);
        if constexpr (RAW_TMA) {
            tma_prefetch_desc(&map_w);
        }
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer (activations) ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t armed = 0, armed_phase = 0;
            int rslot = 0;
            uint32_t rphase = 0;
            uint32_t rarmed = 0, rarmed_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                const TileCoord tc = tile_coord(tile, num_m, num_n);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if constexpr (RAW_TMA) {
                        if ((kb & 1) == 0) {
                            // Raw weights for k-steps kb and kb+1: 4 blocks of every row of the tile.
                            if (!mbar_wait(&raw_empty_bar[rslot], rphase ^ 1u, abort_flag)) {
                                atomicCAS(error_word, 0, kErrProducerWait);
                                ok = false;
                                break;
                            }
                            mbar_expect_tx(&raw_full_bar[rslot], Cfg::kRawSlotBytes);
                            tma_load_2d(raw_base + rslot * Cfg::kRawSlotBytes, &map_w, &raw_full_bar[rslot],
                                        (kb >> 1) * (kRawRowBytes / 4), tc.n_blk * BN);
                            rarmed |= 1u << rslot;
                            rarmed_phase = (rarmed_phase & ~(1u << rslot)) | (rphase << rslot);
                            if (++rslot == kRawSlots) {
                                rslot = 0;
                                rphase ^= 1u;
                            }
                        }
                    }
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
                        atomicCAS(error_word, 0, kErrProducerWait);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&a_full_bar[stage], Cfg::kATileBytes);
                    tma_load_2d(stage_base + stage * Cfg::kStageBytes, &map_a, &a_full_bar[stage], kb * kBlockK,
                                tc.m_blk * kBlockM);
                    armed |= 1u << stage;
                    armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                const long long t0 = clock64();
                for (int s = 0; s < kStages; ++s) {
                    if ((armed >> s) & 1u) {
                        while (!mbar_try_wait(&a_full_bar[s], (armed_phase >> s) & 1u)) {
                            if (clock64() - t0 > kWaitLimitCycles) {
                                atomicCAS(error_word, 0, kErrDrainWait);
                                break;
                            }
                        }
                    }
                }
                for (int s = 0; s < kRawSlots; ++s) {
                    if ((rarmed >> s) & 1u) {
                        while (!mbar_try_wait(&raw_full_bar[s], (rarmed_phase >> s) & 1u)) {
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
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&a_full_bar[stage], phase, abort_flag) ||
                        !mbar_wait(&b_full_bar[stage], phase, abort_flag)) {
                        atomicCAS(error_word, 0, kErrMmaWait);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(stage_base + stage * Cfg::kStageBytes);
                    const uint32_t b_addr = a_addr + Cfg::kATileBytes;
                    const uint64_t a_desc = umma_desc_sw128_kmajor(a_addr);
                    const uint64_t b_desc = umma_desc_sw128_kmajor(b_addr);
#pragma unroll
                    for (int ks = 0; ks < (kBlockK * 2) / kUmmaKBytes; ++ks) {
                        umma_f16(d_tmem, a_desc + static_cast<uint64_t>(ks * 2), b_desc + static_cast<uint64_t>(ks * 2),
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
    } else if (warp < 6) {
        // ---------------- epilogue warps ----------------
        const int quarter = warp & 3;
        int local_tile = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local_tile) {
            const TileCoord tc = tile_coord(tile, num_m, num_n);
            const int acc = local_tile & 1;
            const uint32_t acc_phase = (local_tile >> 1) & 1u;
            const int n_base = tc.n_blk * BN;
            const int64_t m = static_cast<int64_t>(tc.m_blk) * kBlockM + quarter * 32 + lane;
            const bool row_ok = m < m_total;

            // Warp-uniform outcome, so no lane is left behind at a later warp sync.
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(&acc_full_bar[acc], acc_phase, abort_flag))) {
                atomicCAS(error_word, 0, kErrEpilogueWait);
                break;
            }
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(acc * BN);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                const int n0 = n_base + c * 32;
                if (n0 >= n_total) {
                    break;
                }
                uint32_t v[32];
                tmem_ld_32x32(t_row + static_cast<uint32_t>(c * 32), v);
                tmem_ld_wait();
                const bool full = n0 + 32 <= n_total;
                if constexpr (OUT_F16) {
                    uint32_t packed[16];
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float f0 = fp_epilogue_value<true>(ep, __uint_as_float(v[j]), min(n0 + j, n_total - 1));
                        const float f1 =
                            fp_epilogue_value<true>(ep, __uint_as_float(v[j + 1]), min(n0 + j + 1, n_total - 1));
                        packed[j / 2] = static_cast<uint32_t>(__half_as_ushort(__float2half_rn(f0))) |
                                        (static_cast<uint32_t>(__half_as_ushort(__float2half_rn(f1))) << 16);
                    }
                    if (row_ok) {
                        uint16_t* dst = static_cast<uint16_t*>(out) + m * ldc + n0;
                        if (full && vec_ok) {
#pragma unroll
                            for (int j = 0; j < 16; j += 4) {
                                *reinterpret_cast<uint4*>(dst + 2 * j) =
                                    make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (n0 + j < n_total) {
                                    dst[j] = static_cast<uint16_t>(packed[j / 2] >> (16 * (j % 2)));
                                }
                            }
                        }
                    }
                } else {
                    float o[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        o[j] = fp_epilogue_value<false>(ep, __uint_as_float(v[j]), min(n0 + j, n_total - 1));
                    }
                    if (row_ok) {
                        float* dst = static_cast<float*>(out) + m * ldc + n0;
                        if (full && vec_ok) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                *reinterpret_cast<float4*>(dst + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (n0 + j < n_total) {
                                    dst[j] = o[j];
                                }
                            }
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
    } else {
        // ---------------- dequant warps ----------------
        const int r = (warp - 6) * 32 + lane;  // weight row inside the tile
        const int my_tiles = (num_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                             static_cast<int>(gridDim.x);
        const int total_it = my_tiles * num_kb;

        // Raw words of the two blocks of iteration `it` for this row (zeros when out of range).
        auto load_raw = [&](int it, uint32_t (&raw)[10]) {
            const int tile = static_cast<int>(blockIdx.x) + (it / num_kb) * static_cast<int>(gridDim.x);
            const int kb = it % num_kb;
            const TileCoord tc = tile_coord(tile, num_m, num_n);
            const int64_t n = static_cast<int64_t>(tc.n_blk) * BN + r;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int b = kb * 2 + j;
                if (n < n_total && b < nblk) {
                    const uint32_t* src = reinterpret_cast<const uint32_t*>(w + (n * ldw_blocks + b) * kQ4BlockBytes);
#pragma unroll
                    for (int i = 0; i < 5; ++i) {
                        raw[5 * j + i] = __ldg(src + i);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 5; ++i) {
                        raw[5 * j + i] = 0u;
                    }
                }
            }
        };

        // Dequantise blocks (5 words each) raw[0..4] and raw[5..9] of this row into B slot `stage`.
        auto emit_stage = [&](const uint32_t* raw, int stage) {
            uint8_t* b_row = stage_base + stage * Cfg::kStageBytes + Cfg::kATileBytes + r * 128;
            const int sw = r & 7;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t dm = raw[5 * j];
                const __half2 d2 = __half2half2(__ushort_as_half(static_cast<uint16_t>(dm & 0xFFFFu)));
                const __half2 m2 = __half2half2(__ushort_as_half(static_cast<uint16_t>(dm >> 16)));
                uint4 lo0, hi0, lo1, hi1;
                dequant_word_pair(raw[5 * j + 1], raw[5 * j + 2], d2, m2, lo0, hi0);  // k 0..7 and 16..23
                dequant_word_pair(raw[5 * j + 3], raw[5 * j + 4], d2, m2, lo1, hi1);  // k 8..15 and 24..31
                // 16-byte chunk c of the row lives at chunk (c ^ (row & 7)): the 128-byte swizzle.
                *reinterpret_cast<uint4*>(b_row + (((4 * j + 0) ^ sw) << 4)) = lo0;
                *reinterpret_cast<uint4*>(b_row + (((4 * j + 1) ^ sw) << 4)) = lo1;
                *reinterpret_cast<uint4*>(b_row + (((4 * j + 2) ^ sw) << 4)) = hi0;
                *reinterpret_cast<uint4*>(b_row + (((4 * j + 3) ^ sw) << 4)) = hi1;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&b_full_bar[stage]);
            }
        };

        int stage = 0;
        uint32_t phase = 0;
        if constexpr (RAW_TMA) {
            int rslot = 0;
            uint32_t rphase = 0;
            bool ok = true;
            for (int t = 0; ok && t < my_tiles; ++t) {
                for (int kb0 = 0; kb0 < num_kb; kb0 += 2) {
                    if (!__all_sync(0xFFFFFFFFu, mbar_wait(&raw_full_bar[rslot], rphase, abort_flag))) {
                        atomicCAS(error_word, 0, kErrDequantWait);
                        ok = false;
                        break;
                    }
                    // This row's 80 bytes: five 16-byte shared loads, conflict-free (80-byte row stride).
                    uint32_t raw[20];
                    const uint4* src = reinterpret_cast<const uint4*>(raw_base + rslot * Cfg::kRawSlotBytes + r * kRawRowBytes);
#pragma unroll
                    for (int j = 0; j < 5; ++j) {
                        const uint4 v = src[j];
                        raw[4 * j] = v.x;
                        raw[4 * j + 1] = v.y;
                        raw[4 * j + 2] = v.z;
                        raw[4 * j + 3] = v.w;
                    }
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&raw_empty_bar[rslot]);  // the slot can be refilled
                    }
                    if (++rslot == kRawSlots) {
                        rslot = 0;
                        rphase ^= 1u;
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (kb0 + h < num_kb) {
                            if (!__all_sync(0xFFFFFFFFu, mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag))) {
                                atomicCAS(error_word, 0, kErrDequantWait);
                                ok = false;
                                break;
                            }
                            emit_stage(raw + 10 * h, stage);
                            if (++stage == kStages) {
                                stage = 0;
                                phase ^= 1u;
                            }
                        }
                    }
                    if (!ok) {
                        break;
                    }
                }
            }
        } else {
            uint32_t next[10];
            if (total_it > 0) {
                load_raw(0, next);
            }
            for (int it = 0; it < total_it; ++it) {
                uint32_t raw[10];
#pragma unroll
                for (int i = 0; i < 10; ++i) {
                    raw[i] = next[i];
                }
                if (it + 1 < total_it) {
                    load_raw(it + 1, next);
                }
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag))) {
                    atomicCAS(error_word, 0, kErrDequantWait);
                    break;
                }
                emit_stage(raw, stage);
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
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

template <int BN, bool OUT_F16, bool RAW_TMA>
int launch_variant(const nnb200_q4_1_args& q, const CUtensorMap& map_a, const CUtensorMap& map_w, const FpEpilogue& ep,
                   const DeviceInfo& dev, cudaStream_t stream)
{
    using Cfg = Q4Config<BN, RAW_TMA>;
    auto kernel = q4_1_gemm_umma_kernel<BN, OUT_F16, RAW_TMA>;
    static std::once_flag once[kMaxDevices];
    static cudaError_t attr_err[kMaxDevices];
    std::call_once(once[dev.device], [&] {
        attr_err[dev.device] =
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    });
    if (attr_err[dev.device] != cudaSuccess) {
        return NNB200_INTERNAL;
    }
    const int m = static_cast<int>(q.m), n = static_cast<int>(q.n), k = static_cast<int>(q.k);
    const int num_tiles = ((m + kBlockM - 1) / kBlockM) * ((n + BN - 1) / BN);
    const int grid = num_tiles < dev.sm_count ? num_tiles : dev.sm_count;
    const int elem = OUT_F16 ? 2 : 4;
    const int vec_ok = ((reinterpret_cast<uintptr_t>(q.out) & 15u) == 0 &&
                        ((static_cast<uint64_t>(q.ldc) * elem) & 15u) == 0)
                           ? 1
                           : 0;
    kernel<<<grid, Cfg::kNumThreads, Cfg::kSmemBytes, stream>>>(
        map_a, map_w, static_cast<const uint8_t*>(q.w_blocks), q.ldw_blocks, q.out, q.ldc, m, n, k, ep,
        umma_idesc(1, 0, 0, kBlockM, BN), vec_ok, dev.error_word);
    note_launch();
    return cuda_status(cudaGetLastError());
}

}  // namespace

bool q4_1_gemm_umma_supported(const nnb200_q4_1_args& q)
{
    // Activations go through TMA as f16: 16-byte aligned base and row pitch.
    return q.a_f16 != 0 && q.m >= 1 && q.n >= 1 && q.k >= 1 && q.m <= INT32_MAX && q.n <= INT32_MAX &&
           q.k <= INT32_MAX && (reinterpret_cast<uintptr_t>(q.a) & 15u) == 0 && ((q.lda * 2) & 15) == 0 &&
           q.lda >= q.k && (reinterpret_cast<uintptr_t>(q.w_blocks) & 3u) == 0;
}

int launch_q4_1_gemm_umma(const nnb200_q4_1_args& q, const DeviceInfo& dev, cudaStream_t stream)
{
    FpEpilogue ep;
    ep.alpha = q.alpha;
    ep.bias = q.bias;
    ep.activation = q.activation;
    ep.act_alpha = q.act_alpha;
    ep.act_beta = q.act_beta;
    ep.min_clip = q.min_clip;
    ep.max_clip = q.max_clip;

    CUtensorMap map_a;
    if (!make_tma_2d(&map_a, q.a, 2, static_cast<uint64_t>(q.k), static_cast<uint64_t>(q.m),
                     static_cast<uint64_t>(q.lda) * 2, kBlockK, kBlockM)) {
        return NNB200_INTERNAL;
    }
    const int num_m = static_cast<int>((q.m + kBlockM - 1) / kBlockM);
    const bool wide = static_cast<int64_t>(num_m) * ((q.n + 255) / 256) >= dev.sm_count;
    // Raw blocks by TMA when W's rows are addressable as 16-byte aligned runs of 32-bit words.
    const bool raw_tma = (reinterpret_cast<uintptr_t>(q.w_blocks) & 15u) == 0 && (q.ldw_blocks % 4) == 0;
    CUtensorMap map_w;
    std::memset(&map_w, 0, sizeof(map_w));
    if (raw_tma) {
        const int64_t nblk = (q.k + kQ4BlockElems - 1) / kQ4BlockElems;
        if (!make_tma_2d(&map_w, q.w_blocks, 4, static_cast<uint64_t>(nblk * kQ4BlockWords), static_cast<uint64_t>(q.n),
                         static_cast<uint64_t>(q.ldw_blocks) * kQ4BlockBytes, kRawRowBytes / 4, wide ? 256u : 128u,
                         /*swizzle128=*/false)) {
            return NNB200_INTERNAL;
        }
    }
#define NNB200_Q4_LAUNCH(BNV, F16V)                                                              \
    (raw_tma ? launch_variant<BNV, F16V, true>(q, map_a, map_w, ep, dev, stream)                 \
             : launch_variant<BNV, F16V, false>(q, map_a, map_w, ep, dev, stream))
    if (wide) {
        return q.out_f16 ? NNB200_Q4_LAUNCH(256, true) : NNB200_Q4_LAUNCH(256, false);
    }
    return q.out_f16 ? NNB200_Q4_LAUNCH(128, true) : NNB200_Q4_LAUNCH(128, false);
#undef NNB200_Q4_LAUNCH
}

}  // namespace nnb200
