// Q4_1 prefill GEMM, two-pass form: expand the 4.5-bit weights to dense f16 once, then run a
// dense tcgen05 GEMM over them -- the same plan as the reference's CPU route for large M
// (decode W into dense panels, then a dense MMA: FpRoute::pack_b -> pack_q4_1_rhs,
// src/backend/cpu/matmul/matmul.cpp:137-156, src/backend/cpu/x86_64/pack_q4_1.hpp:225-254).
//
// Why a second form beside the fused kernel (q4_1_gemm_umma.cu): in the fused kernel every
// 128-channel weight tile is decoded again for every 256 activation rows, and turning the
// decoded tiles around in shared memory bounds it well below the tensor pipe's rate.  For tall
// problems it is cheaper to pay one streaming pass (read N*K*0.625 bytes, write N*K*2) into
// caller-provided scratch and then keep the tensor pipe fed by TMA alone:
//
//   pass 1  q4_1_expand_f16_kernel   two lanes per block: 16-byte coalesced-enough reads of the
//                                    raw stream, the same nibble -> f16 arithmetic as the fused
//                                    kernel (one f16 rounding per weight), 32-byte sector-complete
//                                    stores.  HBM-bound.
//   pass 2  gemm_f16_umma_kernel     persistent CTAs, 128 x BN output tiles; warp 0 streams A and
//                                    W tiles (64 k = one 128-byte swizzle row per stage) with TMA;
//                                    warp 1 issues tcgen05.mma kind::f16 (M128 x N=BN x K16) into
//                                    one of two TMEM accumulators; warps 2-5 drain the other
//                                    (alpha, bias, clip, activation) while the next tile's main
//                                    loop runs.  BN is picked from {256, 224, 192, 160, 128} to
//                                    minimise the padded work of the last partial wave.  From 512
//                                    rows up, two CTAs on neighbouring SMs share a 256-row tile and
//                                    one tcgen05.mma cta_group::2 (gemm_f16_umma_pair_kernel).
//
// Every barrier wait is bounded; a wait that runs out records an error code and the CTA tears
// down cleanly.

#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "internal.cuh"
#include "ptx.cuh"
#include "ptx_pair.cuh"
#include "q4_1_common.cuh"

namespace nnb200 {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;        // halves per stage = one 128-byte swizzle row
constexpr int kBlockKBytes = 128;
constexpr int kUmmaKBytes = 32;    // 16 halves per tcgen05.mma
constexpr int kNumThreads = 192;   // TMA warp, MMA warp, 4 epilogue warps
constexpr int kEpilogueThreads = 128;

template <int BN>
struct F16Config {
    static constexpr int kATileBytes = kBlockM * kBlockKBytes;
    static constexpr int kBTileBytes = BN * kBlockKBytes;
    static constexpr int kStageBytes = kATileBytes + kBTileBytes;
    static constexpr int kStages = (200 * 1024) / kStageBytes;  // 256: 4, 224: 4, 192: 5, 160: 5, 128: 6
    static constexpr int kTmemCols = 512;                       // two accumulators of BN <= 256 columns
    static constexpr int kBarrierBytes = (2 * kStages + 4) * 8 + 16;
    static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kBarrierBytes;
};

struct TileCoord {
    int m_blk;
    int n_blk;
};

// m-fastest inside groups of group_m m-blocks (their band of A stays in L2), groups n-fastest.
__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m, int num_n, int group_m)
{
    const int group_size = group_m * num_n;
    const int group = tile / group_size;
    const int first_m = group * group_m;
    const int gm = min(num_m - first_m, group_m);
    const int in_group = tile - group * group_size;
    TileCoord c;
    c.m_blk = first_m + in_group % gm;
    c.n_blk = in_group / gm;
    return c;
}

// ---- pass 1: Q4_1 -> dense f16 ---------------------------------------------------------------
// Lane pair (2b, 2b+1) of a warp owns one block: half h = lane & 1 decodes qs bytes 8h..8h+7,
// i.e. weights k 8h..8h+7 (low nibbles) and 16+8h..16+8h+7 (high nibbles), and stores them as
// two 16-byte pieces; a pair thereby completes the 32-byte sectors [k 0..15] and [k 16..31].
// A CTA walks whole rows (no index division anywhere); every thread has the loads of two rows in
// flight before it decodes either.
// dm_plane != nullptr: the weights are packed (nnb200_q4_1_pack) -- `w` is then the nibble plane,
// 16 bytes per block, and dm_plane the (d, m) plane with rows ld_dm entries apart.
__global__ void __launch_bounds__(256) q4_1_expand_f16_kernel(const uint8_t* __restrict__ w, const int64_t ldw_blocks,
                                                              const uint32_t* __restrict__ dm_plane, const int64_t ld_dm,
                                                              const int rows, const int nblk,
                                                              __half* __restrict__ out, const int64_t ld_out)
{
    const int half_blocks = 2 * nblk;
    const bool planes = dm_plane != nullptr;
    const int64_t pitch = ldw_blocks * (planes ? 16 : kQ4BlockBytes);
    for (int r0 = blockIdx.x; r0 < rows; r0 += 2 * gridDim.x) {
        const int r1 = r0 + gridDim.x;
        for (int hb = threadIdx.x; hb < half_blocks; hb += blockDim.x) {
            const int b = hb >> 1;
            const int h = hb & 1;
            uint32_t dm[2], q0[2], q1[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int r = u == 0 ? r0 : r1;
                if (r < rows) {
                    if (planes) {
                        const uint32_t* src = reinterpret_cast<const uint32_t*>(w + r * pitch + b * 16);
                        dm[u] = __ldg(dm_plane + r * ld_dm + b);
                        q0[u] = __ldg(src + 2 * h);
                        q1[u] = __ldg(src + 1 + 2 * h);
                    } else {
                        const uint32_t* src = reinterpret_cast<const uint32_t*>(w + r * pitch + b * kQ4BlockBytes);
                        dm[u] = __ldg(src);
                        q0[u] = __ldg(src + 1 + 2 * h);
                        q1[u] = __ldg(src + 2 + 2 * h);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int r = u == 0 ? r0 : r1;
                if (r < rows) {
                    const __half2 d2 = __half2half2(__ushort_as_half(static_cast<uint16_t>(dm[u] & 0xFFFFu)));
                    const __half2 m2 = __half2half2(__ushort_as_half(static_cast<uint16_t>(dm[u] >> 16)));
                    uint4 lo, hi;
                    dequant_word_pair(q0[u], q1[u], d2, m2, lo, hi);
                    __half* dst = out + r * ld_out + b * kQ4BlockElems + 8 * h;
                    __stcg(reinterpret_cast<uint4*>(dst), lo);
                    __stcg(reinterpret_cast<uint4*>(dst + 16), hi);
                }
            }
        }
    }
}

// ---- pass 1b: f32 activations -> [hi | lo] f16 ------------------------------------------------
// a = hi + lo with hi = f16(a), lo = f16(a - hi): the pair carries 22 mantissa bits, so the dense
// GEMM over [hi | lo] (weights repeating along K) reproduces an f32-activation product to f32
// accuracy.  Row m of `out` is [hi(0..kp) | lo(0..kp)], kp = K rounded up to 64, zeros past K.
// Values beyond the f16 range (|a| > 65504) become infinities, as in any f16 activation pipeline.
__global__ void __launch_bounds__(256) split_f32_to_f16_kernel(const float* __restrict__ a, const int64_t lda,
                                                               const int m, const int k, const int kp,
                                                               __half* __restrict__ out)
{
    const int64_t total = static_cast<int64_t>(m) * kp;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t r = i / kp;
        const int c = static_cast<int>(i - r * kp);
        float v = 0.0f;
        if (c < k) {
            v = a[r * lda + c];
        }
        const __half hi = __float2half_rn(v);
        const __half lo = __float2half_rn(v - __half2float(hi));
        out[r * 2 * kp + c] = hi;
        out[r * 2 * kp + kp + c] = lo;
    }
}

// ---- pass 2: dense f16 GEMM ------------------------------------------------------------------
// Drain one accumulator (this warp's 32 rows x BN columns) through the fp epilogue into `out`.
template <int BN, bool OUT_F16>
__device__ __forceinline__ void drain_accumulator(uint32_t t_row, int64_t m, bool row_ok, int n_base, int n_total,
                                                  void* __restrict__ out, int64_t ldc, const FpEpilogue& ep,
                                                  bool identity, int vec_ok)
{
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
        const int n0 = n_base + c * 32;
        if (n0 >= n_total) {
            break;  // warp-uniform
        }
        uint32_t v[32];
        tmem_ld_32x32(t_row + static_cast<uint32_t>(c * 32), v);
        tmem_ld_wait();
        const bool full = n0 + 32 <= n_total;
        if constexpr (OUT_F16) {
            float o[32];
            fp_epilogue_chunk<true>(ep, identity, v, n0, n_total, o);
            uint32_t packed[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                packed[j / 2] = static_cast<uint32_t>(__half_as_ushort(__float2half_rn(o[j]))) |
                                (static_cast<uint32_t>(__half_as_ushort(__float2half_rn(o[j + 1]))) << 16);
            }
            if (row_ok) {
                uint16_t* dst = static_cast<uint16_t*>(out) + m * ldc + n0;
                if (full && (vec_ok & 2)) {
                    // 64 bytes per lane: two whole 32-byte sectors, one 256-bit store each.
                    st_global_32(dst, packed[0], packed[1], packed[2], packed[3], packed[4], packed[5], packed[6],
                                 packed[7]);
                    st_global_32(dst + 16, packed[8], packed[9], packed[10], packed[11], packed[12], packed[13],
                                 packed[14], packed[15]);
                } else if (full && (vec_ok & 1)) {
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
            fp_epilogue_chunk<false>(ep, identity, v, n0, n_total, o);
            if (row_ok) {
                float* dst = static_cast<float*>(out) + m * ldc + n0;
                if (full && (vec_ok & 1)) {
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
}

template <int BN, bool OUT_F16>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_f16_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                     void* __restrict__ out, const int64_t ldc, const int m_total, const int n_total,
                     const int k_total, const int w_wrap_k, const FpEpilogue ep, const uint32_t idesc,
                     const int vec_ok, const int group_m, int32_t* error_word)
{
    using Cfg = F16Config<BN>;
    constexpr int kStages = Cfg::kStages;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stage_base = smem;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes);
    uint64_t* empty_bar = full_bar + kStages;
    uint64_t* acc_full_bar = empty_bar + kStages;
    uint64_t* acc_empty_bar = acc_full_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_m = (m_total + kBlockM - 1) / kBlockM;
    const int num_n = (n_total + BN - 1) / BN;
    const int num_tiles = num_m * num_n;
    const int num_kb = (k_total + kBlockK - 1) / kBlockK;

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
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_w);
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
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t armed = 0;        // bit s: slot s has been armed at least once
            uint32_t armed_phase = 0;  // bit s: parity of the phase slot s was last armed in
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                const TileCoord tc = tile_coord(tile, num_m, num_n, group_m);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
                        atomicCAS(error_word, 0, kErrProducerWait);
                        ok = false;
                        break;
                    }
                    uint8_t* a_dst = stage_base + stage * Cfg::kStageBytes;
                    uint8_t* b_dst = a_dst + Cfg::kATileBytes;
                    mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
                    // x coordinates are in elements: kb * 64 halves = a multiple of 128 bytes.
                    // With split activations ([hi | lo] along K) the weights repeat every w_wrap_k.
                    const int wk = w_wrap_k > 0 ? (kb * kBlockK) % w_wrap_k : kb * kBlockK;
                    tma_load_2d(a_dst, &map_a, &full_bar[stage], kb * kBlockK, tc.m_blk * kBlockM);
                    tma_load_2d(b_dst, &map_w, &full_bar[stage], wk, tc.n_blk * BN);
                    armed |= 1u << stage;
                    armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                // Copies already issued still land in shared memory: wait (bounded) for the armed
                // slots so the CTA does not exit underneath them.
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
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * 256);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
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
                    for (int ks = 0; ks < kBlockKBytes / kUmmaKBytes; ++ks) {
                        // +32 bytes of K per step = +2 in the descriptor's 16-byte address units.
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
    } else {
        // ---------------- epilogue warps ----------------
        const int quarter = warp & 3;  // the TMEM lane quarter this warp may read
        const bool identity = fp_epilogue_is_identity(ep);
        int local_tile = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local_tile) {
            const TileCoord tc = tile_coord(tile, num_m, num_n, group_m);
            const int acc = local_tile & 1;
            const uint32_t acc_phase = (local_tile >> 1) & 1u;
            const int n_base = tc.n_blk * BN;
            const int64_t m = static_cast<int64_t>(tc.m_blk) * kBlockM + quarter * 32 + lane;
            const bool row_ok = m < m_total;

            // Warp-uniform outcome, so no lane is left behind at a later warp sync.
            if (!mbar_wait_warp(&acc_full_bar[acc], acc_phase, abort_flag)) {
                atomicCAS(error_word, 0, kErrEpilogueWait);
                break;
            }
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(acc * 256);
            drain_accumulator<BN, OUT_F16>(t_row, m, row_ok, n_base, n_total, out, ldc, ep, identity, vec_ok);
            // Accumulator drained: hand it back to the MMA warp.
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


// ---- pass 2, CTA-pair form -------------------------------------------------------------------
// Two CTAs (a cluster of two, on neighbouring SMs) share one 256 x BN output tile: each loads its
// own 128 rows of A and HALF of the tile's W rows, the pair leader issues tcgen05.mma with
// cta_group::2 (M = 256 over both SMs' tensor cores and TMEM, both halves of W read from the two
// CTAs' shared memory), and each CTA drains its own 128 accumulator rows.  Per multiply-add that
// is two thirds of the TMA write traffic and of the L2 -> SM traffic of the single-CTA form, and
// the smaller stages leave room for a deeper ring.
//
// Signalling: TMA loads of both CTAs report their bytes to the LEADER's full barrier; the
// leader's commits arrive on BOTH CTAs' empty / accumulator-full barriers (one instruction with a
// CTA mask; two k-blocks share a barrier slot, see gemm_i8_umma.cu); the epilogue warps of both CTAs arrive on the leader's accumulator-empty
// barrier.  A cluster barrier brackets the kernel so neither CTA initialises late or exits early.
template <int BN>
struct PairConfig {
    static constexpr int kATileBytes = kBlockM * kBlockKBytes;       // this CTA's 128 rows of A
    static constexpr int kBTileBytes = (BN / 2) * kBlockKBytes;      // this CTA's half of the W rows
    static constexpr int kStageBytes = kATileBytes + kBTileBytes;
    static constexpr int kStages = (200 * 1024) / kStageBytes;       // 256: 6, 224: 6, 192: 7
    static constexpr int kTmemCols = 512;
    static constexpr int kBarrierBytes = (2 * kStages + 4) * 8 + 16;
    static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kBarrierBytes;
};

template <int BN, bool OUT_F16, int SUB, bool MC>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreads, 1)
gemm_f16_umma_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                          void* __restrict__ out, const int64_t ldc, const int m_total, const int n_total,
                          const int k_total, const int w_wrap_k, const FpEpilogue ep, const uint32_t idesc,
                          const int vec_ok, const int group_m, int32_t* error_word)
{
    using Cfg = PairConfig<BN>;
    // SUB consecutive k-blocks share one pair of barriers (a "slot"): one wait, one expect-tx and
    // one round of commits per SUB x 4 MMAs.
    constexpr int kStages = Cfg::kStages / SUB;   // slots in the ring
    constexpr int kSlotBytes = SUB * Cfg::kStageBytes;
    constexpr int kPairM = 2 * kBlockM;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stage_base = smem;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
    uint64_t* empty_bar = full_bar + Cfg::kStages;
    uint64_t* acc_full_bar = empty_bar + Cfg::kStages;
    uint64_t* acc_empty_bar = acc_full_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();  // 0 = pair leader
    const int pair = static_cast<int>(blockIdx.x >> 1);
    const int num_pairs = static_cast<int>(gridDim.x >> 1);
    const int num_m = (m_total + kPairM - 1) / kPairM;
    const int num_n = (n_total + BN - 1) / BN;
    const int num_tiles = num_m * num_n;
    const int num_kb = (k_total + kBlockK - 1) / kBlockK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);   // the leader's: its own expect-tx arrival; bytes come from both CTAs
            mbar_init(&empty_bar[s], 1);  // one commit from the leader
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full_bar[a], 1);
            mbar_init(&acc_empty_bar[a], 2 * kEpilogueThreads / 32);  // the leader's: 4 warps of each CTA
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_w);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    cluster_sync_all();  // both CTAs' barriers and TMEM exist before anything is signalled across
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer (each CTA loads its own halves) ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                const TileCoord tc = tile_coord(tile, num_m, num_n, group_m);
                const int m0 = tc.m_blk * kPairM + static_cast<int>(rank) * kBlockM;
                const int n0 = tc.n_blk * BN + static_cast<int>(rank) * (BN / 2);
                for (int kb = 0; kb < num_kb; kb += SUB) {
                    if (!mbar_wait_cluster(&empty_bar[stage], phase ^ 1u, abort_flag)) {
                        atomicCAS(error_word, 0, kErrProducerWait);
                        ok = false;
                        break;
                    }
                    const int nsub = (num_kb - kb) < SUB ? (num_kb - kb) : SUB;
                    if (rank == 0) {
                        mbar_expect_tx(&full_bar[stage], 2 * nsub * Cfg::kStageBytes);
                    }
                    const uint32_t leader_full = map_to_cta(smem_u32(&full_bar[stage]), 0);
#pragma unroll
                    for (int j = 0; j < SUB; ++j) {
                        if (j < nsub) {
                            uint8_t* a_dst = stage_base + stage * kSlotBytes + j * Cfg::kStageBytes;
                            uint8_t* b_dst = a_dst + Cfg::kATileBytes;
                            const int k0 = (kb + j) * kBlockK;
                            const int wk = w_wrap_k > 0 ? k0 % w_wrap_k : k0;
                            tma_load_2d_pair(a_dst, &map_a, leader_full, k0, m0);
                            tma_load_2d_pair(b_dst, &map_w, leader_full, wk, n0);
                        }
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer (pair leader only) ----------------
        if (lane == 0 && rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int local_tile = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs, ++local_tile) {
                const int acc = local_tile & 1;
                const uint32_t acc_phase = (local_tile >> 1) & 1u;
                if (!mbar_wait_cluster(&acc_empty_bar[acc], acc_phase ^ 1u, abort_flag)) {
                    atomicCAS(error_word, 0, kErrAccumWait);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * 256);
                for (int kb = 0; kb < num_kb; kb += SUB) {
                    if (!mbar_wait_cluster(&full_bar[stage], phase, abort_flag)) {
                        atomicCAS(error_word, 0, kErrMmaWait);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const int nsub = (num_kb - kb) < SUB ? (num_kb - kb) : SUB;
#pragma unroll
                    for (int j = 0; j < SUB; ++j) {
                        if (j < nsub) {
                            const uint32_t a_addr = smem_u32(stage_base + stage * kSlotBytes + j * Cfg::kStageBytes);
                            const uint32_t b_addr = a_addr + Cfg::kATileBytes;
                            const uint64_t a_desc = umma_desc_sw128_kmajor(a_addr);
                            const uint64_t b_desc = umma_desc_sw128_kmajor(b_addr);
#pragma unroll
                            for (int ks = 0; ks < kBlockKBytes / kUmmaKBytes; ++ks) {
                                umma_f16_pair(d_tmem, a_desc + static_cast<uint64_t>(ks * 2),
                                              b_desc + static_cast<uint64_t>(ks * 2), idesc,
                                              (kb > 0 || j > 0 || ks > 0) ? 1u : 0u);
                            }
                        }
                    }
                    // The slot is free in BOTH CTAs once these MMAs have read it.
                    if constexpr (MC) {
                        umma_commit_pair_mask(&empty_bar[stage], 3);
                    } else {
                        const uint32_t e = smem_u32(&empty_bar[stage]);
                        umma_commit_pair(map_to_cta(e, 0));
                        umma_commit_pair(map_to_cta(e, 1));
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) {
                    if constexpr (MC) {
                        umma_commit_pair_mask(&acc_full_bar[acc], 3);
                    } else {
                        const uint32_t f = smem_u32(&acc_full_bar[acc]);
                        umma_commit_pair(map_to_cta(f, 0));
                        umma_commit_pair(map_to_cta(f, 1));
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue warps (each CTA drains its own 128 rows) ----------------
        const int quarter = warp & 3;
        const bool identity = fp_epilogue_is_identity(ep);
        int local_tile = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local_tile) {
            const TileCoord tc = tile_coord(tile, num_m, num_n, group_m);
            const int acc = local_tile & 1;
            const uint32_t acc_phase = (local_tile >> 1) & 1u;
            const int n_base = tc.n_blk * BN;
            const int64_t m = static_cast<int64_t>(tc.m_blk) * kPairM + static_cast<int64_t>(rank) * kBlockM +
                              quarter * 32 + lane;
            const bool row_ok = m < m_total;
            int ok = 1;
            if (lane == 0) {
                ok = mbar_wait_cluster(&acc_full_bar[acc], acc_phase, abort_flag) ? 1 : 0;
            }
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) {
                atomicCAS(error_word, 0, kErrEpilogueWait);
                break;
            }
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(acc * 256);
            drain_accumulator<BN, OUT_F16>(t_row, m, row_ok, n_base, n_total, out, ldc, ep, identity, vec_ok);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty_bar[acc]), 0));
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before_sync();
    cluster_sync_all();  // the peer has stopped signalling into / reading from this CTA
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    }
}

// The dense GEMM's operands: A as f16 [m][k_loop] (the caller's activations, or their [hi | lo]
// split) and the expanded weights [n][k_w]; w_wrap_k > 0 makes the weights' k index wrap.
struct F16Operands {
    const __half* a;
    int64_t lda;
    int k_loop;
    const __half* w;
    int64_t ldw;
    int k_w;
    int w_wrap_k;
};

template <int BN, bool OUT_F16>
int launch_f16_variant(const nnb200_q4_1_args& q, const F16Operands& op, const FpEpilogue& ep,
                       const DeviceInfo& dev, cudaStream_t stream)
{
    using Cfg = F16Config<BN>;
    auto kernel = gemm_f16_umma_kernel<BN, OUT_F16>;
    static std::once_flag once[kMaxDevices];
    static cudaError_t attr_err[kMaxDevices];
    std::call_once(once[dev.device], [&] {
        attr_err[dev.device] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    });
    if (attr_err[dev.device] != cudaSuccess) {
        return NNB200_INTERNAL;
    }
    const int m = static_cast<int>(q.m), n = static_cast<int>(q.n), k = op.k_loop;
    CUtensorMap map_a, map_w;
    if (!make_tma_2d(&map_a, op.a, 2, static_cast<uint64_t>(op.k_loop), static_cast<uint64_t>(m),
                     static_cast<uint64_t>(op.lda) * 2, kBlockK, kBlockM) ||
        !make_tma_2d(&map_w, op.w, 2, static_cast<uint64_t>(op.k_w), static_cast<uint64_t>(n),
                     static_cast<uint64_t>(op.ldw) * 2, kBlockK, BN)) {
        return NNB200_INTERNAL;
    }
    const int num_tiles = ((m + kBlockM - 1) / kBlockM) * ((n + BN - 1) / BN);
    const int grid = num_tiles < dev.sm_count ? num_tiles : dev.sm_count;
    const int elem = OUT_F16 ? 2 : 4;
    // Destination vector stores: bit 0 = 16-byte aligned base and row pitch, bit 1 = 32-byte.
    const uint64_t out_pitch = static_cast<uint64_t>(q.ldc) * elem;
    const int vec_ok = (((reinterpret_cast<uintptr_t>(q.out) & 15u) == 0 && (out_pitch & 15u) == 0) ? 1 : 0) |
                       (((reinterpret_cast<uintptr_t>(q.out) & 31u) == 0 && (out_pitch & 31u) == 0) ? 2 : 0);
    // Raster group: m-blocks whose band of A (128 x K halves each) stays within ~40 MB of L2.
    int group_m = static_cast<int>((40ll << 20) / (static_cast<int64_t>(kBlockM) * 2 * (k > 0 ? k : 1)));
    group_m = group_m < 4 ? 4 : group_m;
    kernel<<<grid, kNumThreads, Cfg::kSmemBytes, stream>>>(map_a, map_w, q.out, q.ldc, m, n, k, op.w_wrap_k, ep,
                                                           umma_idesc(1, 0, 0, kBlockM, BN), vec_ok, group_m,
                                                           dev.error_word);
    note_launch();
    return cuda_status(cudaGetLastError());
}


// CTA-pair launch: 256 x BN tiles, two CTAs per tile.  Returns NNB200_UNSUPPORTED when the device
// cannot co-schedule a single pair (the caller then uses the single-CTA form).
template <int BN, bool OUT_F16, int SUB, bool MC>
int launch_f16_pair_variant(const nnb200_q4_1_args& q, const F16Operands& op, const FpEpilogue& ep,
                            const DeviceInfo& dev, cudaStream_t stream)
{
    using Cfg = PairConfig<BN>;
    auto kernel = gemm_f16_umma_pair_kernel<BN, OUT_F16, SUB, MC>;
    static std::once_flag once[kMaxDevices];
    static cudaError_t attr_err[kMaxDevices];
    static int max_pairs[kMaxDevices];
    std::call_once(once[dev.device], [&] {
        attr_err[dev.device] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        max_pairs[dev.device] = 0;
        if (attr_err[dev.device] == cudaSuccess) {
            // How many clusters of two the device can hold at once with this kernel's resources.
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(static_cast<unsigned>(dev.sm_count & ~1));
            cfg.blockDim = dim3(kNumThreads);
            cfg.dynamicSmemBytes = Cfg::kSmemBytes;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) == cudaSuccess) {
                max_pairs[dev.device] = n;
            }
        }
    });
    if (attr_err[dev.device] != cudaSuccess) {
        return NNB200_INTERNAL;
    }
    if (max_pairs[dev.device] < 1) {
        return NNB200_UNSUPPORTED;
    }
    const int m = static_cast<int>(q.m), n = static_cast<int>(q.n), k = op.k_loop;
    CUtensorMap map_a, map_w;
    if (!make_tma_2d(&map_a, op.a, 2, static_cast<uint64_t>(op.k_loop), static_cast<uint64_t>(m),
                     static_cast<uint64_t>(op.lda) * 2, kBlockK, kBlockM) ||
        !make_tma_2d(&map_w, op.w, 2, static_cast<uint64_t>(op.k_w), static_cast<uint64_t>(n),
                     static_cast<uint64_t>(op.ldw) * 2, kBlockK, BN / 2)) {
        return NNB200_INTERNAL;
    }
    const int num_tiles = ((m + 2 * kBlockM - 1) / (2 * kBlockM)) * ((n + BN - 1) / BN);
    const int pairs = num_tiles < max_pairs[dev.device] ? num_tiles : max_pairs[dev.device];
    const int elem = OUT_F16 ? 2 : 4;
    // Destination vector stores: bit 0 = 16-byte aligned base and row pitch, bit 1 = 32-byte.
    const uint64_t out_pitch = static_cast<uint64_t>(q.ldc) * elem;
    const int vec_ok = (((reinterpret_cast<uintptr_t>(q.out) & 15u) == 0 && (out_pitch & 15u) == 0) ? 1 : 0) |
                       (((reinterpret_cast<uintptr_t>(q.out) & 31u) == 0 && (out_pitch & 31u) == 0) ? 2 : 0);
    int group_m = static_cast<int>((40ll << 20) / (static_cast<int64_t>(2 * kBlockM) * 2 * (k > 0 ? k : 1)));
    group_m = group_m < 2 ? 2 : group_m;
    kernel<<<2 * pairs, kNumThreads, Cfg::kSmemBytes, stream>>>(map_a, map_w, q.out, q.ldc, m, n, k, op.w_wrap_k, ep,
                                                               umma_idesc(1, 0, 0, 2 * kBlockM, BN), vec_ok, group_m,
                                                               dev.error_word);
    note_launch();
    return cuda_status(cudaGetLastError());
}

// Width of the output tile: 256 unless a narrower one saves more than 8 % of the padded work
// over whole waves (waves x width) -- about what a narrower tile loses in operand traffic per
// multiply-add.
int pick_bn(int m, int n, int sm_count)
{
    const int num_m = (m + kBlockM - 1) / kBlockM;
    const auto padded_work = [&](int width) {
        const int64_t tiles = static_cast<int64_t>(num_m) * ((n + width - 1) / width);
        return (tiles + sm_count - 1) / sm_count * width;
    };
    int best = 256;
    int64_t best_cost = padded_work(256);
    for (const int bn : {224, 192, 160, 128}) {
        if (padded_work(bn) * 100 < best_cost * 92) {
            best_cost = padded_work(bn);
            best = bn;
        }
    }
    return best;
}

}  // namespace

// Scratch the two-pass form needs: N rows of ceil(K/32)*32 halves for the expanded weights and, for
// f32 activations, M rows of 2 * kp halves (kp = K rounded up to 64) for their [hi | lo] split.
static size_t weights_scratch_bytes(const nnb200_q4_1_args& q)
{
    const int64_t nblk = (q.k + kQ4BlockElems - 1) / kQ4BlockElems;
    const size_t bytes = static_cast<size_t>(q.n) * static_cast<size_t>(nblk) * kQ4BlockElems * sizeof(__half);
    return (bytes + 255) & ~size_t(255);
}

size_t q4_1_two_pass_scratch_bytes(const nnb200_q4_1_args& q)
{
    size_t bytes = weights_scratch_bytes(q);
    if (q.a_f16 == 0) {
        const int64_t kp = (q.k + 63) / 64 * 64;
        bytes += static_cast<size_t>(q.m) * static_cast<size_t>(2 * kp) * sizeof(__half);
    }
    return bytes;
}

// Activations movable by TMA (f16: 16-byte aligned base and pitch; f32 ones are re-laid into the
// scratch), whole problem in 32-bit tile arithmetic, 4-byte aligned blocks, scratch 16-byte aligned.
bool q4_1_two_pass_supported(const nnb200_q4_1_args& q)
{
    const bool a_ok = q.a_f16 != 0 ? ((reinterpret_cast<uintptr_t>(q.a) & 15u) == 0 && ((q.lda * 2) & 15) == 0)
                                   : (reinterpret_cast<uintptr_t>(q.a) & 3u) == 0;
    return a_ok && q.m >= 1 && q.n >= 1 && q.k >= 1 && q.m <= INT32_MAX && q.n <= INT32_MAX &&
           q.k <= (INT32_MAX - 128) / 2 && q.lda >= q.k && (reinterpret_cast<uintptr_t>(q.w_blocks) & 3u) == 0 &&
           q.workspace != nullptr && (reinterpret_cast<uintptr_t>(q.workspace) & 15u) == 0 &&
           q.workspace_bytes >= q4_1_two_pass_scratch_bytes(q);
}

int launch_q4_1_two_pass(const nnb200_q4_1_args& q, const DeviceInfo& dev, cudaStream_t stream)
{
    FpEpilogue ep;
    ep.alpha = q.alpha;
    ep.bias = q.bias;
    ep.activation = q.activation;
    ep.act_alpha = q.act_alpha;
    ep.act_beta = q.act_beta;
    ep.min_clip = q.min_clip;
    ep.max_clip = q.max_clip;

    const int64_t nblk = (q.k + kQ4BlockElems - 1) / kQ4BlockElems;
    const int64_t ldw = nblk * kQ4BlockElems;
    __half* w_f16 = static_cast<__half*>(q.workspace);
    {
        // One CTA per pair of rows, capped at a few waves; the kernel strides.
        const int64_t want = (q.n + 1) / 2;
        const int64_t cap = static_cast<int64_t>(dev.sm_count) * 16;
        const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
        q4_1_expand_f16_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(q.w_blocks), q.ldw_blocks,
                                                         static_cast<const uint32_t*>(q.w_dm), q.ld_dm,
                                                         static_cast<int>(q.n), static_cast<int>(nblk), w_f16, ldw);
        note_launch();
        if (cudaGetLastError() != cudaSuccess) {
            return NNB200_INTERNAL;
        }
    }
    F16Operands op;
    op.w = w_f16;
    op.ldw = ldw;
    op.k_w = static_cast<int>(q.k);
    if (q.a_f16 != 0) {
        op.a = static_cast<const __half*>(q.a);
        op.lda = q.lda;
        op.k_loop = static_cast<int>(q.k);
        op.w_wrap_k = 0;
    } else {
        const int kp = static_cast<int>((q.k + 63) / 64 * 64);
        __half* a16 = reinterpret_cast<__half*>(static_cast<uint8_t*>(q.workspace) + weights_scratch_bytes(q));
        const int64_t total = q.m * kp;
        const int64_t want = (total + 255) / 256;
        const int64_t cap = static_cast<int64_t>(dev.sm_count) * 16;
        split_f32_to_f16_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, stream>>>(
            static_cast<const float*>(q.a), q.lda, static_cast<int>(q.m), static_cast<int>(q.k), kp, a16);
        note_launch();
        if (cudaGetLastError() != cudaSuccess) {
            return NNB200_INTERNAL;
        }
        op.a = a16;
        op.lda = 2 * static_cast<int64_t>(kp);
        op.k_loop = 2 * kp;
        op.w_wrap_k = kp;
    }
    // CTA-pair form (256-row tiles over two SMs) for tall problems: the default there.
    // Knob F16_PAIR: 0 = never; 2 = the pair form or an error; 1 / 3 = older forms kept for
    // comparison (one k-block per barrier slot; two k-blocks but one commit per destination CTA).
    const int pair_knob = knob(NNB200_KNOB_F16_PAIR);
    const char pair_mode = pair_knob == 0 ? '0' : (pair_knob == 2 ? '2' : '1');
    if (pair_mode != '0' && q.m >= 4 * kBlockM) {
        // Same width rule with 256-row tiles over sm_count / 2 pairs.
        const int bn2 = pick_bn((static_cast<int>(q.m) + 1) / 2, static_cast<int>(q.n), dev.sm_count / 2);
        int st = NNB200_UNSUPPORTED;
#define NNB200_F16_PAIR_LAUNCH_V(BNV, SUBV, MCV) \
    (q.out_f16 ? launch_f16_pair_variant<BNV, true, SUBV, MCV>(q, op, ep, dev, stream) \
               : launch_f16_pair_variant<BNV, false, SUBV, MCV>(q, op, ep, dev, stream))
#define NNB200_F16_PAIR_LAUNCH(BNV) \
    (pair_knob == 1 ? NNB200_F16_PAIR_LAUNCH_V(BNV, 1, false) \
     : pair_knob == 3 ? NNB200_F16_PAIR_LAUNCH_V(BNV, 2, false) : NNB200_F16_PAIR_LAUNCH_V(BNV, 2, true))
        if (bn2 >= 256) {
            st = NNB200_F16_PAIR_LAUNCH(256);
        } else if (bn2 >= 224) {
            st = NNB200_F16_PAIR_LAUNCH(224);
        } else {
            st = NNB200_F16_PAIR_LAUNCH(192);
        }
#undef NNB200_F16_PAIR_LAUNCH
#undef NNB200_F16_PAIR_LAUNCH_V
        if (st != NNB200_UNSUPPORTED || pair_mode == '2') {  // '2': the pair form or nothing
            return st;
        }
    }
    const int bn = pick_bn(static_cast<int>(q.m), static_cast<int>(q.n), dev.sm_count);
#define NNB200_F16_LAUNCH(BNV) \
    (q.out_f16 ? launch_f16_variant<BNV, true>(q, op, ep, dev, stream) \
               : launch_f16_variant<BNV, false>(q, op, ep, dev, stream))
    switch (bn) {
    case 256: return NNB200_F16_LAUNCH(256);
    case 224: return NNB200_F16_LAUNCH(224);
    case 192: return NNB200_F16_LAUNCH(192);
    case 160: return NNB200_F16_LAUNCH(160);
    default: return NNB200_F16_LAUNCH(128);
    }
#undef NNB200_F16_LAUNCH
}

}  // namespace nnb200
