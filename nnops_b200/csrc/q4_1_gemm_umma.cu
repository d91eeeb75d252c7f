// Q4_1 weight-decode GEMM for prefill-sized M on sm_100a:
//   out[M,N] = act(alpha * A[M,K] (f16) * dequant(W)[N,K]^T + bias), f32 accumulation.
//
// The reference only has a CPU route for this (decode W into dense f16 panels, then a dense
// MMA: FpRoute::pack_b -> pack_q4_1_rhs, src/backend/cpu/matmul/matmul.cpp:137-156,
// src/backend/cpu/x86_64/pack_q4_1.hpp:225-254).  Here the decode is fused into the operand
// staging of a tcgen05 pipeline, so the 4.5-bit weight stream is all that ever leaves HBM:
//
//   * warp 0 TMA-loads 128 x 64 f16 activation tiles (128-byte swizzle) into a ring;
//   * 16 dequant warps fetch the RAW Q4_1 stream themselves, 128 k (4 blocks = 80 B per row) at
//     a time: coalesced 16-byte global loads issued one step ahead, parked in a double-buffered
//     shared tile, then each lane picks up "its" block -- lane (g, c) of warp w owns block c of
//     row 8w+g, a mapping whose 32-bit shared reads are bank-conflict free (20g + 5c + i is a
//     bijection mod 32).  (TMA was measured first for this stream: with 80-byte box rows it
//     sustained only about one row per 17 clocks per SM and capped the whole kernel.)  Rows that
//     cannot be read 16 bytes at a time (base or pitch unaligned) are read by each lane directly;
//   * the lanes expand the nibbles to f16 with integer tricks
//     (nibble | 0x6400 = 1024 + q exactly, minus 1024, then one hfma2 q*d + m -- a single f16
//     rounding per weight, which is what the reference's f16 route stores), and write them
//     into the ring in the same K-major 128-byte-swizzled layout TMA would have produced;
//   * warp 1 issues tcgen05.mma kind::f16 (M128 x N128 x K16, twice per k-step when the tile
//     stacks two 128-row activation halves over one weight tile) into one of two TMEM
//     accumulator sets; warps 2-5 drain the other and apply alpha / bias / clip / activation.
//
// Every wait is bounded (see ptx.cuh).

#include <cstring>
#include <mutex>

#include "internal.cuh"
#include "ptx.cuh"
#include "q4_1_common.cuh"

namespace nnb200 {

namespace {

constexpr int kHalfM = 128;  // rows per UMMA instruction; a tile stacks MH of them over one weight tile
constexpr int kBlockK = 64;  // halves per stage = one 128-byte swizzle row = two Q4_1 blocks
constexpr int kUmmaKBytes = 32;
constexpr int kGroupM = 8;

constexpr int kRawRowBytes = 4 * kQ4BlockBytes;  // 80 B: the four blocks of one row in a 128-k super-step
constexpr int kDequantWarps = 16;                // 8 rows x 4 blocks per warp
constexpr int kDequantThreads = kDequantWarps * 32;
constexpr int kTileN = 128;                      // weight rows per tile = kDequantWarps * 8
constexpr int kRawAhead = 2;                     // super-steps of raw weights in flight (cp.async)
constexpr int kRawBufs = kRawAhead + 1;          // ring of raw tiles in shared memory

template <bool COOP, int MH>
struct Q4Config {
    static constexpr int kBlockM = kHalfM * MH;
    static constexpr int kATileBytes = kBlockM * kBlockK * 2;
    static constexpr int kBTileBytes = kTileN * kBlockK * 2;
    static constexpr int kStageBytes = kATileBytes + kBTileBytes;
    static constexpr int kRawBufBytes = kTileN * kRawRowBytes;     // 10 240 B
    static constexpr int kRawBytes = COOP ? kRawBufs * kRawBufBytes : 0;
    static constexpr int kStages = (MH == 2) ? 4 : 6;
    static constexpr int kNumThreads = (6 + kDequantWarps) * 32;
    static constexpr int kTmemCols = 2 * MH * kTileN;  // two accumulator sets of MH x 128 columns
    static constexpr int kBarrierBytes = (3 * kStages + 4) * 8 + 16;
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

template <bool OUT_F16, bool COOP, int MH>
__global__ void __launch_bounds__(Q4Config<COOP, MH>::kNumThreads, 1)
q4_1_gemm_umma_kernel(const __grid_constant__ CUtensorMap map_a, const uint8_t* __restrict__ w,
                      const int64_t ldw_blocks, void* __restrict__ out, const int64_t ldc, const int m_total,
                      const int n_total, const int k_total, const FpEpilogue ep, const uint32_t idesc,
                      const int vec_ok, int32_t* error_word)
{
    using Cfg = Q4Config<COOP, MH>;
    constexpr int BN = kTileN;
    constexpr int kStages = Cfg::kStages;
    constexpr int kBlockM = Cfg::kBlockM;
    static_assert(Cfg::kTmemCols <= 512, "accumulators exceed TMEM");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stage_base = smem;
    uint8_t* raw_base = smem + kStages * Cfg::kStageBytes;  // two raw-block tiles (COOP only)
    uint64_t* a_full_bar = reinterpret_cast<uint64_t*>(raw_base + Cfg::kRawBytes);
    uint64_t* b_full_bar = a_full_bar + kStages;
    uint64_t* empty_bar = b_full_bar + kStages;
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
    const int nblk = (k_total + kQ4BlockElems - 1) / kQ4BlockElems;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&a_full_bar[s], 1);
            mbar_init(&b_full_bar[s], kDequantWarps);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full_bar[a], 1);
            mbar_init(&acc_empty_bar[a], 4);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&map_a);
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
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                const TileCoord tc = tile_coord(tile, num_m, num_n);
                for (int kb = 0; kb < num_kb; ++kb) {
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
                // Copies already issued still land in shared memory: wait (bounded) for them.
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
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * MH * BN);
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
#pragma unroll
                        for (int h = 0; h < MH; ++h) {
                            // Each 128-row half of the activation tile meets the same dequantised weights.
                            umma_f16(d_tmem + static_cast<uint32_t>(h * BN),
                                     a_desc + static_cast<uint64_t>(h * ((kHalfM * kBlockK * 2) >> 4) + ks * 2),
                                     b_desc + static_cast<uint64_t>(ks * 2), idesc, (kb > 0 || ks > 0) ? 1u : 0u);
                        }
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
        const bool identity = fp_epilogue_is_identity(ep);
        int local_tile = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local_tile) {
            const TileCoord tc = tile_coord(tile, num_m, num_n);
            const int acc = local_tile & 1;
            const uint32_t acc_phase = (local_tile >> 1) & 1u;
            const int n_base = tc.n_blk * BN;

            // Warp-uniform outcome, so no lane is left behind at a later warp sync.
            if (!mbar_wait_warp(&acc_full_bar[acc], acc_phase, abort_flag)) {
                atomicCAS(error_word, 0, kErrEpilogueWait);
                break;
            }
            tc_fence_after_sync();
#pragma unroll 1
            for (int hc = 0; hc < MH * (BN / 32); ++hc) {
                const int h = hc / (BN / 32);
                const int c = hc % (BN / 32);
                const int64_t m = static_cast<int64_t>(tc.m_blk) * kBlockM + h * kHalfM + quarter * 32 + lane;
                const bool row_ok = m < m_total;
                const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       static_cast<uint32_t>(acc * MH * BN + h * BN);
                const int n0 = n_base + c * 32;
                if (n0 >= n_total) {
                    continue;  // warp-uniform
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
                    fp_epilogue_chunk<false>(ep, identity, v, n0, n_total, o);
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
        // Work unit: one Q4_1 block (32 k) of one weight row per super-step of 128 k.  Lane (g, c)
        // of dequant warp dw owns block c of row 8*dw + g; blocks 0,1 fall in the even k-step of
        // the super-step, blocks 2,3 in the odd one.
        const int dw = warp - 6;
        const int dt = dw * 32 + lane;                // 0..511
        const int g = lane >> 2;
        const int c = lane & 3;
        const int parity = c >> 1;                    // which of the two k-steps this lane feeds
        const int jblk = c & 1;                       // first or second block of that k-step
        const int r = dw * 8 + g;                     // weight row inside the tile
        const int sw = r & 7;
        const int my_tiles = (num_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                             static_cast<int>(gridDim.x);
        const int num_ss = (num_kb + 1) / 2;
        const int total_q = my_tiles * num_ss;        // super-steps this CTA walks through
        const int64_t pitch = ldw_blocks * kQ4BlockBytes;

        // First weight row of local tile t.
        auto tile_row0 = [&](int t) {
            const int tile = static_cast<int>(blockIdx.x) + t * static_cast<int>(gridDim.x);
            return static_cast<int64_t>(tile_coord(tile, num_m, num_n).n_blk) * BN;
        };

        // COOP: the raw tile of a super-step is 128 rows x 80 B = 640 pieces of 16 B; thread dt
        // copies piece dt and (dt < 128) piece 512 + dt with cp.async, kRawAhead super-steps ahead,
        // into a ring of kRawBufs tiles.  Pieces past N or past the row end arrive as zeros.
        // Everything that does not change from one super-step to the next is computed here once.
        const int64_t row_bytes = static_cast<int64_t>(nblk) * kQ4BlockBytes;
        const int p_row[2] = {dt / 5, (512 + dt) / 5};
        const int p_off[2] = {(dt % 5) * 16, ((512 + dt) % 5) * 16};
        const int p_count = dt < 128 ? 2 : 1;
        int pf_t = 0, pf_ss = 0, pf_buf = 0;        // prefetch cursor: local tile, super-step, ring slot
        int64_t pf_row0 = my_tiles > 0 ? tile_row0(0) : 0;
        auto issue_super_step = [&]() {
            if (pf_t < my_tiles) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    if (i < p_count) {
                        const int64_t n = pf_row0 + p_row[i];
                        const int64_t byte0 = static_cast<int64_t>(pf_ss) * kRawRowBytes + p_off[i];
                        int64_t valid = n < n_total ? row_bytes - byte0 : 0;
                        valid = valid < 0 ? 0 : (valid > 16 ? 16 : valid);
                        const uint8_t* src = valid > 0 ? w + n * pitch + byte0 : w;
                        cp_async_16(raw_base + pf_buf * Cfg::kRawBufBytes + (i == 0 ? dt : 512 + dt) * 16, src,
                                    static_cast<uint32_t>(valid));
                    }
                }
                if (++pf_ss == num_ss) {
                    pf_ss = 0;
                    if (++pf_t < my_tiles) {
                        pf_row0 = tile_row0(pf_t);
                    }
                }
            }
            pf_buf = pf_buf + 1 == kRawBufs ? 0 : pf_buf + 1;
            cp_async_commit();  // one group per super-step, empty ones included, so the counts line up
        };
        // Plain path: this lane's own block, five 32-bit loads.
        uint32_t next[5] = {0u, 0u, 0u, 0u, 0u};
        auto fetch_block = [&](int q) {
            const int64_t n = tile_row0(q / num_ss) + r;
            const int b = (q % num_ss) * 4 + c;
            if (n < n_total && b < nblk) {
                const uint32_t* src = reinterpret_cast<const uint32_t*>(w + n * pitch + static_cast<int64_t>(b) * kQ4BlockBytes);
#pragma unroll
                for (int i = 0; i < 5; ++i) {
                    next[i] = __ldg(src + i);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 5; ++i) {
                    next[i] = 0u;
                }
            }
        };

        if (total_q > 0) {
            if constexpr (COOP) {
                for (int q0 = 0; q0 < kRawAhead; ++q0) {
                    issue_super_step();
                }
            } else {
                fetch_block(0);
            }
        }
        int kcount = 0;     // k-steps this CTA has gone through before the current super-step
        bool dead = false;  // a wait ran out: keep walking (the barriers below need every warp) but do nothing
        int cur_buf = 0;    // ring slot of super-step q
        int ss = 0;         // super-step inside the current tile
        int stage_e = 0;    // ring stage of k-step `kcount`
        uint32_t phase_e = 0;
        for (int q = 0; q < total_q; ++q) {
            uint32_t raw[5];
            if constexpr (COOP) {
                uint8_t* buf = raw_base + cur_buf * Cfg::kRawBufBytes;
                cur_buf = cur_buf + 1 == kRawBufs ? 0 : cur_buf + 1;
                // Slot (q + kRawAhead) % kRawBufs was last read in super-step q - 1, which every warp
                // finished before passing that step's barrier... except the readers still inside
                // step q - 1 right now; the barrier below is what orders them, so the refill is
                // issued after it.
                cp_async_wait_group<kRawAhead - 1>();   // this thread's pieces of super-step q have landed
                named_barrier_sync(1, kDequantThreads); // ... and everyone else's; step q - 1 is fully read
                issue_super_step();
                const uint32_t* src = reinterpret_cast<const uint32_t*>(buf + r * kRawRowBytes) + c * kQ4BlockWords;
#pragma unroll
                for (int i = 0; i < 5; ++i) {
                    raw[i] = src[i];
                }
            } else {
#pragma unroll
                for (int i = 0; i < 5; ++i) {
                    raw[i] = next[i];
                }
                if (q + 1 < total_q) {
                    fetch_block(q + 1);
                }
            }
            const int steps_here = min(2, num_kb - 2 * ss);
            if (++ss == num_ss) {
                ss = 0;
            }
            const int stage_o = stage_e + 1 == kStages ? 0 : stage_e + 1;
            const uint32_t phase_o = stage_e + 1 == kStages ? phase_e ^ 1u : phase_e;
            // Decode BEFORE asking for the ring slots: the wait below then only gates four shared
            // stores, which keeps the slot's turnaround (free -> refilled) short.
            const uint32_t dm = raw[0];
            const __half2 d2 = __half2half2(__ushort_as_half(static_cast<uint16_t>(dm & 0xFFFFu)));
            const __half2 m2 = __half2half2(__ushort_as_half(static_cast<uint16_t>(dm >> 16)));
            uint4 lo0, hi0, lo1, hi1;
            dequant_word_pair(raw[1], raw[2], d2, m2, lo0, hi0);  // k 0..7 and 16..23 of the block
            dequant_word_pair(raw[3], raw[4], d2, m2, lo1, hi1);  // k 8..15 and 24..31
            if (!dead) {
                bool ok = mbar_wait_warp(&empty_bar[stage_e], phase_e ^ 1u, abort_flag);
                if (steps_here == 2) {
                    ok = mbar_wait_warp(&empty_bar[stage_o], phase_o ^ 1u, abort_flag) && ok;
                }
                if (!ok) {
                    atomicCAS(error_word, 0, kErrDequantWait);
                    dead = true;
                }
            }
            if (!dead) {
                if (parity < steps_here) {
                    const int stage = parity == 0 ? stage_e : stage_o;
                    uint8_t* b_row = stage_base + stage * Cfg::kStageBytes + Cfg::kATileBytes + r * 128;
                    // 16-byte chunk ch of the row lives at chunk (ch ^ (row & 7)): the 128-byte swizzle.
                    *reinterpret_cast<uint4*>(b_row + (((4 * jblk + 0) ^ sw) << 4)) = lo0;
                    *reinterpret_cast<uint4*>(b_row + (((4 * jblk + 1) ^ sw) << 4)) = lo1;
                    *reinterpret_cast<uint4*>(b_row + (((4 * jblk + 2) ^ sw) << 4)) = hi0;
                    *reinterpret_cast<uint4*>(b_row + (((4 * jblk + 3) ^ sw) << 4)) = hi1;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&b_full_bar[stage_e]);
                    if (steps_here == 2) {
                        mbar_arrive(&b_full_bar[stage_o]);
                    }
                }
            }
            kcount += steps_here;
            for (int adv = 0; adv < steps_here; ++adv) {
                if (++stage_e == kStages) {
                    stage_e = 0;
                    phase_e ^= 1u;
                }
            }
        }
        (void)kcount;
    }

    // ---------------- teardown ----------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

template <bool OUT_F16, bool COOP, int MH>
int launch_variant(const nnb200_q4_1_args& q, const CUtensorMap& map_a, const FpEpilogue& ep, const DeviceInfo& dev,
                   cudaStream_t stream)
{
    using Cfg = Q4Config<COOP, MH>;
    constexpr int kBlockM = Cfg::kBlockM;
    auto kernel = q4_1_gemm_umma_kernel<OUT_F16, COOP, MH>;
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
    const int num_tiles = ((m + kBlockM - 1) / kBlockM) * ((n + kTileN - 1) / kTileN);
    const int grid = num_tiles < dev.sm_count ? num_tiles : dev.sm_count;
    const int elem = OUT_F16 ? 2 : 4;
    const int vec_ok = ((reinterpret_cast<uintptr_t>(q.out) & 15u) == 0 &&
                        ((static_cast<uint64_t>(q.ldc) * elem) & 15u) == 0)
                           ? 1
                           : 0;
    kernel<<<grid, Cfg::kNumThreads, Cfg::kSmemBytes, stream>>>(
        map_a, static_cast<const uint8_t*>(q.w_blocks), q.ldw_blocks, q.out, q.ldc, m, n, k, ep,
        umma_idesc(1, 0, 0, kHalfM, kTileN), vec_ok, dev.error_word);
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

    // Tile shape.  Tall problems stack two 128-row activation halves over one 128-channel
    // weight tile (256 x 128): every dequantised weight then feeds twice the math.  Otherwise
    // 128 x 128.
    const int64_t tiles_tall = ((q.m + 255) / 256) * ((q.n + kTileN - 1) / kTileN);
    const bool tall = q.m >= 256 && tiles_tall >= dev.sm_count;
    const int block_m = tall ? 256 : 128;

    CUtensorMap map_a;
    if (!make_tma_2d(&map_a, q.a, 2, static_cast<uint64_t>(q.k), static_cast<uint64_t>(q.m),
                     static_cast<uint64_t>(q.lda) * 2, kBlockK, static_cast<uint32_t>(block_m))) {
        return NNB200_INTERNAL;
    }
    // 16-byte cooperative loads of the raw stream need 16-byte aligned rows.
    const bool coop = (reinterpret_cast<uintptr_t>(q.w_blocks) & 15u) == 0 && (q.ldw_blocks % 4) == 0;
#define NNB200_Q4_LAUNCH(F16V, MHV)                                                   \
    (coop ? launch_variant<F16V, true, MHV>(q, map_a, ep, dev, stream)                \
          : launch_variant<F16V, false, MHV>(q, map_a, ep, dev, stream))
    if (tall) {
        return q.out_f16 ? NNB200_Q4_LAUNCH(true, 2) : NNB200_Q4_LAUNCH(false, 2);
    }
    return q.out_f16 ? NNB200_Q4_LAUNCH(true, 1) : NNB200_Q4_LAUNCH(false, 1);
#undef NNB200_Q4_LAUNCH
}

}  // namespace nnb200
