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
// Same pipeline skeleton as the square engine (TMA warp, MMA warp, epilogue warps, two TMEM
// accumulators, bounded waits) except that each accumulator has its own four epilogue warps;
// same epilogue arithmetic (epilogue.cuh): results are bit-identical to every other int8 engine.
//
// Work split.  The unit of work is one 128-byte K block of one tile; tile t owns units
// [t * num_kb, (t + 1) * num_kb).  Every CTA takes one contiguous range of units:
//   * whole tiles only (CTA c gets tiles [c T / G, (c + 1) T / G)) when no scratch is given;
//   * an equal share of ALL units (CTA c gets [c U / G, (c + 1) U / G)) when the caller gave
//     scratch: a range then starts and ends in the middle of tiles, so that every SM streams
//     the same number of weight bytes whatever N / 128 is (224 tiles on 148 SMs would otherwise
//     run as two waves, the second half empty).  A CTA that holds only part of a tile's K range
//     writes its int32 partial sums to its own slot of the scratch and counts itself in on the
//     tile's counter; whichever warp counts in last adds the other parts to its own and runs
//     the epilogue.  Nobody waits for anybody, and integer addition makes the result
//     independent of who came last.  The protocol runs per warp (a warp owns 32 channels of the
//     tile in every CTA), so it needs no CTA-wide barrier.

#include <atomic>
#include <chrono>
#include <cstdlib>
#include <mutex>

#include "internal.cuh"
#include "ptx.cuh"

namespace nnb200 {

namespace {

constexpr int kBlockN = 128;       // channels per tile = rows of the MMA's 128-row operand
constexpr int kBlockKBytes = 128;  // one 128-byte swizzle row of K per stage
constexpr int kUmmaK = 32;
// TMA warp, MMA warp and two groups of four epilogue warps.  Group g drains accumulator g, i.e.
// every second piece of the CTA's range, so the drains (and, with shared K, the exchanges of
// partial sums, each a chain of L2 round trips) of consecutive pieces run side by side.
constexpr int kNumThreads = 320;
constexpr int kEpilogueThreads = 128;  // per group

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

// First unit of CTA c's range (c = G gives the end of the last range).
__device__ __forceinline__ int64_t range_begin(int c, int grid, int num_tiles, int num_kb, bool split)
{
    if (split) {
        return static_cast<int64_t>(c) * (static_cast<int64_t>(num_tiles) * num_kb) / grid;
    }
    return (static_cast<int64_t>(c) * num_tiles / grid) * num_kb;
}

// The CTA whose range contains unit u under the equal-share split.
__device__ __forceinline__ int cta_of_unit(int64_t u, int grid, int64_t total_units)
{
    return static_cast<int>(((u + 1) * grid - 1) / total_units);
}

// Bytes of the per-tile, per-warp arrival words at the head of the split scratch.
__host__ __device__ inline size_t split_counter_bytes(int num_tiles)
{
    return (static_cast<size_t>(num_tiles) * 4 * sizeof(unsigned long long) + 255) & ~size_t(255);
}

// One piece of a CTA's range: K blocks [kb0, kb1) of `tile`.
struct Segment {
    int tile, kb0, kb1;
};

// A CTA's range [u_begin, u_end) cut at tile boundaries, in the order it is worked through:
// the part of a tile that somebody else started (head), the part of a tile that somebody else
// finishes (tail), then the whole tiles.  Parts go first so that they are published early and
// the exchange with the neighbours hides behind the whole tiles that follow.
struct SegmentList {
    int64_t head0, head1, tail0, tail1;
    int tile0, tile1;
    int num_kb;

    __device__ __forceinline__ SegmentList(int64_t u_begin, int64_t u_end, int nkb) : num_kb(nkb)
    {
        const int64_t first_full = (u_begin + nkb - 1) / nkb * nkb;
        const int64_t last_full_end = u_end / nkb * nkb;
        head0 = u_begin;
        head1 = first_full < u_end ? first_full : u_end;
        if (last_full_end >= first_full && last_full_end < u_end) {
            tail0 = last_full_end;
            tail1 = u_end;
        } else {
            tail0 = tail1 = 0;
        }
        tile0 = static_cast<int>(first_full / nkb);
        tile1 = last_full_end > first_full ? static_cast<int>(last_full_end / nkb) : tile0;
    }
    __device__ __forceinline__ int count() const
    {
        return (head1 > head0 ? 1 : 0) + (tail1 > tail0 ? 1 : 0) + (tile1 - tile0);
    }
    __device__ __forceinline__ Segment at(int i) const
    {
        Segment s;
        if (head1 > head0) {
            if (i == 0) {
                s.tile = static_cast<int>(head0 / num_kb);
                s.kb0 = static_cast<int>(head0 - static_cast<int64_t>(s.tile) * num_kb);
                s.kb1 = s.kb0 + static_cast<int>(head1 - head0);
                return s;
            }
            --i;
        }
        if (tail1 > tail0) {
            if (i == 0) {
                s.tile = static_cast<int>(tail0 / num_kb);
                s.kb0 = 0;
                s.kb1 = static_cast<int>(tail1 - tail0);
                return s;
            }
            --i;
        }
        s.tile = tile0 + i;
        s.kb0 = 0;
        s.kb1 = num_kb;
        return s;
    }
};

// Arrival words.  The scratch arrives with arbitrary contents and nothing clears it: a word is
// (call tag << 8) | count, the tag unique to this launch, and a word carrying any other tag
// counts as zero.  The warp that finishes a tile writes (tag << 8) | 0 back, so that a replay of
// a captured launch -- same tag -- starts from zero as well.
__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long* p)
{
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ int arrivals_of(unsigned long long word, unsigned long long tag)
{
    return (word >> 8) == tag ? static_cast<int>(word & 0xFFu) : 0;
}

// Count this part in, starting from the word as last seen; returns how many parts had arrived
// before it (-1 if the bounded retry ran out).
__device__ __forceinline__ int arrive(unsigned long long* p, unsigned long long tag, unsigned long long old)
{
    for (int tries = 0; tries < 1024; ++tries) {
        const int before = arrivals_of(old, tag);
        const unsigned long long prev = atomicCAS(p, old, (tag << 8) | static_cast<unsigned long long>(before + 1));
        if (prev == old) {
            return before;
        }
        old = prev;
    }
    return -1;
}

// Sum over the other CTAs' published parts of one tile, rows [row0, row0 + 32) of this thread's
// channel.  All loads of a part are issued before any is used: one L2 round trip per part.
__device__ __forceinline__ void collect_parts(int32_t (&sum)[32], const int32_t* split_slots, size_t slot_elems, int ch,
                                              int first_cta, int last_cta, int self, int row0, int m_total)
{
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        sum[j] = 0;
    }
    for (int other = first_cta; other <= last_cta; ++other) {
        if (other == self) {
            continue;
        }
        const int32_t* theirs = split_slots + (2 * static_cast<size_t>(other) + (other == first_cta ? 1u : 0u)) * slot_elems + ch;
        int32_t part[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            part[j] = (row0 + j < m_total) ? __ldcg(theirs + static_cast<size_t>(row0 + j) * kBlockN) : 0;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            sum[j] += part[j];
        }
    }
}

template <int MP, int KIND>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_i8_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                      const I8Epilogue ep, const int m_total, const int n_total, const int k_total,
                      const uint32_t idesc, int32_t* error_word, unsigned long long* split_counters,
                      int32_t* split_slots, const unsigned long long split_tag)
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
    const bool split = split_counters != nullptr;
    const int grid = static_cast<int>(gridDim.x);
    const int64_t u_begin = range_begin(static_cast<int>(blockIdx.x), grid, num_tiles, num_kb, split);
    const int64_t u_end = range_begin(static_cast<int>(blockIdx.x) + 1, grid, num_tiles, num_kb, split);
    const SegmentList segments(u_begin, u_end, num_kb);
    const int num_segments = segments.count();

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
            for (int si = 0; ok && si < num_segments; ++si) {
                const Segment seg = segments.at(si);
                const int tile = seg.tile;
                for (int kb = seg.kb0; kb < seg.kb1; ++kb) {
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
            int local_seg = 0;
            bool ok = true;
            for (; ok && local_seg < num_segments; ++local_seg) {
                const Segment seg = segments.at(local_seg);
                const int acc = local_seg & 1;
                const uint32_t acc_phase = (local_seg >> 1) & 1u;
                if (!mbar_wait(&acc_empty_bar[acc], acc_phase ^ 1u, abort_flag)) {
                    atomicCAS(error_word, 0, kErrAccumWait);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * MP);
                for (int kb = seg.kb0; kb < seg.kb1; ++kb) {
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
                                idesc, (kb > seg.kb0 || ks > 0) ? 1u : 0u);
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
        const int ch = quarter * 32 + lane;  // this thread's channel within the tile
        const int64_t total_units = static_cast<int64_t>(num_tiles) * num_kb;
        const size_t slot_elems = static_cast<size_t>(kBlockN) * static_cast<size_t>(m_total);
        const int group = (warp - 2) >> 2;
        int local_seg = group;
        for (; local_seg < num_segments; local_seg += 2) {
            const Segment seg = segments.at(local_seg);
            const int tile = seg.tile;
            const int acc = local_seg & 1;
            const uint32_t acc_phase = (local_seg >> 1) & 1u;
            const bool partial = seg.kb0 != 0 || seg.kb1 != num_kb;  // only under the equal-share split
            const int64_t n = static_cast<int64_t>(tile) * kBlockN + ch;
            const bool n_ok = n < n_total;
            // This channel's terms, in registers for the whole tile.
            const int32_t zpw = (n_ok && ep.zp_w != nullptr) ? ep.zp_w[n] : ep.zp_w_scalar;
            const int32_t rw = (n_ok && ep.compensate && ep.r_w != nullptr) ? ep.r_w[n] : 0;
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

            // Part of a tile.  While this piece's MMAs are still running, look whether everybody else
            // has published already; if so this warp will finish the tile and fetches the others'
            // sums for the first 32 rows now, off the critical path.
            int first_cta = 0, last_cta = -1;
            bool early = false;
            int32_t early_sum[32];
            if (partial) {
                first_cta = cta_of_unit(static_cast<int64_t>(tile) * num_kb, grid, total_units);
                last_cta = cta_of_unit(static_cast<int64_t>(tile + 1) * num_kb - 1, grid, total_units);
                int seen = 0;
                if (MP == 32 && lane == 0) {
                    seen = arrivals_of(ld_acquire_gpu_u64(&split_counters[tile * 4 + quarter]), split_tag);
                }
                seen = __shfl_sync(0xFFFFFFFFu, seen, 0);
                // Only where 32 rows are all there is: with more rows the early fetch covers a part of
                // the work and measured slower than none.
                early = MP == 32 && seen == last_cta - first_cta;
                if (early) {
                    __threadfence();  // every lane's reads of the others' slots come after lane 0's look
                    collect_parts(early_sum, split_slots, slot_elems, ch, first_cta, last_cta, static_cast<int>(blockIdx.x),
                                  0, m_total);
                }
            }

            if (!mbar_wait_warp(&acc_full_bar[acc], acc_phase, abort_flag)) {
                atomicCAS(error_word, 0, kErrEpilogueWait);
                break;
            }
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(acc * MP);
            // Otherwise: publish this warp's 32 channels, count in, and carry on only if every other
            // part of the tile has been published by then.
            bool finish = true;
            bool publish = partial && !early;
            unsigned long long seen_word = 0;  // lane 0's last look at the tile's arrival word
            if (publish) {
                // Everybody else in by now?  Then this warp finishes the tile and has nothing to publish.
                int seen = 0;
                if (lane == 0) {
                    seen_word = ld_acquire_gpu_u64(&split_counters[tile * 4 + quarter]);
                    seen = arrivals_of(seen_word, split_tag);
                }
                seen = __shfl_sync(0xFFFFFFFFu, seen, 0);
                publish = seen != last_cta - first_cta;
                if (!publish) {
                    __threadfence();  // every lane's reads of the others' slots come after lane 0's look
                }
            }
            if (publish) {
                int32_t* mine = split_slots +
                                (2 * static_cast<size_t>(blockIdx.x) + (seg.kb0 == 0 ? 1u : 0u)) * slot_elems + ch;
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
                        if (c * 32 + j < m_total) {
                            __stcg(mine + static_cast<size_t>(c * 32 + j) * kBlockN, static_cast<int32_t>(v[j]));
                        }
                    }
                }
                __threadfence();
                __syncwarp();
                int ticket = 0;
                if (lane == 0) {
                    ticket = arrive(&split_counters[tile * 4 + quarter], split_tag, seen_word);
                }
                ticket = __shfl_sync(0xFFFFFFFFu, ticket, 0);
                if (ticket < 0) {
                    atomicCAS(error_word, 0, kErrEpilogueWait);  // cannot happen with at most 148 parts per word
                }
                finish = ticket == last_cta - first_cta;
                if (finish) {
                    __threadfence();
                }
            }
            if (partial && finish && lane == 0) {
                split_counters[tile * 4 + quarter] = split_tag << 8;  // nobody else touches it in this launch
            }
#pragma unroll 1
            for (int c = 0; c < MP / 32; ++c) {
                if (c * 32 >= m_total || !finish) {
                    break;  // uniform
                }
                uint32_t v[32];
                tmem_ld_32x32(t_row + static_cast<uint32_t>(c * 32), v);
                tmem_ld_wait();
                if (partial) {
                    if (!(early && c == 0)) {
                        collect_parts(early_sum, split_slots, slot_elems, ch, first_cta, last_cta,
                                      static_cast<int>(blockIdx.x), c * 32, m_total);
                    }
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        v[j] += static_cast<uint32_t>(early_sum[j]);
                    }
                }
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

// A 56-bit tag no earlier launch of this process has used, never zero; the sequence starts at
// a point derived from the clock so that words left in recycled memory by another process do
// not match either.
unsigned long long next_split_tag()
{
    static std::atomic<unsigned long long> counter{
        static_cast<unsigned long long>(std::chrono::steady_clock::now().time_since_epoch().count()) * 0x9E3779B97F4A7C15ull};
    unsigned long long t;
    do {
        t = counter.fetch_add(1, std::memory_order_relaxed) & ((1ull << 56) - 1);
    } while (t == 0);
    return t;
}

template <int MP, int KIND>
int launch_skinny_variant(const I8Problem& p, const I8Epilogue& ep, const DeviceInfo& dev, void* split_scratch,
                          cudaStream_t stream)
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
    int grid = num_tiles < dev.sm_count ? num_tiles : dev.sm_count;
    unsigned long long* counters = nullptr;
    int32_t* slots = nullptr;
    unsigned long long tag = 0;
    if (split_scratch != nullptr) {
        // Equal shares of all K blocks over every SM.
        grid = dev.sm_count;
        counters = static_cast<unsigned long long*>(split_scratch);
        slots = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(split_scratch) + split_counter_bytes(num_tiles));
        tag = next_split_tag();
    }
    // 128-row operand = weights (s8), N operand = activations (s8 or u8).
    const uint32_t idesc = umma_idesc(2, 1, p.a_unsigned ? 0u : 1u, kBlockN, MP);
    kernel<<<grid, kNumThreads, Cfg::kSmemBytes, stream>>>(map_w, map_a, ep, m, n, k, idesc, dev.error_word, counters,
                                                             slots, tag);
    note_launch();
    return cuda_status(cudaGetLastError());
}

template <int MP>
int launch_skinny_mp(const I8Problem& p, const I8Epilogue& ep, const DeviceInfo& dev, void* split_scratch,
                     cudaStream_t stream)
{
    switch (ep.out_kind) {
    case NNB200_OUT_S32: return launch_skinny_variant<MP, NNB200_OUT_S32>(p, ep, dev, split_scratch, stream);
    case NNB200_OUT_S8: return launch_skinny_variant<MP, NNB200_OUT_S8>(p, ep, dev, split_scratch, stream);
    case NNB200_OUT_U8: return launch_skinny_variant<MP, NNB200_OUT_U8>(p, ep, dev, split_scratch, stream);
    case NNB200_OUT_F32: return launch_skinny_variant<MP, NNB200_OUT_F32>(p, ep, dev, split_scratch, stream);
    case NNB200_OUT_F16: return launch_skinny_variant<MP, NNB200_OUT_F16>(p, ep, dev, split_scratch, stream);
    default: return NNB200_UNSUPPORTED;
    }
}

}  // namespace

// Same operand rules as the square tensor-core engine, at most 128 activation rows.
bool skinny_i8_supported(const I8Problem& p)
{
    return p.m >= 1 && p.m <= 128 && umma_i8_supported(p);
}

// Scratch for the equal-share split of K over all SMs, or 0 when it would not pay.  Publishing a
// part, counting in and collecting the others' parts is a chain of L2 round trips at the end of
// the kernel, each well over a microsecond while every SM is streaming: about 6 us in all plus
// ~0.1 us per activation row, against ~0.3 us per 128-byte K block that the busiest CTA no longer
// has to stream.  Measured, 24 rows, whole tiles -> shared K (us):
//   one wave of tiles:  N=4096,K=28672 70.1 -> 31.6;  N=4096,K=14336 38.5 -> 22.2;  N=8192,K=8192
//   25.3 -> 22.2;  N=14336,K=8192 28.1 -> 29.5;  N=11008,K=4096 16.5 -> 18.3;
//   two waves, the second half empty:  N=28672,K=8192 52.0 -> 47.6 (48 rows 54.9 -> 51.8).
// Hence: with one wave, share when the busiest CTA sheds at least 30 K blocks, plus 0.7 per row
// above 12; with several waves, when the last one is less than 9/10 full, a share is at least 48
// K blocks and there are at most 64 rows.
// Knob I8_SHARE_K = 0 turns the split off; 2 offers it from 8 K blocks per SM (measurement, tests).
size_t skinny_i8_split_bytes(const I8Problem& p, const DeviceInfo& dev)
{
    if (!skinny_i8_supported(p)) {
        return 0;
    }
    const int share_knob = knob(NNB200_KNOB_I8_SHARE_K);
    const char mode = share_knob < 0 ? '1' : static_cast<char>('0' + (share_knob > 2 ? 1 : share_knob));
    if (mode == '0') {
        return 0;
    }
    const int64_t tiles = (p.n + kBlockN - 1) / kBlockN;
    const int64_t num_kb = (p.k + kBlockKBytes - 1) / kBlockKBytes;
    const int64_t sms = dev.sm_count;
    const int64_t waves = (tiles + sms - 1) / sms;
    const int64_t share = (tiles * num_kb + sms - 1) / sms;
    if (tiles * 10 >= waves * sms * 9 || share < 8) {
        return 0;  // whole tiles already fill the SMs, or there is next to nothing to share
    }
    if (mode != '2') {
        if (waves == 1) {
            const int64_t rows_over = p.m > 12 ? p.m - 12 : 0;
            if ((num_kb - share) * 10 < 300 + 7 * rows_over) {
                return 0;
            }
        } else if (share < 48 || p.m > 64) {
            return 0;
        }
    }
    // Two slots per CTA (the tile it finishes for someone and the tile it leaves to someone),
    // each 128 channels x m int32.
    return split_counter_bytes(static_cast<int>(tiles)) +
           2 * static_cast<size_t>(sms) * kBlockN * static_cast<size_t>(p.m) * sizeof(int32_t);
}

int launch_gemm_i8_skinny(const I8Problem& p, const I8Epilogue& ep, const DeviceInfo& dev, void* split_scratch,
                          cudaStream_t stream)
{
    if (p.m <= 32) {
        return launch_skinny_mp<32>(p, ep, dev, split_scratch, stream);
    }
    if (p.m <= 64) {
        return launch_skinny_mp<64>(p, ep, dev, split_scratch, stream);
    }
    return launch_skinny_mp<128>(p, ep, dev, split_scratch, stream);
}

}  // namespace nnb200
