// Q4_1 decode GEMV, bandwidth-optimised form (f16 activations, M <= 8 per pass).
//
// Why warp-level MMA in a "bandwidth kernel": at the HBM rate a B200 SM must retire ~36
// weights per clock.  On CUDA cores every weight costs an int->float conversion plus one FMA
// per activation row, i.e. 3+M instructions per weight against a budget of ~3.5 issue slots,
// so M = 8 cannot reach the roofline and M = 1 only barely.  mma.sync.m16n8k16 takes 16 weight
// rows x 16 k per instruction with the (up to 8) activation rows as its n dimension, which
// leaves only the nibble->f16 expansion on the issue ports for every M <= 8.  The tensor pipe
// is nowhere near busy; it is used as a wide FMA.
//
// Data movement:
//   * One CTA owns 16 consecutive output channels; its 8 warps split K into eighths and
//     combine through shared memory (deterministic, no atomics).
//   * Every warp is its own little pipeline: lanes 0-15 each issue one bulk async copy
//     (cp.async.bulk) of "row r, this warp's K slice" (up to 320 contiguous bytes) into the
//     warp's private shared buffer, completion counted on the warp's own mbarrier, so a warp
//     starts decoding as soon as ITS bytes have landed while the rest of the tile is still in
//     flight.  All copies of a tile are issued in the first few hundred cycles of the CTA, so
//     the memory system sees the 16 rows as long sequential bursts.
//   * Shared rows are padded by 16 bytes: with a row stride of 4 (mod 8) words the per-lane
//     32-bit reads (row g, block 4j+c, word i) hit 32 distinct banks.
//   * Lane (g, c) = (lane / 4, lane % 4) decodes block 4j+c for rows g and g+8.  The MMA's 16 k-slots fall into four groups by c, and group c may carry
//     any four k's as long as the activation fragment uses the same ones -- so each lane feeds
//     "its" block's weights, no shuffles, and reads the matching 64 B of activations via L1.
//   * Weight = hfma2(q, d, m) after the exact nibble->half trick (q | 0x6400 = 1024 + q), one
//     f16 rounding per weight like the reference's f16 route; products accumulate in f32.
//
//   * Launched with programmatic stream serialization when the caller allows it
//     (NNB200_Q4_FLAG_OVERLAP_PREVIOUS): the weight copies are issued before
//     griddepcontrol.wait, so they overlap the tail of the preceding kernel in the stream;
//     activations are read and outputs written only after it.  Such a launch begins before the
//     kernel that produces the activations has finished, so no kernel boundary has invalidated
//     this SM's L1 since an earlier step may have read the same buffer: the vector loads of the
//     activations therefore go to L2 (ld.global.cg), never through the non-coherent path.
//
// CPU twin: mma_qblock_trans (src/backend/cpu/x86_64/mma_qblock.hpp:144-291).

#include <mutex>
#include <type_traits>

#include "internal.cuh"
#include "ptx.cuh"
#include "q4_1_common.cuh"

namespace nnb200 {

namespace {

constexpr int kRows = 16;              // output channels per CTA (one MMA m-tile)
constexpr int kWarps = 8;              // K slices
constexpr int kMaxChunkBlocks = 128;   // blocks of one row staged per pass (4096 k)
constexpr int kMaxSliceBlocks = kMaxChunkBlocks / kWarps;  // 16 blocks = 320 B per row per warp
constexpr int kRowPadBytes = 16;
constexpr int kSliceStride = kMaxSliceBlocks * kQ4BlockBytes + kRowPadBytes;  // 336 B: 84 words = 4 (mod 8)
constexpr int kSliceBufBytes = kRows * kSliceStride;                           // 5376 B
constexpr int kBufs = 2;               // chunks in flight per warp when K spans several chunks

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// (a & b) | c in one LOP3.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// (BIAS + q) pairs -> d*q + m, rounded once to f16.  BIAS is the half bit pattern the nibble
// was or-ed into: 0x6400 (1024, nibble in mantissa bits 0-3) or 0x5400 (64, nibble in bits 4-7).
template <uint16_t BIAS>
__device__ __forceinline__ uint32_t scale_pair(uint32_t biased, uint32_t d, uint32_t m)
{
    constexpr uint32_t kb = (static_cast<uint32_t>(BIAS) << 16) | BIAS;
    uint32_t q, r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(q) : "r"(biased), "r"(kb));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(q), "r"(d), "r"(m));
    return r;
}

// The 32 activations of one block for this lane's MMA column (activation row g), as four uint4.
// Lanes whose row does not exist keep the zeros they were initialised with: no work per step.
__device__ __forceinline__ void load_act_block(const __half* a_blk, bool vec_ok, uint4 (&av)[4])
{
    if (vec_ok) {
        const uint4* src = reinterpret_cast<const uint4*>(a_blk);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            av[j] = __ldcg(src + j);   // L2, not the non-coherent path: see the launch note below
        }
    } else {
        uint32_t* dst = reinterpret_cast<uint32_t*>(av);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const unsigned short* u = reinterpret_cast<const unsigned short*>(a_blk);
            dst[j] = static_cast<uint32_t>(__ldcg(u + 2 * j)) | (static_cast<uint32_t>(__ldcg(u + 2 * j + 1)) << 16);
        }
    }
}

// f32 activations: the 32 values of one block as f16, either their high parts hi = f16(a) or the
// remainders lo = f16(a - hi).  An MMA column fed with hi and another fed with lo, summed, give
// the product to f32 accuracy (the pair carries 22 mantissa bits).
__device__ __forceinline__ void load_act_block_f32(const float* a_blk, bool vec_ok, bool want_lo, uint4 (&av)[4])
{
    uint32_t* dst = reinterpret_cast<uint32_t*>(av);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float4 v;
        if (vec_ok) {
            v = __ldcg(reinterpret_cast<const float4*>(a_blk) + j);
        } else {
            v = make_float4(__ldcg(a_blk + 4 * j), __ldcg(a_blk + 4 * j + 1), __ldcg(a_blk + 4 * j + 2), __ldcg(a_blk + 4 * j + 3));
        }
        __half2 h01 = __floats2half2_rn(v.x, v.y);
        __half2 h23 = __floats2half2_rn(v.z, v.w);
        if (want_lo) {
            const float2 f01 = __half22float2(h01);
            const float2 f23 = __half22float2(h23);
            h01 = __floats2half2_rn(v.x - f01.x, v.y - f01.y);
            h23 = __floats2half2_rn(v.z - f23.x, v.w - f23.y);
        }
        dst[2 * j] = *reinterpret_cast<const uint32_t*>(&h01);
        dst[2 * j + 1] = *reinterpret_cast<const uint32_t*>(&h23);
    }
}

// Low half / high half of a word duplicated into both halves (f16 scale and min of a block).
__device__ __forceinline__ uint32_t dup_lo16(uint32_t w) { return __byte_perm(w, w, 0x1010); }
__device__ __forceinline__ uint32_t dup_hi16(uint32_t w) { return __byte_perm(w, w, 0x3232); }

// One block group: 16 rows x 32 k against the activation fragment `av`.  s_lo / s_hi point at
// this lane's block in rows g and g + 8 of the shared slice.
__device__ __forceinline__ void mma_block(const uint32_t* s_lo, const uint32_t* s_hi, const uint4 (&av)[4],
                                          float (&acc0)[4], float (&acc1)[4])
{
    uint32_t w_lo[5], w_hi[5];
#pragma unroll
    for (int j = 0; j < 5; ++j) {
        w_lo[j] = s_lo[j];
        w_hi[j] = s_hi[j];
    }
    const uint32_t d_lo = dup_lo16(w_lo[0]), m_lo = dup_hi16(w_lo[0]);
    const uint32_t d_hi = dup_lo16(w_hi[0]), m_hi = dup_hi16(w_hi[0]);
    const uint32_t* avw = reinterpret_cast<const uint32_t*>(av);
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
        const uint32_t x = w_lo[1 + wi];  // row g:     bytes 4wi..4wi+3
        const uint32_t y = w_hi[1 + wi];  // row g + 8
        const uint32_t x8 = x >> 8;
        const uint32_t y8 = y >> 8;
        // Low nibbles (k 4wi..4wi+3): nibble | 0x6400 = 1024 + q.  Pair A = bytes 0, 2
        // -> (k+0, k+2); pair B = bytes 1, 3 -> (k+1, k+3).
        {
            const uint32_t r0 = avw[2 * wi];
            const uint32_t r1 = avw[2 * wi + 1];
            mma_m16n8k16(acc0, scale_pair<0x6400>(and_or(x, 0x000F000Fu, 0x64006400u), d_lo, m_lo),
                         scale_pair<0x6400>(and_or(y, 0x000F000Fu, 0x64006400u), d_hi, m_hi),
                         scale_pair<0x6400>(and_or(x8, 0x000F000Fu, 0x64006400u), d_lo, m_lo),
                         scale_pair<0x6400>(and_or(y8, 0x000F000Fu, 0x64006400u), d_hi, m_hi),
                         __byte_perm(r0, r1, 0x5410), __byte_perm(r0, r1, 0x7632));
        }
        // High nibbles (k 16+4wi..): left in place, (nibble << 4) | 0x5400 = 64 + q.
        {
            const uint32_t r0 = avw[8 + 2 * wi];
            const uint32_t r1 = avw[8 + 2 * wi + 1];
            mma_m16n8k16(acc1, scale_pair<0x5400>(and_or(x, 0x00F000F0u, 0x54005400u), d_lo, m_lo),
                         scale_pair<0x5400>(and_or(y, 0x00F000F0u, 0x54005400u), d_hi, m_hi),
                         scale_pair<0x5400>(and_or(x8, 0x00F000F0u, 0x54005400u), d_lo, m_lo),
                         scale_pair<0x5400>(and_or(y8, 0x00F000F0u, 0x54005400u), d_hi, m_hi),
                         __byte_perm(r0, r1, 0x5410), __byte_perm(r0, r1, 0x7632));
        }
    }
}

// A_F32: activations are f32; MMA columns 0..m_count-1 carry their hi parts and columns
// m_count..2*m_count-1 their lo parts (so m_count <= 4), summed in the final reduction.
template <bool OUT_F16, bool A_F32>
__global__ void __launch_bounds__(kWarps * 32, 2)
q4_1_gemv_mma_kernel(const uint8_t* __restrict__ w, const int64_t w_pitch_bytes, const void* __restrict__ a_v,
                     const int64_t lda, void* __restrict__ out, const int64_t ldc, const int m_count,
                     const int n_total, const int k_total, const int num_bufs, const FpEpilogue ep,
                     const int a_vec_ok, int32_t* error_word)
{
    // [warp][buf][kSliceBufBytes]; num_bufs = min(kBufs, chunks of K).
    extern __shared__ __align__(128) uint8_t slices[];
    __shared__ __align__(8) uint64_t bars[kWarps][kBufs];
    __shared__ float4 partial[kWarps][32];
    __shared__ int abort_word;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;
    const int c = lane & 3;
    const int n0 = blockIdx.x * kRows;
    const int rows_valid = min(kRows, n_total - n0);

    const int nblk = k_total / kQ4BlockElems;            // the engine requires K % 128 == 0
    const int chunk_blocks = min(nblk, kMaxChunkBlocks);
    const int num_chunks = (nblk + chunk_blocks - 1) / chunk_blocks;

    // This warp's slice of chunk `ch`: block range [sb, sb + snb) of the row, snb a multiple of 4.
    auto slice_of = [&](int ch, int& sb, int& snb) {
        const int b0 = ch * chunk_blocks;
        const int groups = min(chunk_blocks, nblk - b0) / 4;
        const int per_warp = (groups + kWarps - 1) / kWarps;
        const int g_begin = min(groups, warp * per_warp);
        const int g_end = min(groups, g_begin + per_warp);
        sb = b0 + g_begin * 4;
        snb = (g_end - g_begin) * 4;
    };
    // Lanes 0..15 copy "row lane, this warp's slice" of chunk `ch` into buffer `buf`.
    auto issue_slice = [&](int ch, int buf) {
        int sb, snb;
        slice_of(ch, sb, snb);
        if (snb == 0) {
            return;
        }
        const uint32_t bytes = static_cast<uint32_t>(snb) * kQ4BlockBytes;
        if (lane == 0) {
            mbar_expect_tx(&bars[warp][buf], bytes * static_cast<uint32_t>(rows_valid));
        }
        __syncwarp();
        if (lane < rows_valid) {
            bulk_load_1d(slices + (warp * num_bufs + buf) * kSliceBufBytes + lane * kSliceStride,
                         w + static_cast<int64_t>(n0 + lane) * w_pitch_bytes + static_cast<int64_t>(sb) * kQ4BlockBytes,
                         bytes, &bars[warp][buf]);
        }
    };

    if (threadIdx.x == 0) {
        abort_word = 0;
    }
    if (lane == 0) {
        for (int b = 0; b < kBufs; ++b) {
            mbar_init(&bars[warp][b], 1);
        }
        mbar_init_fence();
    }
    __syncwarp();
    // Weights never depend on the preceding kernel: start streaming them right away.
    for (int b = 0; b < num_bufs && b < num_chunks; ++b) {
        issue_slice(b, b);
    }
    // Let the next kernel in the stream begin its own prologue, then wait until the previous
    // one has completed before touching activations or outputs.  Both are no-ops for a launch
    // without the programmatic-serialization attribute.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();  // abort_word initialised for every warp

    float acc0[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float acc1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    // Activation row this lane feeds as MMA column g (f32: column g carries the hi part of row g
    // for g < m_count and the lo part of row g - m_count after that).
    const bool row_live = A_F32 ? g < 2 * m_count : g < m_count;
    const bool want_lo = A_F32 && g >= m_count;
    const int a_row = row_live ? (want_lo ? g - m_count : g) : 0;
    const bool vec_ok = a_vec_ok != 0;
    using ActT = typename std::conditional<A_F32, float, __half>::type;
    // This lane's activations: its row, starting at its block c of the first group.
    const ActT* a_lane = static_cast<const ActT*>(a_v) + static_cast<int64_t>(a_row) * lda + c * kQ4BlockElems;
    const auto load_act = [&](const ActT* blk, uint4 (&av)[4]) {
        if constexpr (A_F32) {
            load_act_block_f32(blk, vec_ok, want_lo, av);
        } else {
            load_act_block(blk, vec_ok, av);
        }
    };
    // Two fragment register sets, used alternately; lanes without a row keep zeros throughout.
    uint4 av0[4], av1[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        av0[j] = make_uint4(0u, 0u, 0u, 0u);
        av1[j] = make_uint4(0u, 0u, 0u, 0u);
    }

    for (int ch = 0; ch < num_chunks; ++ch) {
        const int buf = ch % num_bufs;
        const uint32_t phase = static_cast<uint32_t>(ch / num_bufs) & 1u;
        int sb, snb;
        slice_of(ch, sb, snb);
        if (snb > 0) {
            const int groups = snb / 4;
            const ActT* a_grp = a_lane + static_cast<int64_t>(sb) * kQ4BlockElems;  // group 0 of this slice
            // First group's activations are fetched while the weights are still landing.
            if (row_live) {
                load_act(a_grp, av0);
            }
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(&bars[warp][buf], phase, &abort_word))) {
                atomicCAS(error_word, 0, kErrMmaWait);
                break;
            }
            const uint8_t* base = slices + (warp * num_bufs + buf) * kSliceBufBytes;
            const uint32_t* s_lo = reinterpret_cast<const uint32_t*>(base + g * kSliceStride) + c * kQ4BlockWords;
            const uint32_t* s_hi = reinterpret_cast<const uint32_t*>(base + (g + 8) * kSliceStride) + c * kQ4BlockWords;
            constexpr int kGroupWords = 4 * kQ4BlockWords;   // four blocks further along the row
            constexpr int kGroupElems = 4 * kQ4BlockElems;
            int gi = 0;
            for (; gi + 2 <= groups; gi += 2) {
                if (row_live) {
                    load_act(a_grp + (gi + 1) * kGroupElems, av1);
                }
                mma_block(s_lo + gi * kGroupWords, s_hi + gi * kGroupWords, av0, acc0, acc1);
                if (row_live && gi + 2 < groups) {
                    load_act(a_grp + (gi + 2) * kGroupElems, av0);
                }
                mma_block(s_lo + (gi + 1) * kGroupWords, s_hi + (gi + 1) * kGroupWords, av1, acc0, acc1);
            }
            if (gi < groups) {
                mma_block(s_lo + gi * kGroupWords, s_hi + gi * kGroupWords, av0, acc0, acc1);
            }
        }
        if (ch + num_bufs < num_chunks) {
            __syncwarp();  // every lane has finished reading this buffer
            issue_slice(ch + num_bufs, buf);
        }
    }

    partial[warp][lane] = make_float4(acc0[0] + acc1[0], acc0[1] + acc1[1], acc0[2] + acc1[2], acc0[3] + acc1[3]);
    __syncthreads();
    if (warp == 0) {
        float4 s = partial[0][lane];
#pragma unroll
        for (int wq = 1; wq < kWarps; ++wq) {
            const float4 p = partial[wq][lane];
            s.x += p.x;
            s.y += p.y;
            s.z += p.z;
            s.w += p.w;
        }
        // Fragment layout: (x, y) = channel n0+g, activation rows 2c and 2c+1; (z, w) = channel n0+g+8.
        float vals[4] = {s.x, s.y, s.z, s.w};
        if constexpr (A_F32) {
            // Column col holds the hi product of row col; its lo product sits m_count columns on,
            // i.e. in lane (g, (col + m_count) / 2), component (col + m_count) % 2 of the same quad.
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int col = 2 * c + (j & 1);
                const int pcol = (col + m_count) & 7;
                const int src_lane = (lane & ~3) | (pcol >> 1);
                const float even = __shfl_sync(0xFFFFFFFFu, j < 2 ? s.x : s.z, src_lane);
                const float odd = __shfl_sync(0xFFFFFFFFu, j < 2 ? s.y : s.w, src_lane);
                vals[j] += (pcol & 1) ? odd : even;
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + g + (j >= 2 ? 8 : 0);
            const int m = 2 * c + (j & 1);
            if (n < n_total && m < m_count) {
                const float v = fp_epilogue_value<OUT_F16>(ep, vals[j], n);
                if constexpr (OUT_F16) {
                    static_cast<__half*>(out)[static_cast<int64_t>(m) * ldc + n] = __float2half_rn(v);
                } else {
                    static_cast<float*>(out)[static_cast<int64_t>(m) * ldc + n] = v;
                }
            }
        }
    }
}

template <bool OUT_F16, bool A_F32>
cudaError_t launch_one(unsigned grid, bool overlap, cudaStream_t stream, const uint8_t* w, int64_t pitch,
                       const void* a, int64_t lda, void* out, int64_t ldc, int m_count, int n, int k, int num_bufs,
                       const FpEpilogue& ep, int a_vec_ok, int32_t* error_word)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = static_cast<size_t>(kWarps) * num_bufs * kSliceBufBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, q4_1_gemv_mma_kernel<OUT_F16, A_F32>, w, pitch, a, lda, out, ldc, m_count, n, k,
                              num_bufs, ep, a_vec_ok, error_word);
}

}  // namespace

bool q4_1_gemv_mma_supported(const nnb200_q4_1_args& q)
{
    // f16 or f32 activations; weight rows movable by 16-byte bulk copies: 16-byte aligned base and
    // pitch, whole rows a multiple of 4 blocks (K % 128 == 0).
    return q.n <= INT32_MAX && q.k <= INT32_MAX - 128 && (q.k % 128) == 0 &&
           (reinterpret_cast<uintptr_t>(q.w_blocks) & 15u) == 0 && (q.ldw_blocks % 4) == 0;
}

int launch_q4_1_gemv_mma(const nnb200_q4_1_args& q, const DeviceInfo& dev, cudaStream_t stream)
{
    FpEpilogue ep;
    ep.alpha = q.alpha;
    ep.bias = q.bias;
    ep.activation = q.activation;
    ep.act_alpha = q.act_alpha;
    ep.act_beta = q.act_beta;
    ep.min_clip = q.min_clip;
    ep.max_clip = q.max_clip;

    static std::once_flag once[kMaxDevices];
    static cudaError_t attr_err[kMaxDevices];
    std::call_once(once[dev.device], [&] {
        const int max_smem = kWarps * kBufs * kSliceBufBytes;
        cudaError_t e = cudaSuccess;
        const auto raise = [&](auto kernel) {
            if (e == cudaSuccess) {
                e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
            }
        };
        raise(q4_1_gemv_mma_kernel<false, false>);
        raise(q4_1_gemv_mma_kernel<true, false>);
        raise(q4_1_gemv_mma_kernel<false, true>);
        raise(q4_1_gemv_mma_kernel<true, true>);
        attr_err[dev.device] = e;
    });
    if (attr_err[dev.device] != cudaSuccess) {
        return NNB200_INTERNAL;
    }
    const int chunks = static_cast<int>((q.k / kQ4BlockElems + kMaxChunkBlocks - 1) / kMaxChunkBlocks);
    const int num_bufs = chunks < kBufs ? chunks : kBufs;
    const unsigned grid = static_cast<unsigned>((q.n + kRows - 1) / kRows);
    const bool a_f32 = q.a_f16 == 0;
    // 16-byte activation loads: aligned base and a row pitch that keeps every block aligned.
    const int a_vec_ok = ((reinterpret_cast<uintptr_t>(q.a) & 15u) == 0 && (q.lda % (a_f32 ? 4 : 8)) == 0) ? 1 : 0;
    const uint8_t* w = static_cast<const uint8_t*>(q.w_blocks);
    const int64_t pitch = q.ldw_blocks * kQ4BlockBytes;
    const bool overlap = (q.flags & NNB200_Q4_FLAG_OVERLAP_PREVIOUS) != 0;
    const int64_t a_elem = a_f32 ? 4 : 2;
    const int64_t out_elem = q.out_f16 ? 2 : 4;
    // Activation rows per launch: the MMA has 8 columns; f32 rows take two of them (hi and lo).
    const int rows_per_pass = a_f32 ? 4 : 8;
    for (int64_t m0 = 0; m0 < q.m; m0 += rows_per_pass) {
        const int m_count = static_cast<int>(q.m - m0 < rows_per_pass ? q.m - m0 : rows_per_pass);
        const void* a = static_cast<const uint8_t*>(q.a) + m0 * q.lda * a_elem;
        void* out = static_cast<uint8_t*>(q.out) + m0 * q.ldc * out_elem;
        const int n = static_cast<int>(q.n), k = static_cast<int>(q.k);
        cudaError_t e;
        if (a_f32) {
            e = q.out_f16 ? launch_one<true, true>(grid, overlap, stream, w, pitch, a, q.lda, out, q.ldc, m_count, n, k,
                                                   num_bufs, ep, a_vec_ok, dev.error_word)
                          : launch_one<false, true>(grid, overlap, stream, w, pitch, a, q.lda, out, q.ldc, m_count, n, k,
                                                    num_bufs, ep, a_vec_ok, dev.error_word);
        } else {
            e = q.out_f16 ? launch_one<true, false>(grid, overlap, stream, w, pitch, a, q.lda, out, q.ldc, m_count, n, k,
                                                    num_bufs, ep, a_vec_ok, dev.error_word)
                          : launch_one<false, false>(grid, overlap, stream, w, pitch, a, q.lda, out, q.ldc, m_count, n,
                                                     k, num_bufs, ep, a_vec_ok, dev.error_word);
        }
        note_launch();
        if (e != cudaSuccess) {
            return NNB200_INTERNAL;
        }
    }
    return NNB200_OK;
}

}  // namespace nnb200
