// Q4_1 decode GEMV with deferred scaling: the weights reach the tensor pipe as raw nibbles.
//
// Per weight the per-weight-dequantising GEMV (q4_1_gemv_mma.cu) pays a mask, a subtract and a
// fused multiply-add before its warp MMA, and that instruction issue -- not HBM -- is what
// bounds it.  Here a block's scale d and minimum m are applied once per (channel, block)
// AFTER the MMA:
//
//     sum_k (d q_k + m) a_k  =  d * sum_k q_k a_k  +  m * sum_k a_k
//
//   * q_k goes into the MMA exactly as it sits in the byte: (x & 0x000F000F) is a pair of f16
//     SUBNORMALS q * 2^-24, (x & 0x00F000F0) a pair q * 2^-20 (high nibbles, left in place).
//     One mask per weight pair, nothing else; products are exact in f32.  The two kinds
//     accumulate separately and are rejoined as 2^20 * (16 * D_lo + D_hi).
//   * sum_k a_k per block (T) depends only on the activations: computed once per CTA.
//   * The MMA's eight output columns would be wasted on one activation row, so they separate
//     BLOCKS instead: the B operand of the MMA that covers block j of a group is non-zero only
//     in the columns that belong to block j.  One accumulator then collects the complete
//     32-k sums of G = 8 / Mp blocks (Mp = activation rows padded to a power of two; f32
//     activations take two columns each, hi = f16(a) and lo = f16(a - hi)), and the fix-up
//     d * S + m * T is paid once per (channel, block, activation row).
//
// Data movement: persistent CTAs, one per SM, each owning a contiguous range of channels (so
// every SM streams the same number of bytes, whatever N is).  A producer warp brings 16
// channels x KC of k at a time into a shared ring with one bulk async copy per channel
// (cp.async.bulk, completion on the stage's mbarrier); for a small matrix the CTA's whole share
// is in flight from its first cycles.  Eight consumer warps take the block groups of a stage in
// turn; lane (g, c) reads nibble word c of each block of the group for channels g and g+8
// (bank-conflict free with the padded row stride) and feeds two MMAs per word.  The
// activations are staged once per CTA in the permuted pair order the masks produce -- pairs
// (k, k+2), (k+1, k+3), so no per-weight permute exists anywhere.  Partial sums of the eight
// warps meet in shared memory, double-buffered per 16-channel tile, and a ninth warp reduces
// them in a fixed order (deterministic), applies the output arithmetic and stores.
//
// Launched with programmatic stream serialization when the caller allows it
// (NNB200_Q4_FLAG_OVERLAP_PREVIOUS): the producer never touches anything the previous kernel
// wrote, so its copies run ahead of griddepcontrol.wait; a CTA uses at most half an SM's shared
// memory whenever the activations allow, so that the next GEMV's weight stream overlaps this
// one's tail.
//
// CPU twin: mma_qblock_trans (src/backend/cpu/x86_64/mma_qblock.hpp:144-291); same sum, other
// order, f32 accumulation.

#include <mutex>

#include "internal.cuh"
#include "ptx.cuh"
#include "q4_1_common.cuh"

namespace nnb200 {

namespace {

constexpr int kTileRows = 16;          // channels per tile (one MMA m-tile)
constexpr int kConsumers = 8;          // consumer warps
constexpr int kProducerWarp = kConsumers;
constexpr int kReducerWarp = kConsumers + 1;
constexpr int kThreads = (kConsumers + 2) * 32;
constexpr int kMaxStages = 4;
constexpr int kMaxActBytes = 64 * 1024;   // staged activations: Mp * K * 2 bytes at most

// Everything the kernel needs to know about its shared-memory carve-up; computed on the host.
struct DsqLayout {
    int kc_blocks;        // blocks of k per ring stage (multiple of 8)
    int stages;           // ring depth
    int row_stride;       // bytes between the 16 channel rows of a stage (16-byte multiple, padded)
    int stage_bytes;      // 16 * row_stride
    int nblk_pad;         // K / 32 rounded up to a multiple of 8
    int off_pairs;        // permuted activation pairs: [nblk_pad][Mp][16] u32
    int off_sums;         // per-block activation sums:  [nblk_pad][Mp] f32
    int off_zero;         // 16 zero bytes (B operand of lanes whose columns belong to another block)
    int off_partial;      // [2][kConsumers][32] float4
    int off_bars;         // full[kMaxStages], empty[kMaxStages], tile_done[2], partial_free[2]
    int total;
};

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 lds128(const void* p)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(smem_u32(p)));
    return v;
}


// Eight activations of one (block, nibble word): k0..k0+3 and k0+16..k0+19, as four f16 pairs
// in the order the weight masks produce them -- (k0, k0+2), (k0+1, k0+3), (k0+16, k0+18),
// (k0+17, k0+19) -- plus their f32 sum.  part = 1 stages the remainders a - f16(a) of f32
// activations instead of their f16 values.
template <bool A_F32>
__device__ __forceinline__ uint4 stage_act_word(const void* a_row, int k0, bool vec_ok, int part, float& sum)
{
    uint32_t w[4];  // (k0, k0+1), (k0+2, k0+3), (k0+16, k0+17), (k0+18, k0+19) as f16 pairs
    if constexpr (A_F32) {
        const float* a = static_cast<const float*>(a_row);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float* src = a + k0 + 16 * h;
            float4 v;
            if (vec_ok) {
                v = __ldg(reinterpret_cast<const float4*>(src));
            } else {
                v = make_float4(src[0], src[1], src[2], src[3]);
            }
            __half2 h01 = __floats2half2_rn(v.x, v.y);
            __half2 h23 = __floats2half2_rn(v.z, v.w);
            if (part != 0) {
                const float2 f01 = __half22float2(h01);
                const float2 f23 = __half22float2(h23);
                h01 = __floats2half2_rn(v.x - f01.x, v.y - f01.y);
                h23 = __floats2half2_rn(v.z - f23.x, v.w - f23.y);
            }
            w[2 * h] = *reinterpret_cast<const uint32_t*>(&h01);
            w[2 * h + 1] = *reinterpret_cast<const uint32_t*>(&h23);
        }
    } else {
        const __half* a = static_cast<const __half*>(a_row);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const __half* src = a + k0 + 16 * h;
            if (vec_ok) {
                const uint2 v = __ldg(reinterpret_cast<const uint2*>(src));
                w[2 * h] = v.x;
                w[2 * h + 1] = v.y;
            } else {
                w[2 * h] = static_cast<uint32_t>(__half_as_ushort(src[0])) |
                           (static_cast<uint32_t>(__half_as_ushort(src[1])) << 16);
                w[2 * h + 1] = static_cast<uint32_t>(__half_as_ushort(src[2])) |
                               (static_cast<uint32_t>(__half_as_ushort(src[3])) << 16);
            }
        }
    }
    sum = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
        sum += f.x + f.y;
    }
    return make_uint4(__byte_perm(w[0], w[1], 0x5410), __byte_perm(w[0], w[1], 0x7632),
                      __byte_perm(w[2], w[3], 0x5410), __byte_perm(w[2], w[3], 0x7632));
}

// One group of G = 8 / MP blocks x 16 channels: 2 G MMAs, then the fix-up into acc.
//   wlo / whi   this lane's channel rows g and g + 8 of the stage, as words
//   ul / ub     first block of the group, counted inside the stage / inside the row
template <int MP>
__device__ __forceinline__ void dsq_group(const uint32_t* wlo, const uint32_t* whi, int ul, int ub, int nblk,
                                          const uint32_t* pairs, const float* sums, const uint32_t* zero, int g,
                                          int c, float (&acc)[4])
{
    constexpr int G = 8 / MP;
    constexpr uint32_t kLo = 0x000F000Fu;   // low nibbles of bytes 0 and 2: q * 2^-24 as f16 subnormals
    constexpr uint32_t kHi = 0x00F000F0u;   // high nibbles, in place: q * 2^-20
    const int my_j = g / MP;                // the block of the group this lane's B columns belong to
    const int my_col = g % MP;
    float dl[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    float dh[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    const uint32_t* mine = pairs + (static_cast<size_t>(ub + my_j) * MP + my_col) * 16 + 4 * c;
#pragma unroll
    for (int j = 0; j < G; ++j) {
        const int word = 5 * (ul + j) + 1 + c;
        const uint32_t x = wlo[word];
        const uint32_t y = whi[word];
        const uint4 b = lds128(j == my_j ? mine : zero);
        const uint32_t xs = x >> 8;
        const uint32_t ys = y >> 8;
        mma_m16n8k16(dl[j & 1], x & kLo, y & kLo, xs & kLo, ys & kLo, b.x, b.y);
        mma_m16n8k16(dh[j & 1], x & kHi, y & kHi, xs & kHi, ys & kHi, b.z, b.w);
    }
    // q-sums in units of 2^-20: entry e = (channel g + 8 * (e >> 1), column 2c + (e & 1)).
    float s[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float lo = G > 1 ? dl[0][e] + dl[1][e] : dl[0][e];
        const float hi = G > 1 ? dh[0][e] + dh[1][e] : dh[0][e];
        s[e] = fmaf(lo, 16.0f, hi);
    }
    const float2 t = *reinterpret_cast<const float2*>(sums + static_cast<size_t>(ub) * MP + 2 * c);
    constexpr float kUnit = 1048576.0f;  // 2^20
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const uint32_t* row = half == 0 ? wlo : whi;
#pragma unroll
        for (int e2 = 0; e2 < 2; ++e2) {
            // Block of column 2c + e2; with MP >= 2 both columns belong to one block.
            const int jb = (2 * c + e2) / MP;
            const uint32_t dm = row[5 * (ul + jb)];
            float2 f = __half22float2(*reinterpret_cast<const __half2*>(&dm));   // (d, m)
            if (ub + jb >= nblk) {
                f = make_float2(0.0f, 0.0f);   // past the end of K: the stage holds no such block
            }
            const int e = 2 * half + e2;
            acc[e] = fmaf(f.x * kUnit, s[e], acc[e]);
            acc[e] = fmaf(f.y, e2 == 0 ? t.x : t.y, acc[e]);
        }
    }
}


// MP: MMA columns per block (activation rows padded to 1, 2, 4 or 8; f32 rows count twice).
template <int MP, bool OUT_F16, bool A_F32>
__global__ void __launch_bounds__(kThreads, 2)
q4_1_gemv_dsq_kernel(const uint8_t* __restrict__ w, const int64_t w_pitch_bytes, const void* __restrict__ a_v,
                     const int64_t lda, void* __restrict__ out, const int64_t ldc, const int m_count,
                     const int n_total, const int k_total, const DsqLayout lay, const FpEpilogue ep,
                     const int a_vec_ok, int32_t* error_word)
{
    constexpr int G = 8 / MP;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int abort_word;

    uint64_t* full = reinterpret_cast<uint64_t*>(smem + lay.off_bars);
    uint64_t* empty = full + kMaxStages;
    uint64_t* tile_done = empty + kMaxStages;
    uint64_t* partial_free = tile_done + 2;
    uint32_t* pairs = reinterpret_cast<uint32_t*>(smem + lay.off_pairs);
    float* sums = reinterpret_cast<float*>(smem + lay.off_sums);
    const uint32_t* zero = reinterpret_cast<const uint32_t*>(smem + lay.off_zero);
    float4* partial = reinterpret_cast<float4*>(smem + lay.off_partial);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // This CTA's channels: an equal, contiguous share of all of them.
    const int row_begin = static_cast<int>(static_cast<int64_t>(blockIdx.x) * n_total / gridDim.x);
    const int row_end = static_cast<int>(static_cast<int64_t>(blockIdx.x + 1) * n_total / gridDim.x);
    const int tiles = (row_end - row_begin + kTileRows - 1) / kTileRows;
    const int nblk = k_total / kQ4BlockElems;
    const int chunks = (nblk + lay.kc_blocks - 1) / lay.kc_blocks;
    const int total_stages = tiles * chunks;

    if (threadIdx.x == 0) {
        abort_word = 0;
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumers);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tile_done[b], kConsumers);
            mbar_init(&partial_free[b], 1);
        }
        mbar_init_fence();
    }
    __syncthreads();
    // The next kernel in the stream may start its own prologue (and its weight stream) now.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == kProducerWarp) {
        // ---- producer: weights never depend on the preceding kernel, so no griddepcontrol.wait here ----
        for (int s = 0; s < total_stages; ++s) {
            const int slot = s % lay.stages;
            const int round = s / lay.stages;
            if (round > 0 && !mbar_wait_warp(&empty[slot], static_cast<uint32_t>(round - 1) & 1u, &abort_word)) {
                atomicCAS(error_word, 0, kErrProducerWait);
                break;
            }
            const int tile = s / chunks;
            const int b0 = (s % chunks) * lay.kc_blocks;
            const uint32_t bytes = static_cast<uint32_t>(min(lay.kc_blocks, nblk - b0)) * kQ4BlockBytes;
            const int r0 = row_begin + tile * kTileRows;
            const int valid = min(kTileRows, row_end - r0);
            if (lane == 0) {
                mbar_expect_tx(&full[slot], bytes * static_cast<uint32_t>(valid));
            }
            __syncwarp();
            if (lane < valid) {
                bulk_load_1d(smem + static_cast<size_t>(slot) * lay.stage_bytes + lane * lay.row_stride,
                             w + static_cast<int64_t>(r0 + lane) * w_pitch_bytes + static_cast<int64_t>(b0) * kQ4BlockBytes,
                             bytes, &full[slot]);
            }
        }
        // No copy may still be in flight when the CTA retires: the latest phase of every slot
        // has landed (a parity wait does not consume the phase).
        const int first = total_stages > lay.stages ? total_stages - lay.stages : 0;
        for (int s = first; s < total_stages; ++s) {
            if (!mbar_wait_warp(&full[s % lay.stages], static_cast<uint32_t>(s / lay.stages) & 1u, &abort_word)) {
                atomicCAS(error_word, 0, kErrDrainWait);
                break;
            }
        }
        return;
    }

    // Activations are read and outputs written only after the preceding kernel has completed.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == kReducerWarp) {
        // ---- reducer: sum the consumer warps' partials per tile in a fixed order, finish, store ----
        for (int tile = 0; tile < tiles; ++tile) {
            const int buf = tile & 1;
            if (!mbar_wait_warp(&tile_done[buf], static_cast<uint32_t>(tile >> 1) & 1u, &abort_word)) {
                atomicCAS(error_word, 0, kErrEpilogueWait);
                break;
            }
            const float4* part = partial + buf * (kConsumers * 32);
            const int r0 = row_begin + tile * kTileRows;
            for (int idx = lane; idx < kTileRows * m_count; idx += 32) {
                const int r = idx & (kTileRows - 1);
                const int mm = idx / kTileRows;
                const int g = r & 7;
                const int hi = r >> 3;
                float sum = 0.0f;
#pragma unroll
                for (int wq = 0; wq < kConsumers; ++wq) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float4 p = part[wq * 32 + g * 4 + c];
                        const float v0 = hi ? p.z : p.x;   // column 2c
                        const float v1 = hi ? p.w : p.y;   // column 2c + 1
                        const int col0 = (2 * c) % MP;
                        const int col1 = (2 * c + 1) % MP;
                        if ((A_F32 ? col0 >> 1 : col0) == mm) {
                            sum += v0;
                        }
                        if ((A_F32 ? col1 >> 1 : col1) == mm) {
                            sum += v1;
                        }
                    }
                }
                const int n = r0 + r;
                if (n < row_end) {
                    const float v = fp_epilogue_value<OUT_F16>(ep, sum, n);
                    if constexpr (OUT_F16) {
                        static_cast<__half*>(out)[static_cast<int64_t>(mm) * ldc + n] = __float2half_rn(v);
                    } else {
                        static_cast<float*>(out)[static_cast<int64_t>(mm) * ldc + n] = v;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&partial_free[buf]);
            }
        }
        return;
    }

    // ---- consumers ----
    // Stage the activations once: permuted pairs and per-block sums, zeros past M and past K.
    {
        const int tid = threadIdx.x;   // 0 .. 255
        if (tid < 4) {
            reinterpret_cast<uint32_t*>(smem + lay.off_zero)[tid] = 0u;
        }
        const int tasks = lay.nblk_pad * MP * 4;   // (block, column, nibble word); a multiple of 32
        for (int t = tid; t < tasks; t += kConsumers * 32) {
            const int i = t & 3;
            const int col = (t >> 2) % MP;
            const int blk = (t >> 2) / MP;
            const int row = A_F32 ? col >> 1 : col;
            float sum = 0.0f;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (blk < nblk && row < m_count) {
                const void* a_row = static_cast<const uint8_t*>(a_v) + static_cast<int64_t>(row) * lda * (A_F32 ? 4 : 2);
                v = stage_act_word<A_F32>(a_row, blk * kQ4BlockElems + 4 * i, a_vec_ok != 0, A_F32 ? (col & 1) : 0, sum);
            }
            *reinterpret_cast<uint4*>(pairs + static_cast<size_t>(t >> 2) * 16 + 4 * i) = v;
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
            if (i == 0) {
                sums[t >> 2] = sum;
            }
        }
        named_barrier_sync(1, kConsumers * 32);
    }

    const int g = lane >> 2;
    const int c = lane & 3;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    bool ok = true;
    for (int s = 0; s < total_stages && ok; ++s) {
        const int slot = s % lay.stages;
        const int tile = s / chunks;
        const int chunk = s % chunks;
        if (chunk == 0) {
            acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
        }
        if (!mbar_wait_warp(&full[slot], static_cast<uint32_t>(s / lay.stages) & 1u, &abort_word)) {
            atomicCAS(error_word, 0, kErrMmaWait);
            break;
        }
        const uint8_t* base = smem + static_cast<size_t>(slot) * lay.stage_bytes;
        const uint32_t* wlo = reinterpret_cast<const uint32_t*>(base + g * lay.row_stride);
        const uint32_t* whi = reinterpret_cast<const uint32_t*>(base + (g + 8) * lay.row_stride);
        const int b0 = chunk * lay.kc_blocks;
        const int groups = (min(lay.kc_blocks, nblk - b0) + G - 1) / G;
        for (int u = warp; u < groups; u += kConsumers) {
            dsq_group<MP>(wlo, whi, u * G, b0 + u * G, nblk, pairs, sums, zero, g, c, acc);
        }
        __syncwarp();   // every lane has finished reading the stage
        if (lane == 0) {
            mbar_arrive(&empty[slot]);
        }
        if (chunk == chunks - 1) {
            const int buf = tile & 1;
            if (tile >= 2 &&
                !mbar_wait_warp(&partial_free[buf], static_cast<uint32_t>((tile >> 1) - 1) & 1u, &abort_word)) {
                atomicCAS(error_word, 0, kErrAccumWait);
                ok = false;
                break;
            }
            partial[buf * (kConsumers * 32) + warp * 32 + lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&tile_done[buf]);
            }
        }
    }
}


int round_up(int v, int to) { return (v + to - 1) / to * to; }

// Columns per block for a pass of `rows` activation rows: rows (f32: twice that) rounded up to a
// power of two.
int columns_per_block(int rows, bool a_f32)
{
    const int cols = a_f32 ? 2 * rows : rows;
    return cols <= 1 ? 1 : (cols <= 2 ? 2 : (cols <= 4 ? 4 : 8));
}

// Shared-memory plan.  First choice: stay within half an SM (so that the next GEMV of a
// programmatically chained sequence fits beside this one) with at least ~40 KB of weights in
// flight; otherwise take what one CTA per SM can have.  Returns false when the staged
// activations alone are too large.
bool plan_layout(int mp, int64_t k, DsqLayout* out)
{
    DsqLayout l = {};
    const int nblk = static_cast<int>(k / kQ4BlockElems);
    l.nblk_pad = round_up(nblk, 8);
    const int64_t act_bytes = static_cast<int64_t>(l.nblk_pad) * mp * 64;
    if (act_bytes > kMaxActBytes) {
        return false;
    }
    int off = 0;
    l.off_pairs = off;
    off += static_cast<int>(act_bytes);
    l.off_sums = off;
    off += round_up(l.nblk_pad * mp * 4, 128);
    l.off_zero = off;
    off += 128;
    l.off_partial = off;
    off += 2 * kConsumers * 32 * 16;
    l.off_bars = off;
    off += 128;
    const int fixed = off;
    constexpr int kHalfSm = 110 * 1024;
    constexpr int kWholeSm = 224 * 1024;
    const int budgets[2] = {kHalfSm, kWholeSm};
    for (int pass = 0; pass < 2; ++pass) {
        int best_flight = 0, best_kc = 0, best_stages = 0;
        for (int kc = 64; kc >= 16; kc /= 2) {
            const int kcb = kc < l.nblk_pad ? kc : l.nblk_pad;
            const int stride = kcb * kQ4BlockBytes + 16;   // 5 * kcb + 4 words: 4 * odd (mod 32) for kcb % 8 == 0
            const int stage = kTileRows * stride;
            int stages = (budgets[pass] - fixed) / stage;
            stages = stages > kMaxStages ? kMaxStages : stages;
            if (stages >= 2 && stages * stage > best_flight) {
                best_flight = stages * stage;
                best_kc = kcb;
                best_stages = stages;
            }
        }
        if (best_stages >= 2 && (best_flight >= 40 * 1024 || pass == 1)) {
            l.kc_blocks = best_kc;
            l.stages = best_stages;
            l.row_stride = best_kc * kQ4BlockBytes + 16;
            l.stage_bytes = kTileRows * l.row_stride;
            // The ring sits in front; everything else follows it.
            const int ring = round_up(l.stages * l.stage_bytes, 128);
            l.off_pairs += ring;
            l.off_sums += ring;
            l.off_zero += ring;
            l.off_partial += ring;
            l.off_bars += ring;
            l.total = ring + fixed;
            *out = l;
            return true;
        }
    }
    return false;
}

using DsqKernel = void (*)(const uint8_t*, int64_t, const void*, int64_t, void*, int64_t, int, int, int, DsqLayout,
                           FpEpilogue, int, int32_t*);

template <int MP>
DsqKernel pick_kernel(bool out_f16, bool a_f32)
{
    if (a_f32) {
        if constexpr (MP >= 2) {
            return out_f16 ? q4_1_gemv_dsq_kernel<MP, true, true> : q4_1_gemv_dsq_kernel<MP, false, true>;
        } else {
            return nullptr;
        }
    }
    return out_f16 ? q4_1_gemv_dsq_kernel<MP, true, false> : q4_1_gemv_dsq_kernel<MP, false, false>;
}

DsqKernel pick_kernel(int mp, bool out_f16, bool a_f32)
{
    switch (mp) {
    case 1: return pick_kernel<1>(out_f16, a_f32);
    case 2: return pick_kernel<2>(out_f16, a_f32);
    case 4: return pick_kernel<4>(out_f16, a_f32);
    default: return pick_kernel<8>(out_f16, a_f32);
    }
}

}  // namespace

bool q4_1_gemv_dsq_supported(const nnb200_q4_1_args& q)
{
    // Weight rows movable by 16-byte bulk copies (aligned base and pitch, K % 128 == 0) and one
    // pass's activations small enough to stage whole in shared memory.
    if (!(q.n <= INT32_MAX && q.k <= INT32_MAX - 128 && (q.k % 128) == 0 &&
          (reinterpret_cast<uintptr_t>(q.w_blocks) & 15u) == 0 && (q.ldw_blocks % 4) == 0)) {
        return false;
    }
    const bool a_f32 = q.a_f16 == 0;
    const int rows_per_pass = a_f32 ? 4 : 8;
    const int first = static_cast<int>(q.m < rows_per_pass ? q.m : rows_per_pass);
    DsqLayout l;
    return plan_layout(columns_per_block(first, a_f32), q.k, &l);
}

int launch_q4_1_gemv_dsq(const nnb200_q4_1_args& q, const DeviceInfo& dev, cudaStream_t stream)
{
    FpEpilogue ep;
    ep.alpha = q.alpha;
    ep.bias = q.bias;
    ep.activation = q.activation;
    ep.act_alpha = q.act_alpha;
    ep.act_beta = q.act_beta;
    ep.min_clip = q.min_clip;
    ep.max_clip = q.max_clip;

    const bool a_f32 = q.a_f16 == 0;
    const bool out_f16 = q.out_f16 != 0;
    const int rows_per_pass = a_f32 ? 4 : 8;
    const int64_t a_elem = a_f32 ? 4 : 2;
    const int64_t out_elem = out_f16 ? 2 : 4;
    const int n = static_cast<int>(q.n), k = static_cast<int>(q.k);
    // Vector loads of the activations: 8-byte (f16) / 16-byte (f32) aligned groups of four.
    const int a_vec_ok = ((reinterpret_cast<uintptr_t>(q.a) & (a_f32 ? 15u : 7u)) == 0 && (q.lda % 4) == 0) ? 1 : 0;
    const uint8_t* w = static_cast<const uint8_t*>(q.w_blocks);
    const int64_t pitch = q.ldw_blocks * kQ4BlockBytes;
    const bool overlap = (q.flags & NNB200_Q4_FLAG_OVERLAP_PREVIOUS) != 0;
    const int tiles = (n + kTileRows - 1) / kTileRows;
    const unsigned grid = static_cast<unsigned>(tiles < dev.sm_count ? tiles : dev.sm_count);

    // Opt-in to large dynamic shared memory once per device and kernel variant.
    static std::mutex attr_mutex;
    static bool attr_done[kMaxDevices][4][2][2];

    for (int64_t m0 = 0; m0 < q.m; m0 += rows_per_pass) {
        const int m_count = static_cast<int>(q.m - m0 < rows_per_pass ? q.m - m0 : rows_per_pass);
        const int mp = columns_per_block(m_count, a_f32);
        DsqLayout lay;
        if (!plan_layout(mp, k, &lay)) {
            return NNB200_UNSUPPORTED;
        }
        DsqKernel kernel = pick_kernel(mp, out_f16, a_f32);
        if (kernel == nullptr) {
            return NNB200_INTERNAL;
        }
        const int mp_idx = mp == 1 ? 0 : (mp == 2 ? 1 : (mp == 4 ? 2 : 3));
        {
            std::lock_guard<std::mutex> lock(attr_mutex);
            bool& done = attr_done[dev.device][mp_idx][out_f16 ? 1 : 0][a_f32 ? 1 : 0];
            if (!done) {
                if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024) != cudaSuccess) {
                    (void)cudaGetLastError();
                    return NNB200_INTERNAL;
                }
                done = true;
            }
        }
        const void* a = static_cast<const uint8_t*>(q.a) + m0 * q.lda * a_elem;
        void* out = static_cast<uint8_t*>(q.out) + m0 * q.ldc * out_elem;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = static_cast<size_t>(lay.total);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = overlap ? 1 : 0;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, w, pitch, a, q.lda, out, q.ldc, m_count, n, k, lay, ep,
                                                 a_vec_ok, dev.error_word);
        note_launch();
        if (e != cudaSuccess) {
            return NNB200_INTERNAL;
        }
    }
    return NNB200_OK;
}

}  // namespace nnb200
