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
constexpr int kMaxConsumers = 16;      // consumer warps: 8 or 16 (NC), then one producer and one reducer warp
constexpr int kMaxStages = 4;
constexpr int kMaxActBytes = 64 * 1024;   // staged activations: Mp * K * 2 bytes at most

// Everything the kernel needs to know about its shared-memory carve-up; computed on the host.
struct DsqLayout {
    int kc_blocks;        // blocks of k per ring stage (multiple of 8)
    int stages;           // ring depth
    int row_stride;       // bytes between the 16 channel rows of a stage (16-byte multiple, padded)
    int dm_off;           // packed weights: where the stage's 16 rows of (d, m) entries start
    int dm_stride;        // packed weights: bytes between those rows
    int stage_bytes;      // 16 * row_stride (+ 16 * dm_stride)
    int nblk_pad;         // K / 32 rounded up to a multiple of 8
    int off_pairs;        // permuted activation pairs: [nblk_pad][Mp][16] u32
    int off_sums;         // per-block activation sums:  [nblk_pad][Mp] f32
    int off_zero;         // 128 zero bytes (B operand of lanes whose columns belong to another block)
    int off_partial;      // [2][consumer warps][16 channels][Mp] f32
    int off_bars;         // full[kMaxStages], empty[kMaxStages], tile_done[2], partial_free[2]
    int total;
};

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1)
{
    // Not volatile: a pure function of its operands, so that loads of the next block may be
    // scheduled across it.
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}


// Same, starting a fresh accumulator (C = 0): spares the sixteen register clears a group would
// otherwise pay for its four accumulators.
__device__ __forceinline__ void mma_m16n8k16_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                   uint32_t b0, uint32_t b1)
{
    const float z = 0.0f;
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%10, %10, %10, %10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z));
}

// Bounded wait polled by every lane of the warp (one warp-wide instruction per poll, no lane
// election and no divergence).  False when the wait ran out or another role aborted.
__device__ __forceinline__ bool mbar_wait_all_lanes(uint64_t* bar, uint32_t parity, volatile int* abort_flag)
{
    // Both votes are taken by all lanes whatever each lane saw, so the warp cannot split.
    if (__all_sync(0xFFFFFFFFu, mbar_try_wait(bar, parity))) {
        return true;
    }
    return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, abort_flag));
}

// Eight activations of one (block, nibble word): k0..k0+3 and k0+16..k0+19.  Loading and
// finishing are separate steps so that a thread can have several words' loads in flight.
// The loads go to L2 (ld.global.cg): a programmatically chained launch starts while the kernel
// that produces the activations is still running, so this SM's L1 may hold lines of the same
// buffer from an earlier step that no kernel boundary has invalidated.
template <bool A_F32>
struct ActRaw {
    uint32_t r[A_F32 ? 8 : 4];
};

template <bool A_F32>
__device__ __forceinline__ ActRaw<A_F32> load_act_word(const void* a_row, int k0, bool vec_ok)
{
    ActRaw<A_F32> raw;
    if constexpr (A_F32) {
        const float* a = static_cast<const float*>(a_row);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float* src = a + k0 + 16 * h;
            float4 v;
            if (vec_ok) {
                v = __ldcg(reinterpret_cast<const float4*>(src));
            } else {
                v = make_float4(__ldcg(src), __ldcg(src + 1), __ldcg(src + 2), __ldcg(src + 3));
            }
            raw.r[4 * h] = __float_as_uint(v.x);
            raw.r[4 * h + 1] = __float_as_uint(v.y);
            raw.r[4 * h + 2] = __float_as_uint(v.z);
            raw.r[4 * h + 3] = __float_as_uint(v.w);
        }
    } else {
        const __half* a = static_cast<const __half*>(a_row);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const __half* src = a + k0 + 16 * h;
            if (vec_ok) {
                const uint2 v = __ldcg(reinterpret_cast<const uint2*>(src));
                raw.r[2 * h] = v.x;
                raw.r[2 * h + 1] = v.y;
            } else {
                const unsigned short* u = reinterpret_cast<const unsigned short*>(src);
                raw.r[2 * h] = static_cast<uint32_t>(__ldcg(u)) | (static_cast<uint32_t>(__ldcg(u + 1)) << 16);
                raw.r[2 * h + 1] = static_cast<uint32_t>(__ldcg(u + 2)) | (static_cast<uint32_t>(__ldcg(u + 3)) << 16);
            }
        }
    }
    return raw;
}

// The word's four f16 pairs in the order the weight masks produce them -- (k0, k0+2),
// (k0+1, k0+3), (k0+16, k0+18), (k0+17, k0+19) -- plus their f32 sum.  part = 1 stages the
// remainders a - f16(a) of f32 activations instead of their f16 values.
template <bool A_F32>
__device__ __forceinline__ uint4 finish_act_word(const ActRaw<A_F32>& raw, int part, float& sum)
{
    uint32_t w[4];  // (k0, k0+1), (k0+2, k0+3), (k0+16, k0+17), (k0+18, k0+19) as f16 pairs
    if constexpr (A_F32) {
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const float x = __uint_as_float(raw.r[2 * p]);
            const float y = __uint_as_float(raw.r[2 * p + 1]);
            __half2 h = __floats2half2_rn(x, y);
            if (part != 0) {
                const float2 f = __half22float2(h);
                h = __floats2half2_rn(x - f.x, y - f.y);
            }
            w[p] = *reinterpret_cast<const uint32_t*>(&h);
        }
    } else {
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            w[p] = raw.r[p];
        }
    }
    sum = 0.0f;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[p]));
        sum += f.x + f.y;
    }
    return make_uint4(__byte_perm(w[0], w[1], 0x5410), __byte_perm(w[0], w[1], 0x7632),
                      __byte_perm(w[2], w[3], 0x5410), __byte_perm(w[2], w[3], 0x7632));
}

// Shared-memory loads by 32-bit shared-window address.  Volatile keeps them in program order
// among themselves and behind the barrier waits; the (non-volatile) MMAs and the arithmetic
// may still be scheduled around them.
__device__ __forceinline__ uint32_t lds32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 lds_f2(uint32_t addr)
{
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}

// Where lane (g, c) takes the two halves of its MMA A operand from, inside a group of
// G = 8 / MP blocks, and which of its B halves carry activations:
//   half 0 fills k-slots 2c, 2c+1 (registers a0/a1, b0), half 1 k-slots 2c+8, 2c+9 (a2/a3, b1);
//   each half walks kWords consecutive nibble words of ONE block, and every word gives four
//   MMAs (low nibbles of bytes 0/2, of bytes 1/3, high nibbles of bytes 0/2, of bytes 1/3).
//   MP = 1: half 0 = block c, half 1 = block c + 4, four words each        (16 MMAs)
//   MP = 2: both halves block c; words 0-1 and 2-3                          (8 MMAs)
//   MP = 4: both halves block c & 1; word c >> 1 and word (c >> 1) + 2      (4 MMAs)
//   MP = 8: one block; word c; the low-nibble pair feeds a0/a2 of one MMA, the high-nibble pair
//           the other                                                       (2 MMAs)
// A B half is live only in the lanes whose output column (= g) belongs to that half's block:
// g / MP == block.  That is a per-lane constant, so "activations or zeros" is decided once,
// in the address the lane loads its B operand from, never per MMA.
template <int MP>
struct DsqLane {
    static constexpr int kWords = MP == 1 ? 4 : (MP == 2 ? 2 : 1);
    __device__ static int block_of(int c, int half) { return MP == 1 ? c + 4 * half : (MP == 2 ? c : (MP == 4 ? (c & 1) : 0)); }
    __device__ static int word_of(int c, int half) { return MP == 1 ? 0 : (MP == 2 ? 2 * half : (MP == 4 ? (c >> 1) + 2 * half : c)); }
};

// One group of G = 8 / MP blocks x 16 channels: 2 G MMAs, then the fix-up into acc.
//   wlo / whi   shared addresses of this lane's channel rows g and g + 8 at the group's first block
//   dlo / dhi   packed weights only: the same for the rows of (d, m) entries
//   b0_at/b1_at shared addresses of the activation pairs for the lane's two operand halves (or of
//               zeros, in lanes whose columns belong to another block)
//   sums_at     shared address of the two per-block activation sums of columns 2c and 2c + 1
//   blocks_left blocks from the group's first one to the end of K (>= 1; < G only in a row's last group)
template <int MP, bool PACKED>
__device__ __forceinline__ void dsq_group(uint32_t wlo, uint32_t whi, uint32_t dlo, uint32_t dhi, uint32_t b0_at,
                                          uint32_t b1_at, uint32_t sums_at, int blocks_left, int c, float (&acc)[4])
{
    constexpr int G = 8 / MP;
    constexpr uint32_t kLo = 0x000F000Fu;   // low nibbles of bytes 0 and 2: q * 2^-24 as f16 subnormals
    constexpr uint32_t kHi = 0x00F000F0u;   // high nibbles, in place: q * 2^-20
    // Raw stream: a block is 20 bytes, its nibble words 1..4.  Packed: 16 bytes, words 0..3, and
    // 16-byte aligned, so a lane that walks a whole block takes it in one load.
    constexpr uint32_t kBlk = PACKED ? 16u : 20u;
    constexpr uint32_t kFirst = PACKED ? 0u : 4u;
    float dl[2][4], dh[2][4];               // two accumulator chains per nibble kind
    if constexpr (MP == 8) {
        const uint32_t x = lds32(wlo + kFirst + 4u * c);
        const uint32_t y = lds32(whi + kFirst + 4u * c);
        const uint4 b = lds128(b0_at);
        const uint32_t xs = x >> 8;
        const uint32_t ys = y >> 8;
        mma_m16n8k16_first(dl[0], x & kLo, y & kLo, xs & kLo, ys & kLo, b.x, b.y);
        mma_m16n8k16_first(dh[0], x & kHi, y & kHi, xs & kHi, ys & kHi, b.z, b.w);
    } else {
        using L = DsqLane<MP>;
        const uint32_t at0 = kBlk * L::block_of(c, 0) + kFirst + 4u * L::word_of(c, 0);
        const uint32_t at1 = kBlk * L::block_of(c, 1) + kFirst + 4u * L::word_of(c, 1);
        uint32_t xw0[L::kWords], yw0[L::kWords], xw1[L::kWords], yw1[L::kWords];
        if constexpr (PACKED && MP == 1) {
            // Whole blocks: four 16-byte loads instead of sixteen 4-byte ones.
            const uint4 a = lds128(wlo + at0), b = lds128(whi + at0), cc = lds128(wlo + at1), d = lds128(whi + at1);
            xw0[0] = a.x; xw0[1] = a.y; xw0[2] = a.z; xw0[3] = a.w;
            yw0[0] = b.x; yw0[1] = b.y; yw0[2] = b.z; yw0[3] = b.w;
            xw1[0] = cc.x; xw1[1] = cc.y; xw1[2] = cc.z; xw1[3] = cc.w;
            yw1[0] = d.x; yw1[1] = d.y; yw1[2] = d.z; yw1[3] = d.w;
        } else if constexpr (PACKED && MP == 2) {
            // Both halves walk the same block (words 0-1 and 2-3): one 16-byte load per channel.
            const uint4 a = lds128(wlo + at0), b = lds128(whi + at0);
            xw0[0] = a.x; xw0[1] = a.y; xw1[0] = a.z; xw1[1] = a.w;
            yw0[0] = b.x; yw0[1] = b.y; yw1[0] = b.z; yw1[1] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < L::kWords; ++i) {
                xw0[i] = lds32(wlo + at0 + 4u * i);
                yw0[i] = lds32(whi + at0 + 4u * i);
                xw1[i] = lds32(wlo + at1 + 4u * i);
                yw1[i] = lds32(whi + at1 + 4u * i);
            }
        }
#pragma unroll
        for (int i = 0; i < L::kWords; ++i) {
            const uint32_t x0 = xw0[i], y0 = yw0[i], x1 = xw1[i], y1 = yw1[i];
            const uint4 p0 = lds128(b0_at + 16u * i);
            const uint4 p1 = lds128(b1_at + 16u * i);
            const uint32_t x0s = x0 >> 8, y0s = y0 >> 8, x1s = x1 >> 8, y1s = y1 >> 8;
            if (i == 0) {
                mma_m16n8k16_first(dl[0], x0 & kLo, y0 & kLo, x1 & kLo, y1 & kLo, p0.x, p1.x);
                mma_m16n8k16_first(dl[1], x0s & kLo, y0s & kLo, x1s & kLo, y1s & kLo, p0.y, p1.y);
                mma_m16n8k16_first(dh[0], x0 & kHi, y0 & kHi, x1 & kHi, y1 & kHi, p0.z, p1.z);
                mma_m16n8k16_first(dh[1], x0s & kHi, y0s & kHi, x1s & kHi, y1s & kHi, p0.w, p1.w);
            } else {
                mma_m16n8k16(dl[0], x0 & kLo, y0 & kLo, x1 & kLo, y1 & kLo, p0.x, p1.x);
                mma_m16n8k16(dl[1], x0s & kLo, y0s & kLo, x1s & kLo, y1s & kLo, p0.y, p1.y);
                mma_m16n8k16(dh[0], x0 & kHi, y0 & kHi, x1 & kHi, y1 & kHi, p0.z, p1.z);
                mma_m16n8k16(dh[1], x0s & kHi, y0s & kHi, x1s & kHi, y1s & kHi, p0.w, p1.w);
            }
        }
    }
    // (d, m) of the blocks behind this lane's two output columns 2c and 2c + 1 (column j * MP + r =
    // block j, activation column r), for channels g and g + 8.  With MP >= 2 both belong to one block.
    constexpr int kBlocksPerLane = MP == 1 ? 2 : 1;
    uint32_t dm[2][kBlocksPerLane];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int q = 0; q < kBlocksPerLane; ++q) {
            const int jb = MP == 1 ? 2 * c + q : (2 * c) / MP;
            // Raw stream: word 0 of the block; packed: entry jb of the (d, m) row.
            dm[half][q] = PACKED ? lds32((half == 0 ? dlo : dhi) + 4u * jb) : lds32((half == 0 ? wlo : whi) + 20u * jb);
        }
    }
    const float2 t = lds_f2(sums_at);
    if (blocks_left < G) {   // warp-uniform and rare: the stage holds no block past the end of K
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int q = 0; q < kBlocksPerLane; ++q) {
                const int jb = MP == 1 ? 2 * c + q : (2 * c) / MP;
                if (jb >= blocks_left) {
                    dm[half][q] = 0u;
                }
            }
        }
    }
    // q-sums in units of 2^-20: entry e = (channel g + 8 * (e >> 1), column 2c + (e & 1)).
    constexpr float kUnit = 1048576.0f;  // 2^20
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float lo = MP == 8 ? dl[0][e] : dl[0][e] + dl[1][e];
        const float hi = MP == 8 ? dh[0][e] : dh[0][e] + dh[1][e];
        const float qsum = fmaf(lo, 16.0f, hi);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&dm[e >> 1][MP == 1 ? (e & 1) : 0]));   // (d, m)
        acc[e] = fmaf(f.x * kUnit, qsum, acc[e]);
        acc[e] = fmaf(f.y, (e & 1) == 0 ? t.x : t.y, acc[e]);
    }
}

// MP: MMA columns per block (activation rows padded to 1, 2, 4 or 8; f32 rows count twice).
// PACKED: `w` is the nibble plane of a packed weight (16 bytes per block) and `w_dm` its (d, m)
// plane with rows dm_pitch_bytes apart; otherwise `w` is the raw 20-byte-block stream.
template <int MP, bool OUT_F16, bool A_F32, int NC, bool PACKED>
__global__ void __launch_bounds__((NC + 2) * 32, NC == 8 ? 2 : 1)
q4_1_gemv_dsq_kernel(const uint8_t* __restrict__ w, const int64_t w_pitch_bytes, const uint8_t* __restrict__ w_dm,
                     const int64_t dm_pitch_bytes, const void* __restrict__ a_v,
                     const int64_t lda, void* __restrict__ out, const int64_t ldc, const int m_count,
                     const int n_total, const int k_total, const DsqLayout lay, const FpEpilogue ep,
                     const int a_vec_ok, int32_t* error_word)
{
    constexpr int G = 8 / MP;
    constexpr int kConsumers = NC;
    constexpr int kProducerWarp = NC;
    constexpr int kReducerWarp = NC + 1;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int abort_word;

    uint64_t* full = reinterpret_cast<uint64_t*>(smem + lay.off_bars);
    uint64_t* empty = full + kMaxStages;
    uint64_t* tile_done = empty + kMaxStages;
    uint64_t* partial_free = tile_done + 2;
    uint32_t* pairs = reinterpret_cast<uint32_t*>(smem + lay.off_pairs);
    float* sums = reinterpret_cast<float*>(smem + lay.off_sums);
    const uint32_t* zero = reinterpret_cast<const uint32_t*>(smem + lay.off_zero);
    float* partial = reinterpret_cast<float*>(smem + lay.off_partial);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // This CTA's channels: an equal, contiguous share of all of them.
    const int row_begin = static_cast<int>(static_cast<int64_t>(blockIdx.x) * n_total / gridDim.x);
    const int row_end = static_cast<int>(static_cast<int64_t>(blockIdx.x + 1) * n_total / gridDim.x);
    const int tiles = (row_end - row_begin + kTileRows - 1) / kTileRows;
    const int nblk = k_total / kQ4BlockElems;
    const int total_stages = tiles * ((nblk + lay.kc_blocks - 1) / lay.kc_blocks);

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
        int slot = 0;
        uint32_t empty_parity = 1;   // a fresh barrier passes a wait on parity 1: the first round needs no wait
        bool ok = true;
        for (int tile = 0; tile < tiles && ok; ++tile) {
            const int r0 = row_begin + tile * kTileRows;
            const int valid = min(kTileRows, row_end - r0);
            const uint8_t* src = w + static_cast<int64_t>(r0 + lane) * w_pitch_bytes;
            for (int b0 = 0; b0 < nblk; b0 += lay.kc_blocks) {
                if (!mbar_wait_all_lanes(&empty[slot], empty_parity, &abort_word)) {
                    atomicCAS(error_word, 0, kErrProducerWait);
                    ok = false;
                    break;
                }
                const uint32_t nb = static_cast<uint32_t>(min(lay.kc_blocks, nblk - b0));
                const uint32_t bytes = nb * (PACKED ? 16u : static_cast<uint32_t>(kQ4BlockBytes));
                if (lane == 0) {
                    mbar_expect_tx(&full[slot], (bytes + (PACKED ? nb * 4u : 0u)) * static_cast<uint32_t>(valid));
                }
                __syncwarp();
                if (lane < valid) {
                    uint8_t* dst = smem + static_cast<size_t>(slot) * lay.stage_bytes;
                    bulk_load_1d(dst + lane * lay.row_stride, src + static_cast<int64_t>(b0) * (PACKED ? 16 : kQ4BlockBytes),
                                 bytes, &full[slot]);
                    if constexpr (PACKED) {
                        bulk_load_1d(dst + lay.dm_off + lane * lay.dm_stride,
                                     w_dm + static_cast<int64_t>(r0 + lane) * dm_pitch_bytes + static_cast<int64_t>(b0) * 4,
                                     nb * 4u, &full[slot]);
                    }
                }
                if (++slot == lay.stages) {
                    slot = 0;
                    empty_parity ^= 1u;
                }
            }
        }
        // No copy may still be in flight when the CTA retires: wait (without consuming) for the
        // latest phase of every slot that was ever filled.
        if (ok) {
            const int used = total_stages < lay.stages ? total_stages : lay.stages;
            for (int q = 0; q < used; ++q) {
                // Slot q was last filled in round ceil((total_stages - q) / stages) - 1.
                const int last_round = (total_stages - q + lay.stages - 1) / lay.stages - 1;
                if (!mbar_wait_all_lanes(&full[q], static_cast<uint32_t>(last_round) & 1u, &abort_word)) {
                    atomicCAS(error_word, 0, kErrDrainWait);
                    break;
                }
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
            if (!mbar_wait_all_lanes(&tile_done[buf], static_cast<uint32_t>(tile >> 1) & 1u, &abort_word)) {
                atomicCAS(error_word, 0, kErrEpilogueWait);
                break;
            }
            const float* part = partial + buf * (kConsumers * kTileRows * MP);
            const int r0 = row_begin + tile * kTileRows;
            for (int idx = lane; idx < kTileRows * m_count; idx += 32) {
                const int r = idx & (kTileRows - 1);
                const int mm = idx / kTileRows;
                // One entry per consumer warp (two for f32 activations: the hi and lo columns),
                // summed in warp order: the result does not depend on timing.
                float sum = 0.0f;
#pragma unroll
                for (int wq = 0; wq < kConsumers; ++wq) {
                    const float* p = part + (wq * kTileRows + r) * MP;
                    sum += A_F32 ? p[2 * mm] + p[2 * mm + 1] : p[mm];
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
        const int tid = threadIdx.x;   // consumer threads only
        if (tid < 32) {
            reinterpret_cast<uint32_t*>(smem + lay.off_zero)[tid] = 0u;   // 128 bytes: four words' worth of zero pairs and more
        }
        const int tasks = lay.nblk_pad * MP * 4;   // (block, column, nibble word); a multiple of 32
        constexpr int kBatch = A_F32 ? 4 : 8;      // words whose loads a thread keeps in flight together
        constexpr int kStep = NC * 32;
        for (int t0 = tid; t0 < tasks; t0 += kStep * kBatch) {
            ActRaw<A_F32> raw[kBatch];
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                const int t = t0 + b * kStep;
                const int col = (t >> 2) % MP;
                const int blk = (t >> 2) / MP;
                const int row = A_F32 ? col >> 1 : col;
                if (t < tasks && blk < nblk && row < m_count) {
                    const void* a_row = static_cast<const uint8_t*>(a_v) + static_cast<int64_t>(row) * lda * (A_F32 ? 4 : 2);
                    raw[b] = load_act_word<A_F32>(a_row, blk * kQ4BlockElems + 4 * (t & 3), a_vec_ok != 0);
                } else {
#pragma unroll
                    for (int q = 0; q < (A_F32 ? 8 : 4); ++q) {
                        raw[b].r[q] = 0u;   // +0.0 in either type: zeros past M and past K
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                const int t = t0 + b * kStep;
                if (t < tasks) {   // warp-uniform: tasks and kStep are multiples of 32
                    const int col = (t >> 2) % MP;
                    float sum;
                    const uint4 v = finish_act_word<A_F32>(raw[b], A_F32 ? (col & 1) : 0, sum);
                    *reinterpret_cast<uint4*>(pairs + static_cast<size_t>(t >> 2) * 16 + 4 * (t & 3)) = v;
                    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
                    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
                    if ((t & 3) == 0) {
                        sums[t >> 2] = sum;
                    }
                }
            }
        }
        named_barrier_sync(1, kConsumers * 32);
    }

    const int g = lane >> 2;
    const int c = lane & 3;
    // Shared-window addresses.  B halves: base + (first block of the group) * stride; lanes whose
    // output column belongs to another block read zeros (stride 0).
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t zero_at = smem_u32(zero);
    uint32_t b_base[2], b_stride[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int blk = MP == 8 ? 0 : DsqLane<MP>::block_of(c, half);
        const int word = MP == 8 ? c : DsqLane<MP>::word_of(c, half);
        const bool live = g / MP == blk;
        b_base[half] = live ? smem_u32(pairs) + static_cast<uint32_t>((blk * MP + g % MP) * 64 + 16 * word) : zero_at;
        b_stride[half] = live ? MP * 64u : 0u;
    }
    const uint32_t sums_base = smem_u32(sums) + 8u * c;
    int slot = 0;
    uint32_t full_parity = 0;
    bool ok = true;
    for (int tile = 0; tile < tiles && ok; ++tile) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int b0 = 0; b0 < nblk; b0 += lay.kc_blocks) {
            if (!mbar_wait_all_lanes(&full[slot], full_parity, &abort_word)) {
                atomicCAS(error_word, 0, kErrMmaWait);
                ok = false;
                break;
            }
            const uint32_t base = smem_base + static_cast<uint32_t>(slot * lay.stage_bytes);
            const uint32_t wlo = base + static_cast<uint32_t>(g * lay.row_stride);
            const uint32_t whi = base + static_cast<uint32_t>((g + 8) * lay.row_stride);
            const uint32_t dlo = base + static_cast<uint32_t>(lay.dm_off + g * lay.dm_stride);
            const uint32_t dhi = base + static_cast<uint32_t>(lay.dm_off + (g + 8) * lay.dm_stride);
            const int nb = min(lay.kc_blocks, nblk - b0);
            constexpr uint32_t kBlk = PACKED ? 16u : 20u;
            for (int ul = warp * G; ul < nb; ul += kConsumers * G) {
                const int ub = b0 + ul;   // the group's first block, counted inside the row
                dsq_group<MP, PACKED>(wlo + kBlk * ul, whi + kBlk * ul, dlo + 4u * ul, dhi + 4u * ul,
                                      b_base[0] + static_cast<uint32_t>(ub) * b_stride[0],
                                      b_base[1] + static_cast<uint32_t>(ub) * b_stride[1],
                                      sums_base + static_cast<uint32_t>(ub) * (MP * 4u), nblk - ub, c, acc);
            }
            __syncwarp();   // every lane has finished reading the stage
            if (lane == 0) {
                mbar_arrive(&empty[slot]);
            }
            if (++slot == lay.stages) {
                slot = 0;
                full_parity ^= 1u;
            }
        }
        if (!ok) {
            break;
        }
        const int buf = tile & 1;
        if (tile >= 2 &&
            !mbar_wait_all_lanes(&partial_free[buf], static_cast<uint32_t>((tile >> 1) - 1) & 1u, &abort_word)) {
            atomicCAS(error_word, 0, kErrAccumWait);
            break;
        }
        // Fold the lanes that hold the same (channel, activation column): entry e is channel
        // g + 8 * (e >> 1), column (2c + (e & 1)) % MP.
        if (MP == 1) {
            acc[0] += acc[1];
            acc[2] += acc[3];
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (MP <= 2) {
                acc[e] += __shfl_xor_sync(0xFFFFFFFFu, acc[e], 1);
            }
            if (MP <= 4) {
                acc[e] += __shfl_xor_sync(0xFFFFFFFFu, acc[e], 2);
            }
        }
        if (c < (MP >= 2 ? MP / 2 : 1)) {
            float* mine_out = partial + (buf * kConsumers + warp) * (kTileRows * MP);
            if (MP == 1) {
                mine_out[g] = acc[0];
                mine_out[g + 8] = acc[2];
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    mine_out[(g + 8 * (e >> 1)) * MP + 2 * c + (e & 1)] = acc[e];
                }
            }
        }
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(&tile_done[buf]);
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
bool plan_layout(int mp, int64_t k, int consumers, bool packed, DsqLayout* out)
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
    off += round_up(2 * consumers * kTileRows * mp * 4, 128);
    l.off_bars = off;
    off += 128;
    const int fixed = off;
    constexpr int kHalfSm = 110 * 1024;
    constexpr int kWholeSm = 224 * 1024;
    const int budgets[2] = {kHalfSm, kWholeSm};
    for (int pass = 0; pass < 2; ++pass) {
        int best_flight = 0, best_kc = 0, best_stages = 0;
        for (int kc = 128; kc >= 16; kc /= 2) {
            const int kcb = kc < l.nblk_pad ? kc : l.nblk_pad;
            // Raw stream: 5 * kcb + 4 words per row = 4 * odd (mod 32) for kcb % 8 == 0, which spreads
            // the eight channels a lane group reads over all banks.  Packed: nibble rows of
            // 16 * kcb + 64 bytes (two rows fill the 128-byte bank span of a quarter-warp's 16-byte
            // loads) and (d, m) rows of 4 * kcb + 32 bytes.
            const int stride = packed ? kcb * 16 + 64 : kcb * kQ4BlockBytes + 16;
            const int dm_stride = packed ? kcb * 4 + 32 : 0;
            const int stage = kTileRows * (stride + dm_stride);
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
            l.row_stride = packed ? best_kc * 16 + 64 : best_kc * kQ4BlockBytes + 16;
            l.dm_stride = packed ? best_kc * 4 + 32 : 0;
            l.dm_off = kTileRows * l.row_stride;
            l.stage_bytes = kTileRows * (l.row_stride + l.dm_stride);
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

using DsqKernel = void (*)(const uint8_t*, int64_t, const uint8_t*, int64_t, const void*, int64_t, void*, int64_t, int, int,
                           int, DsqLayout, FpEpilogue, int, int32_t*);

template <int MP, int NC, bool PACKED>
DsqKernel pick_kernel(bool out_f16, bool a_f32)
{
    if (a_f32) {
        if constexpr (MP >= 2) {
            return out_f16 ? q4_1_gemv_dsq_kernel<MP, true, true, NC, PACKED> : q4_1_gemv_dsq_kernel<MP, false, true, NC, PACKED>;
        } else {
            return nullptr;
        }
    }
    return out_f16 ? q4_1_gemv_dsq_kernel<MP, true, false, NC, PACKED> : q4_1_gemv_dsq_kernel<MP, false, false, NC, PACKED>;
}

template <bool PACKED>
DsqKernel pick_kernel(int mp, bool out_f16, bool a_f32)
{
    switch (mp) {
    case 1: return pick_kernel<1, 8, PACKED>(out_f16, a_f32);
    case 2: return pick_kernel<2, 8, PACKED>(out_f16, a_f32);
    case 4: return pick_kernel<4, 8, PACKED>(out_f16, a_f32);
    default: return pick_kernel<8, 8, PACKED>(out_f16, a_f32);
    }
}

// Consumer warps per CTA.  Eight keep a CTA within half an SM's registers and threads; sixteen
// (with stages twice as long) measured slower on every shape tried.
int consumer_warps()
{
    return 8;
}

}  // namespace

bool q4_1_gemv_dsq_supported(const nnb200_q4_1_args& q)
{
    // Weight rows movable by 16-byte bulk copies (aligned base and pitch, K % 128 == 0) and one
    // pass's activations small enough to stage whole in shared memory.  The planes of a packed
    // weight are 16-byte aligned by construction; their (d, m) rows need ld_dm % 4 == 0.
    const bool packed = q.w_dm != nullptr;
    if (!(q.n <= INT32_MAX && q.k <= INT32_MAX - 128 && (q.k % 128) == 0 &&
          (reinterpret_cast<uintptr_t>(q.w_blocks) & 15u) == 0 && (packed || (q.ldw_blocks % 4) == 0) &&
          (!packed || ((reinterpret_cast<uintptr_t>(q.w_dm) & 15u) == 0 && (q.ld_dm % 4) == 0)))) {
        return false;
    }
    const bool a_f32 = q.a_f16 == 0;
    const int rows_per_pass = a_f32 ? 4 : 8;
    const int first = static_cast<int>(q.m < rows_per_pass ? q.m : rows_per_pass);
    DsqLayout l;
    return plan_layout(columns_per_block(first, a_f32), q.k, consumer_warps(), packed, &l);
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
    const bool packed = q.w_dm != nullptr;
    const uint8_t* w = static_cast<const uint8_t*>(q.w_blocks);
    const int64_t pitch = q.ldw_blocks * (packed ? 16 : kQ4BlockBytes);
    const uint8_t* w_dm = static_cast<const uint8_t*>(q.w_dm);
    const int64_t dm_pitch = q.ld_dm * 4;
    const bool overlap = (q.flags & NNB200_Q4_FLAG_OVERLAP_PREVIOUS) != 0;
    const int tiles = (n + kTileRows - 1) / kTileRows;

    // Opt-in to large dynamic shared memory once per device and kernel variant.
    static std::mutex attr_mutex;
    static bool attr_done[kMaxDevices][4][2][2][2];   // [device][columns][out f16][a f32][packed]
    const int consumers = consumer_warps();

    for (int64_t m0 = 0; m0 < q.m; m0 += rows_per_pass) {
        const int m_count = static_cast<int>(q.m - m0 < rows_per_pass ? q.m - m0 : rows_per_pass);
        const int mp = columns_per_block(m_count, a_f32);
        DsqLayout lay;
        if (!plan_layout(mp, k, consumers, packed, &lay)) {
            return NNB200_UNSUPPORTED;
        }
        DsqKernel kernel = packed ? pick_kernel<true>(mp, out_f16, a_f32) : pick_kernel<false>(mp, out_f16, a_f32);
        if (kernel == nullptr) {
            return NNB200_INTERNAL;
        }
        const int mp_idx = mp == 1 ? 0 : (mp == 2 ? 1 : (mp == 4 ? 2 : 3));
        {
            std::lock_guard<std::mutex> lock(attr_mutex);
            bool& done = attr_done[dev.device][mp_idx][out_f16 ? 1 : 0][a_f32 ? 1 : 0][packed ? 1 : 0];
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
        // Two CTAs per SM when two fit: sixteen consumer warps per SM hide the latencies eight
        // cannot (measured: 43 -> 33 us on 147 MB of weights, 4.9 -> 4.6 us on 10 MB).
        const int ctas = dev.sm_count * (lay.total <= 110 * 1024 ? 2 : 1);
        const unsigned grid = static_cast<unsigned>(tiles < ctas ? tiles : ctas);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3((consumers + 2) * 32);
        cfg.dynamicSmemBytes = static_cast<size_t>(lay.total);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = overlap ? 1 : 0;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, w, pitch, w_dm, dm_pitch, a, q.lda, out, q.ldc, m_count, n, k, lay, ep,
                                                 a_vec_ok, dev.error_word);
        note_launch();
        if (e != cudaSuccess) {
            return NNB200_INTERNAL;
        }
    }
    return NNB200_OK;
}

}  // namespace nnb200
