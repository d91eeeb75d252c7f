// int8 decode engine (M <= 16): the bandwidth-bound twin of the tensor-core GEMM, for the
// token-by-token phase where every weight byte is used once per call
// (replaces dense_gemm_i8_narrow_kernel + dense_gemm_i8_reduce_kernel, matmul_i8.cuh:93-278).
//
// The whole cost is streaming W [n, k] from HBM once, so the kernel is organised around the
// loads and spends as few issue slots as possible on arithmetic:
//   * One CTA owns 16 consecutive output channels; its 8 warps split K into eighths and
//     combine through shared memory (fixed order: integer sums, deterministic anyway).
//   * Lane (g, c) = (lane / 4, lane % 4) reads 16 bytes of row g and of row g + 8 at byte
//     offset 64 j + 16 c with one 128-bit streaming load each (a quad covers 64 contiguous
//     bytes of a row).  Loads of kUnroll consecutive j are issued back to back before any is
//     consumed: 2 * kUnroll * 16 bytes in flight per lane.
//   * The four words of a load feed two mma.sync.m16n8k32 (s8 x s8 / s8 x u8 -> s32) with the
//     weights as the 16-row operand and the (up to 8, or 2 x 8) activation rows as the n
//     dimension.  The instruction's 32 k-slots split into eight groups of four bytes; which
//     four k's a group carries is free as long as the activation fragment uses the same
//     ones, and activation row g's fragment for this lane is exactly the 16 bytes at the same
//     offset 64 j + 16 c -- so there is no shuffle, no shared-memory staging and no unpacking:
//     3 loads + 2 MMAs per 32 weight bytes and lane.
//   * Activations (M * K bytes, tiny) are read through L1, where they stay resident because
//     the weight loads do not allocate there.
//   * Rows past N and activation rows past M are clamped to the last valid one for the
//     loads; their results are simply not stored.
//
// The epilogue is the shared int8 epilogue, element by element (the output is M * N values).

#include <mutex>

#include "internal.cuh"

namespace nnb200 {

namespace {

constexpr int kRows = 16;    // output channels per CTA = the MMA's m
constexpr int kWarps = 8;    // K slices per CTA
constexpr int kChunk = 64;   // bytes of K per lane-quad step
constexpr int kUnroll = 4;   // steps whose loads are in flight together

__device__ __forceinline__ uint4 ld_stream_16(const void* p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <bool A_UNSIGNED>
__device__ __forceinline__ void mma_m16n8k32(int32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1)
{
    if constexpr (A_UNSIGNED) {
        asm volatile(
            "mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
            "{%0, %1, %2, %3};"
            : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
            "{%0, %1, %2, %3};"
            : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

// M_TILES = 1: activation rows 0..7; 2: rows 0..15 (two MMA column tiles over the same weights).
template <int M_TILES, bool A_UNSIGNED>
__global__ void __launch_bounds__(kWarps * 32, 3) gemm_i8_decode_kernel(const I8Problem p, const I8Epilogue ep)
{
    __shared__ int4 partial[kWarps][M_TILES][32];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;
    const int c = lane & 3;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * kRows;
    const int m_count = static_cast<int>(p.m);

    // This warp's range of 64-byte steps.
    const int steps = static_cast<int>(p.k / kChunk);
    const int per_warp = (steps + kWarps - 1) / kWarps;
    const int s_begin = min(steps, warp * per_warp);
    const int s_end = min(steps, s_begin + per_warp);

    const uint8_t* w = static_cast<const uint8_t*>(p.w);
    const uint8_t* a = static_cast<const uint8_t*>(p.a);
    const int64_t last_row = p.n - 1;
    const uint8_t* w_lo = w + min(n0 + g, last_row) * p.w_stride_n + c * 16;
    const uint8_t* w_hi = w + min(n0 + g + 8, last_row) * p.w_stride_n + c * 16;
    const uint8_t* a_row[M_TILES];
#pragma unroll
    for (int t = 0; t < M_TILES; ++t) {
        a_row[t] = a + static_cast<int64_t>(min(g + 8 * t, m_count - 1)) * p.a_stride_m + c * 16;
    }

    int32_t acc[M_TILES][4];
#pragma unroll
    for (int t = 0; t < M_TILES; ++t) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc[t][i] = 0;
        }
    }

    int s = s_begin;
    for (; s + kUnroll <= s_end; s += kUnroll) {
        uint4 lo[kUnroll], hi[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            lo[u] = ld_stream_16(w_lo + static_cast<int64_t>(s + u) * kChunk);
            hi[u] = ld_stream_16(w_hi + static_cast<int64_t>(s + u) * kChunk);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
            for (int t = 0; t < M_TILES; ++t) {
                const uint4 av = __ldg(reinterpret_cast<const uint4*>(a_row[t] + static_cast<int64_t>(s + u) * kChunk));
                mma_m16n8k32<A_UNSIGNED>(acc[t], lo[u].x, hi[u].x, lo[u].y, hi[u].y, av.x, av.y);
                mma_m16n8k32<A_UNSIGNED>(acc[t], lo[u].z, hi[u].z, lo[u].w, hi[u].w, av.z, av.w);
            }
        }
    }
    for (; s < s_end; ++s) {
        const uint4 lo = ld_stream_16(w_lo + static_cast<int64_t>(s) * kChunk);
        const uint4 hi = ld_stream_16(w_hi + static_cast<int64_t>(s) * kChunk);
#pragma unroll
        for (int t = 0; t < M_TILES; ++t) {
            const uint4 av = __ldg(reinterpret_cast<const uint4*>(a_row[t] + static_cast<int64_t>(s) * kChunk));
            mma_m16n8k32<A_UNSIGNED>(acc[t], lo.x, hi.x, lo.y, hi.y, av.x, av.y);
            mma_m16n8k32<A_UNSIGNED>(acc[t], lo.z, hi.z, lo.w, hi.w, av.z, av.w);
        }
    }

#pragma unroll
    for (int t = 0; t < M_TILES; ++t) {
        partial[warp][t][lane] = make_int4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
    }
    __syncthreads();
    if (warp < M_TILES) {
        const int t = warp;  // warp t finishes activation rows 8t .. 8t+7
        int4 sum = partial[0][t][lane];
#pragma unroll
        for (int wq = 1; wq < kWarps; ++wq) {
            const int4 q = partial[wq][t][lane];
            sum.x += q.x;
            sum.y += q.y;
            sum.z += q.z;
            sum.w += q.w;
        }
        // Fragment layout: (x, y) = channel n0+g, activation rows 2c and 2c+1; (z, w) = channel n0+g+8.
        const int32_t vals[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
        for (int mm = 0; mm < 2; ++mm) {
            const int m = 8 * t + 2 * c + mm;
            if (m < m_count) {
                const I8RowTerms terms = i8_row_terms(ep, m);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int64_t n = n0 + g + 8 * h;
                    if (n < p.n) {
                        i8_store_element(ep, terms, m, n, vals[2 * h + mm]);
                    }
                }
            }
        }
    }
}

}  // namespace

bool decode_i8_supported(const I8Problem& p)
{
    const auto aligned16 = [](uint64_t v) { return (v & 15u) == 0; };
    return p.m >= 1 && p.m <= 16 && p.k >= kChunk && (p.k % kChunk) == 0 && p.k <= INT32_MAX &&
           p.a_stride_k == 1 && p.w_stride_k == 1 && aligned16(reinterpret_cast<uintptr_t>(p.a)) &&
           aligned16(reinterpret_cast<uintptr_t>(p.w)) && aligned16(static_cast<uint64_t>(p.a_stride_m)) &&
           aligned16(static_cast<uint64_t>(p.w_stride_n));
}

int launch_gemm_i8_decode(const I8Problem& p, const I8Epilogue& ep, const DeviceInfo&, cudaStream_t stream)
{
    const unsigned grid = static_cast<unsigned>((p.n + kRows - 1) / kRows);
    const int threads = kWarps * 32;
    if (p.m <= 8) {
        if (p.a_unsigned) {
            gemm_i8_decode_kernel<1, true><<<grid, threads, 0, stream>>>(p, ep);
        } else {
            gemm_i8_decode_kernel<1, false><<<grid, threads, 0, stream>>>(p, ep);
        }
    } else {
        if (p.a_unsigned) {
            gemm_i8_decode_kernel<2, true><<<grid, threads, 0, stream>>>(p, ep);
        } else {
            gemm_i8_decode_kernel<2, false><<<grid, threads, 0, stream>>>(p, ep);
        }
    }
    note_launch();
    return cuda_status(cudaGetLastError());
}

}  // namespace nnb200
