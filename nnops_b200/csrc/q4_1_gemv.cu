// Q4_1 weight-decode GEMV for decode-sized M (<= 8 rows per pass): a bandwidth kernel.
//
// The CPU twin is the reference's fused small-M route (mma_qblock_trans,
// src/backend/cpu/x86_64/mma_qblock.hpp:144-291): decode each 32-value block on the fly,
// w = fma(q, d, m) in f32, multiply with the activation slice, accumulate in f32 over the
// whole K, one store.  Here one warp owns one output channel n; its lanes stride over the
// row's 20-byte blocks, each lane decoding whole blocks with 32-bit loads and integer nibble
// extraction, partial sums meet in a butterfly of warp shuffles, and lane 0 applies the
// output arithmetic.  Activations are read through L1 (they are at most 8 x K halves and
// shared by every warp).  No tensor cores, no shared memory.
//
// This file also holds the row decoder used by tests and by callers that want the dense
// weight (device twin of pack_q4, include/nnops/detail/q4_1.hpp:152-184).

#include "internal.cuh"
#include "q4_1_common.cuh"

namespace nnb200 {

namespace {

constexpr int kGemvWarps = 4;

template <bool A_F16>
__device__ __forceinline__ float load_act(const void* a, int64_t idx)
{
    if constexpr (A_F16) {
        return __half2float(static_cast<const __half*>(a)[idx]);
    } else {
        return static_cast<const float*>(a)[idx];
    }
}

// Activations for 4 consecutive k of one row as floats (k0 is a multiple of 4).
template <bool A_F16>
__device__ __forceinline__ void load_act4(const void* a, int64_t idx, bool vec_ok, float (&o)[4])
{
    if constexpr (A_F16) {
        if (vec_ok) {
            const uint2 v = __ldg(reinterpret_cast<const uint2*>(static_cast<const __half*>(a) + idx));
            const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
            const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
            o[0] = lo.x; o[1] = lo.y; o[2] = hi.x; o[3] = hi.y;
            return;
        }
    } else {
        if (vec_ok) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(a) + idx));
            o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
            return;
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        o[i] = load_act<A_F16>(a, idx + i);
    }
}

template <int M_TILE, bool A_F16, bool OUT_F16>
__global__ void __launch_bounds__(kGemvWarps * 32)
q4_1_gemv_kernel(const void* __restrict__ a, int64_t lda, const uint8_t* __restrict__ w, int64_t ldw_blocks,
                 void* __restrict__ out, int64_t ldc, int m_count, int64_t n_total, int64_t k_total,
                 const FpEpilogue ep, const int a_vec_ok)
{
    const int lane = threadIdx.x & 31;
    const int64_t n = static_cast<int64_t>(blockIdx.x) * kGemvWarps + (threadIdx.x >> 5);
    if (n >= n_total) {
        return;
    }
    const int64_t nblk = (k_total + kQ4BlockElems - 1) / kQ4BlockElems;
    const uint32_t* row = reinterpret_cast<const uint32_t*>(w + n * ldw_blocks * kQ4BlockBytes);

    float acc[M_TILE];
#pragma unroll
    for (int i = 0; i < M_TILE; ++i) {
        acc[i] = 0.0f;
    }

    for (int64_t b = lane; b < nblk; b += 32) {
        const uint32_t* blk = row + b * kQ4BlockWords;
        const uint32_t dm = __ldg(blk);
        uint32_t qs[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            qs[i] = __ldg(blk + 1 + i);
        }
        const float d = __half2float(__ushort_as_half(static_cast<uint16_t>(dm & 0xFFFFu)));
        const float mn = __half2float(__ushort_as_half(static_cast<uint16_t>(dm >> 16)));
        const int64_t k0 = b * kQ4BlockElems;
        const bool whole = k0 + kQ4BlockElems <= k_total;

        // Decode: word i holds bytes 4i..4i+3 -> values 4i..4i+3 (low) and 16+4i.. (high).
        float wlo[16], whi[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t byte = (qs[i] >> (8 * j)) & 0xFFu;
                wlo[4 * i + j] = fmaf(static_cast<float>(byte & 0xFu), d, mn);
                whi[4 * i + j] = fmaf(static_cast<float>(byte >> 4), d, mn);
            }
        }
#pragma unroll
        for (int r = 0; r < M_TILE; ++r) {
            if (r < m_count) {
                float s = acc[r];
                if (whole) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float av[4];
                        load_act4<A_F16>(a, r * lda + k0 + 4 * i, a_vec_ok != 0, av);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            s = fmaf(av[j], wlo[4 * i + j], s);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float av[4];
                        load_act4<A_F16>(a, r * lda + k0 + 16 + 4 * i, a_vec_ok != 0, av);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            s = fmaf(av[j], whi[4 * i + j], s);
                        }
                    }
                } else {
                    // Last, partial block: only values below K exist.
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (k0 + j < k_total) {
                            s = fmaf(load_act<A_F16>(a, r * lda + k0 + j), wlo[j], s);
                        }
                        if (k0 + 16 + j < k_total) {
                            s = fmaf(load_act<A_F16>(a, r * lda + k0 + 16 + j), whi[j], s);
                        }
                    }
                }
                acc[r] = s;
            }
        }
    }

#pragma unroll
    for (int r = 0; r < M_TILE; ++r) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            acc[r] += __shfl_xor_sync(0xFFFFFFFFu, acc[r], o);
        }
    }
#pragma unroll
    for (int r = 0; r < M_TILE; ++r) {
        if (lane == r && r < m_count) {
            const float v = fp_epilogue_value<OUT_F16>(ep, acc[r], n);
            if constexpr (OUT_F16) {
                static_cast<__half*>(out)[r * ldc + n] = __float2half_rn(v);
            } else {
                static_cast<float*>(out)[r * ldc + n] = v;
            }
        }
    }
}

template <bool OUT_F16>
__global__ void __launch_bounds__(128) q4_1_decode_kernel(const uint8_t* __restrict__ w, int64_t ldw_blocks,
                                                          int64_t rows, int64_t k, void* __restrict__ out,
                                                          int64_t ld_out)
{
    const int64_t nblk = (k + kQ4BlockElems - 1) / kQ4BlockElems;
    const int64_t total = rows * nblk;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / nblk;
        const int64_t b = i - r * nblk;
        const uint32_t* blk = reinterpret_cast<const uint32_t*>(w + (r * ldw_blocks + b) * kQ4BlockBytes);
        const uint32_t dm = blk[0];
        const float d = __half2float(__ushort_as_half(static_cast<uint16_t>(dm & 0xFFFFu)));
        const float mn = __half2float(__ushort_as_half(static_cast<uint16_t>(dm >> 16)));
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
            const uint32_t q = blk[1 + wi];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t byte = (q >> (8 * j)) & 0xFFu;
                const float lo = fmaf(static_cast<float>(byte & 0xFu), d, mn);
                const float hi = fmaf(static_cast<float>(byte >> 4), d, mn);
                const int64_t klo = b * kQ4BlockElems + 4 * wi + j;
                const int64_t khi = klo + 16;
                if (klo < k) {
                    if constexpr (OUT_F16) {
                        static_cast<__half*>(out)[r * ld_out + klo] = __float2half_rn(lo);
                    } else {
                        static_cast<float*>(out)[r * ld_out + klo] = lo;
                    }
                }
                if (khi < k) {
                    if constexpr (OUT_F16) {
                        static_cast<__half*>(out)[r * ld_out + khi] = __float2half_rn(hi);
                    } else {
                        static_cast<float*>(out)[r * ld_out + khi] = hi;
                    }
                }
            }
        }
    }
}

template <int M_TILE>
int launch_gemv_tile(const nnb200_q4_1_args& q, const void* a, void* out, int m_count, const FpEpilogue& ep,
                     cudaStream_t stream)
{
    const unsigned grid = static_cast<unsigned>((q.n + kGemvWarps - 1) / kGemvWarps);
    const int threads = kGemvWarps * 32;
    const uint8_t* w = static_cast<const uint8_t*>(q.w_blocks);
    // Vector activation loads: 8-byte (f16) / 16-byte (f32) alignment of every 4-k group.
    const int a_elem = q.a_f16 ? 2 : 4;
    const int a_vec_ok = ((reinterpret_cast<uintptr_t>(a) % (4 * a_elem)) == 0 && (q.lda % 4) == 0) ? 1 : 0;
    if (q.a_f16 && q.out_f16) {
        q4_1_gemv_kernel<M_TILE, true, true><<<grid, threads, 0, stream>>>(a, q.lda, w, q.ldw_blocks, out, q.ldc, m_count, q.n, q.k, ep, a_vec_ok);
    } else if (q.a_f16) {
        q4_1_gemv_kernel<M_TILE, true, false><<<grid, threads, 0, stream>>>(a, q.lda, w, q.ldw_blocks, out, q.ldc, m_count, q.n, q.k, ep, a_vec_ok);
    } else if (q.out_f16) {
        q4_1_gemv_kernel<M_TILE, false, true><<<grid, threads, 0, stream>>>(a, q.lda, w, q.ldw_blocks, out, q.ldc, m_count, q.n, q.k, ep, a_vec_ok);
    } else {
        q4_1_gemv_kernel<M_TILE, false, false><<<grid, threads, 0, stream>>>(a, q.lda, w, q.ldw_blocks, out, q.ldc, m_count, q.n, q.k, ep, a_vec_ok);
    }
    note_launch();
    return cuda_status(cudaGetLastError());
}

}  // namespace

int launch_q4_1_gemv(const nnb200_q4_1_args& q, const DeviceInfo&, cudaStream_t stream)
{
    FpEpilogue ep;
    ep.alpha = q.alpha;
    ep.bias = q.bias;
    ep.activation = q.activation;
    ep.act_alpha = q.act_alpha;
    ep.act_beta = q.act_beta;
    ep.min_clip = q.min_clip;
    ep.max_clip = q.max_clip;
    const int64_t a_row_bytes = q.lda * (q.a_f16 ? 2 : 4);
    const int64_t o_row_bytes = q.ldc * (q.out_f16 ? 2 : 4);
    // Rows of M are taken eight at a time; decode shapes fit one pass.
    for (int64_t m0 = 0; m0 < q.m; m0 += 8) {
        const int m_count = static_cast<int>(q.m - m0 < 8 ? q.m - m0 : 8);
        const void* a = static_cast<const uint8_t*>(q.a) + m0 * a_row_bytes;
        void* out = static_cast<uint8_t*>(q.out) + m0 * o_row_bytes;
        int st;
        if (m_count == 1) {
            st = launch_gemv_tile<1>(q, a, out, m_count, ep, stream);
        } else if (m_count == 2) {
            st = launch_gemv_tile<2>(q, a, out, m_count, ep, stream);
        } else if (m_count <= 4) {
            st = launch_gemv_tile<4>(q, a, out, m_count, ep, stream);
        } else {
            st = launch_gemv_tile<8>(q, a, out, m_count, ep, stream);
        }
        if (st != NNB200_OK) {
            return st;
        }
    }
    return NNB200_OK;
}

int launch_q4_1_decode(const void* w_blocks, int64_t ldw_blocks, int64_t rows, int64_t k, void* out, int out_f16,
                       int64_t ld_out, cudaStream_t stream)
{
    const int64_t nblk = (k + kQ4BlockElems - 1) / kQ4BlockElems;
    const int64_t total = rows * nblk;
    if (total == 0) {
        return NNB200_OK;
    }
    const unsigned grid = static_cast<unsigned>(total / 128 + 1 < 65535 * 8 ? total / 128 + 1 : 65535 * 8);
    const uint8_t* w = static_cast<const uint8_t*>(w_blocks);
    if (out_f16) {
        q4_1_decode_kernel<true><<<grid, 128, 0, stream>>>(w, ldw_blocks, rows, k, out, ld_out);
    } else {
        q4_1_decode_kernel<false><<<grid, 128, 0, stream>>>(w, ldw_blocks, rows, k, out, ld_out);
    }
    note_launch();
    return cuda_status(cudaGetLastError());
}

}  // namespace nnb200
