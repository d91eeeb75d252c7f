// int8 engines that do not use the tensor cores:
//
//   * generic  -- any pose (either operand k-contiguous or not), any alignment, any shape.
//                 A small shared-memory tile per CTA; the correctness tier that the
//                 tensor-core engine's alignment rules fall back to (the reference keeps a
//                 byte-fill tier for the same reason, matmul_i8_ptx.cuh:112-162).
//   * narrow   -- M <= 16 decode shapes with k-contiguous operands: a bandwidth kernel, one
//                 warp per output channel, 16-byte weight loads, dp4a, warp-shuffle reduce
//                 (replaces dense_gemm_i8_narrow_kernel, matmul_i8.cuh:93-253).
//   * sums     -- R_a[m] = sum_k A[m][k], R_w[n] = sum_k W[n][k] for zero-point compensation
//                 (replaces i8_row_sums_kernel / i8_col_sums_kernel, matmul_i8_common.cuh:270-350).

#include "internal.cuh"

namespace nnb200 {

namespace {

constexpr int kTile = 32;
constexpr int kTileK = 32;

template <bool A_UNSIGNED>
__global__ void __launch_bounds__(256) gemm_i8_generic_kernel(const I8Problem p, const I8Epilogue ep)
{
    __shared__ int32_t a_s[kTile][kTileK + 1];
    __shared__ int32_t w_s[kTile][kTileK + 1];

    const int tx = threadIdx.x & 15;
    const int ty = threadIdx.x >> 4;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kTile;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * kTile;
    const uint8_t* a = static_cast<const uint8_t*>(p.a);
    const int8_t* w = static_cast<const int8_t*>(p.w);

    int32_t acc[2][2] = {{0, 0}, {0, 0}};
    for (int64_t k0 = 0; k0 < p.k; k0 += kTileK) {
        for (int i = threadIdx.x; i < kTile * kTileK; i += 256) {
            // Walk the k-contiguous direction fastest when there is one.
            const int r = p.a_stride_k == 1 ? i / kTileK : i % kTile;
            const int c = p.a_stride_k == 1 ? i % kTileK : i / kTile;
            int32_t v = 0;
            if (m0 + r < p.m && k0 + c < p.k) {
                const uint8_t raw = a[(m0 + r) * p.a_stride_m + (k0 + c) * p.a_stride_k];
                v = A_UNSIGNED ? static_cast<int32_t>(raw) : static_cast<int32_t>(static_cast<int8_t>(raw));
            }
            a_s[r][c] = v;
        }
        for (int i = threadIdx.x; i < kTile * kTileK; i += 256) {
            const int r = p.w_stride_k == 1 ? i / kTileK : i % kTile;
            const int c = p.w_stride_k == 1 ? i % kTileK : i / kTile;
            int32_t v = 0;
            if (n0 + r < p.n && k0 + c < p.k) {
                v = w[(n0 + r) * p.w_stride_n + (k0 + c) * p.w_stride_k];
            }
            w_s[r][c] = v;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < kTileK; ++kk) {
            const int32_t a0 = a_s[ty][kk], a1 = a_s[ty + 16][kk];
            const int32_t w0 = w_s[tx][kk], w1 = w_s[tx + 16][kk];
            acc[0][0] += a0 * w0;
            acc[0][1] += a0 * w1;
            acc[1][0] += a1 * w0;
            acc[1][1] += a1 * w1;
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int64_t m = m0 + ty + 16 * i;
        if (m >= p.m) {
            continue;
        }
        const I8RowTerms t = i8_row_terms(ep, m);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int64_t n = n0 + tx + 16 * j;
            if (n < p.n) {
                i8_store_element(ep, t, m, n, acc[i][j]);
            }
        }
    }
}

// One block per row of a [rows, k] int8 matrix with arbitrary strides.
template <bool UNSIGNED>
__global__ void __launch_bounds__(128) i8_sums_kernel(const uint8_t* x, int64_t rows, int64_t k, int64_t stride_row,
                                                      int64_t stride_k, int32_t* out)
{
    const int64_t r = blockIdx.x;
    const uint8_t* row = x + r * stride_row;
    int32_t s = 0;
    if (stride_k == 1 && (reinterpret_cast<uintptr_t>(row) & 3u) == 0) {
        const int64_t k4 = k / 4;
        const uint32_t* row4 = reinterpret_cast<const uint32_t*>(row);
        for (int64_t i = threadIdx.x; i < k4; i += blockDim.x) {
            const uint32_t v = row4[i];
            s = UNSIGNED ? __dp4a(v, 0x01010101u, static_cast<uint32_t>(s))
                         : __dp4a(static_cast<int32_t>(v), 0x01010101, s);
        }
        for (int64_t i = k4 * 4 + threadIdx.x; i < k; i += blockDim.x) {
            s += UNSIGNED ? static_cast<int32_t>(row[i]) : static_cast<int32_t>(static_cast<int8_t>(row[i]));
        }
    } else {
        for (int64_t i = threadIdx.x; i < k; i += blockDim.x) {
            const uint8_t v = row[i * stride_k];
            s += UNSIGNED ? static_cast<int32_t>(v) : static_cast<int32_t>(static_cast<int8_t>(v));
        }
    }
    __shared__ int32_t part[4];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    }
    if ((threadIdx.x & 31) == 0) {
        part[threadIdx.x >> 5] = s;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        out[r] = part[0] + part[1] + part[2] + part[3];
    }
}

// ---- narrow-M decode engine ---------------------------------------------------------------

constexpr int kNarrowWarps = 8;

// One warp per output channel n.  The lane strides over W's row in 16-byte pieces and, for
// every piece, over the M activation rows (read through L1; they are tiny and shared by all
// warps).  s8 x s8 uses dp4a directly; a u8 A is taken as stored by the unsigned/signed dp4a
// form, so no sign shift and no extra compensation term is needed.
template <int M_MAX, bool A_UNSIGNED>
__global__ void __launch_bounds__(kNarrowWarps * 32) gemm_i8_narrow_kernel(const I8Problem p, const I8Epilogue ep)
{
    const int lane = threadIdx.x & 31;
    const int64_t n = static_cast<int64_t>(blockIdx.x) * kNarrowWarps + (threadIdx.x >> 5);
    if (n >= p.n) {
        return;
    }
    const uint8_t* a = static_cast<const uint8_t*>(p.a);
    const uint8_t* wrow = static_cast<const uint8_t*>(p.w) + n * p.w_stride_n;
    const int m_count = static_cast<int>(p.m);

    int32_t acc[M_MAX];
#pragma unroll
    for (int i = 0; i < M_MAX; ++i) {
        acc[i] = 0;
    }
    const int64_t k16 = p.k / 16;
    for (int64_t c = lane; c < k16; c += 32) {
        const uint4 wv = *reinterpret_cast<const uint4*>(wrow + c * 16);
#pragma unroll
        for (int i = 0; i < M_MAX; ++i) {
            if (i < m_count) {
                const uint4 av = *reinterpret_cast<const uint4*>(a + i * p.a_stride_m + c * 16);
                if (A_UNSIGNED) {
                    // dp4a(unsigned, signed): first operand unsigned bytes, second signed bytes
                    int32_t s = acc[i];
                    asm("dp4a.u32.s32 %0, %1, %2, %0;" : "+r"(s) : "r"(av.x), "r"(wv.x));
                    asm("dp4a.u32.s32 %0, %1, %2, %0;" : "+r"(s) : "r"(av.y), "r"(wv.y));
                    asm("dp4a.u32.s32 %0, %1, %2, %0;" : "+r"(s) : "r"(av.z), "r"(wv.z));
                    asm("dp4a.u32.s32 %0, %1, %2, %0;" : "+r"(s) : "r"(av.w), "r"(wv.w));
                    acc[i] = s;
                } else {
                    int32_t s = acc[i];
                    s = __dp4a(static_cast<int32_t>(av.x), static_cast<int32_t>(wv.x), s);
                    s = __dp4a(static_cast<int32_t>(av.y), static_cast<int32_t>(wv.y), s);
                    s = __dp4a(static_cast<int32_t>(av.z), static_cast<int32_t>(wv.z), s);
                    s = __dp4a(static_cast<int32_t>(av.w), static_cast<int32_t>(wv.w), s);
                    acc[i] = s;
                }
            }
        }
    }
    // k tail (k % 16), byte at a time.
    for (int64_t kk = k16 * 16 + lane; kk < p.k; kk += 32) {
        const int32_t wv = static_cast<int8_t>(wrow[kk]);
#pragma unroll
        for (int i = 0; i < M_MAX; ++i) {
            if (i < m_count) {
                const uint8_t raw = a[i * p.a_stride_m + kk];
                acc[i] += wv * (A_UNSIGNED ? static_cast<int32_t>(raw) : static_cast<int32_t>(static_cast<int8_t>(raw)));
            }
        }
    }
#pragma unroll
    for (int i = 0; i < M_MAX; ++i) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            acc[i] += __shfl_xor_sync(0xFFFFFFFFu, acc[i], o);
        }
    }
    // Lane i finishes row i.
#pragma unroll
    for (int i = 0; i < M_MAX; ++i) {
        if (lane == i && i < m_count) {
            const I8RowTerms t = i8_row_terms(ep, i);
            i8_store_element(ep, t, i, n, acc[i]);
        }
    }
}

}  // namespace

int launch_gemm_i8_generic(const I8Problem& p, const I8Epilogue& ep, const DeviceInfo&, cudaStream_t stream)
{
    const dim3 grid(static_cast<unsigned>((p.n + kTile - 1) / kTile), static_cast<unsigned>((p.m + kTile - 1) / kTile));
    if (grid.y > 65535u) {
        return NNB200_UNSUPPORTED;
    }
    if (p.a_unsigned) {
        gemm_i8_generic_kernel<true><<<grid, 256, 0, stream>>>(p, ep);
    } else {
        gemm_i8_generic_kernel<false><<<grid, 256, 0, stream>>>(p, ep);
    }
    note_launch();
    return cuda_status(cudaGetLastError());
}

bool narrow_i8_supported(const I8Problem& p)
{
    const auto aligned16 = [](uint64_t v) { return (v & 15u) == 0; };
    return p.m >= 1 && p.m <= 16 && p.k >= 256 && p.a_stride_k == 1 && p.w_stride_k == 1 &&
           aligned16(reinterpret_cast<uintptr_t>(p.a)) && aligned16(reinterpret_cast<uintptr_t>(p.w)) &&
           aligned16(static_cast<uint64_t>(p.a_stride_m)) && aligned16(static_cast<uint64_t>(p.w_stride_n));
}

int launch_gemm_i8_narrow(const I8Problem& p, const I8Epilogue& ep, const DeviceInfo&, cudaStream_t stream)
{
    const unsigned grid = static_cast<unsigned>((p.n + kNarrowWarps - 1) / kNarrowWarps);
    const int threads = kNarrowWarps * 32;
#define NNB200_NARROW(MM)                                                          \
    do {                                                                           \
        if (p.a_unsigned) {                                                        \
            gemm_i8_narrow_kernel<MM, true><<<grid, threads, 0, stream>>>(p, ep);  \
        } else {                                                                   \
            gemm_i8_narrow_kernel<MM, false><<<grid, threads, 0, stream>>>(p, ep); \
        }                                                                          \
    } while (0)
    if (p.m <= 1) {
        NNB200_NARROW(1);
    } else if (p.m <= 2) {
        NNB200_NARROW(2);
    } else if (p.m <= 4) {
        NNB200_NARROW(4);
    } else if (p.m <= 8) {
        NNB200_NARROW(8);
    } else {
        NNB200_NARROW(16);
    }
#undef NNB200_NARROW
    note_launch();
    return cuda_status(cudaGetLastError());
}

int launch_i8_sums(const I8Problem& p, int32_t* r_a, int32_t* r_w, cudaStream_t stream)
{
    // Either destination may be null: that sweep is skipped.
    const uint8_t* a = static_cast<const uint8_t*>(p.a);
    const uint8_t* w = static_cast<const uint8_t*>(p.w);
    if (r_a != nullptr) {
        if (p.a_unsigned) {
            i8_sums_kernel<true><<<static_cast<unsigned>(p.m), 128, 0, stream>>>(a, p.m, p.k, p.a_stride_m, p.a_stride_k, r_a);
        } else {
            i8_sums_kernel<false><<<static_cast<unsigned>(p.m), 128, 0, stream>>>(a, p.m, p.k, p.a_stride_m, p.a_stride_k, r_a);
        }
    }
    if (r_w != nullptr) {
        i8_sums_kernel<false><<<static_cast<unsigned>(p.n), 128, 0, stream>>>(w, p.n, p.k, p.w_stride_n, p.w_stride_k, r_w);
    }
    note_launch((r_a != nullptr ? 1 : 0) + (r_w != nullptr ? 1 : 0));
    return cuda_status(cudaGetLastError());
}

}  // namespace nnb200
