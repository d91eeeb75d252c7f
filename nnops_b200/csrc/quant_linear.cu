// QuantizeLinear / DequantizeLinear: the elementwise steps either side of an int8 Linear in a
// W8A8 graph.  The reference declares the CUDA entry points but leaves them as
// Status::unsupported stubs (src/backend/cuda/not_implemented.cu:28-37); the arithmetic
// implemented here is the one of its CPU route (src/backend/cpu/quant_linear.cpp:80-262 over
// the arch kernels src/backend/cpu/x86_64/quant.hpp:117-165, 278-325), bit for bit:
//
//   quantize:   inv = 1.0f / scale;  v = fma(x, inv, zp) (one rounding);  q = round-half-even
//               to int32 where NaN and anything outside int32 become INT32_MIN (the x86
//               conversion's "integer indefinite");  saturate to s8 / u8.
//   dequantize: elements in the first (inner - inner % 16) positions of a row:
//                   fma(float(q), scale, -(zp * scale))
//               the remaining inner % 16 (the CPU kernel's scalar tail):
//                   (float(q) - zp) * scale
//               -- the two forms round differently, and the position rule is part of the
//               reference's observable behaviour.
//
// The tensor is a flat row-major array viewed as [outer][rows][inner]; parameter r serves row
// r of every outer group (per tensor: [1][1][numel]; per token: [1][numel/last][last]; per
// channel: [outer][shape[axis]][inner]).
//
// Both kernels are pure streaming (5 bytes per element with f32, 3 with f16): every thread
// handles groups of four consecutive elements -- one 16-byte (f32) / 8-byte (f16) / 4-byte
// (int8) access each way, fully coalesced -- and has kUnroll groups in flight before it
// touches any.  A group never straddles a row (the vector path needs inner % 4 == 0), so its
// scale / zero point are looked up once.  Rows that break the rule, or misaligned bases, run
// an element-at-a-time kernel with the same arithmetic.

#include <cuda_fp16.h>

#include <climits>

#include "internal.cuh"

namespace nnb200 {

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

struct QuantView {
    const void* x;
    void* y;
    int64_t outer, rows, inner;
    const float* scale;
    const void* zero_point;
    int32_t zp_unsigned;
};

__device__ __forceinline__ float load_zp(const QuantView& v, int64_t r)
{
    return v.zp_unsigned ? static_cast<float>(static_cast<const uint8_t*>(v.zero_point)[r])
                         : static_cast<float>(static_cast<const int8_t*>(v.zero_point)[r]);
}

template <bool OUT_U8>
__device__ __forceinline__ uint32_t quant_one(float x, float inv, float zp)
{
    const float v = __fmaf_rn(x, inv, zp);
    int32_t q = (v >= -2147483648.0f && v < 2147483648.0f) ? __float2int_rn(v) : INT_MIN;
    if constexpr (OUT_U8) {
        q = min(max(q, 0), 255);
    } else {
        q = min(max(q, -128), 127);
    }
    return static_cast<uint32_t>(q) & 0xFFu;
}

template <bool IN_U8>
__device__ __forceinline__ float dequant_one(uint32_t byte, float scale, float zp, float neg_zs, bool tail)
{
    const float q = IN_U8 ? static_cast<float>(byte) : static_cast<float>(static_cast<int8_t>(byte));
    return tail ? __fmul_rn(__fsub_rn(q, zp), scale) : __fmaf_rn(q, scale, neg_zs);
}

// Parameter row of the group that starts at flat element 4 * group.  IDX is uint32_t when the
// tensor has fewer than 2^32 elements (two cheap divisions), uint64_t otherwise.
template <typename IDX>
__device__ __forceinline__ void locate(const QuantView& v, IDX groups_per_row, IDX group, int64_t& r, int64_t& i0)
{
    if (v.rows == 1 && v.outer == 1) {
        r = 0;
        i0 = static_cast<int64_t>(group) * 4;
        return;
    }
    const IDX row = group / groups_per_row;
    i0 = static_cast<int64_t>(group - row * groups_per_row) * 4;
    r = v.outer == 1 ? static_cast<int64_t>(row) : static_cast<int64_t>(row % static_cast<IDX>(v.rows));
}

template <bool X_F16, bool OUT_U8, typename IDX>
__global__ void __launch_bounds__(kThreads) quantize_vec_kernel(const QuantView v, const IDX groups)
{
    const IDX groups_per_row = static_cast<IDX>(v.inner / 4);
    const IDX stride = static_cast<IDX>(gridDim.x) * kThreads;
    uint32_t* y = static_cast<uint32_t*>(v.y);
    for (IDX base = static_cast<IDX>(blockIdx.x) * kThreads + threadIdx.x; base < groups; base += stride * kUnroll) {
        float4 xv[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const IDX gidx = base + static_cast<IDX>(u) * stride;
            if (gidx < groups) {
                if constexpr (X_F16) {
                    const uint2 raw = __ldcs(static_cast<const uint2*>(v.x) + gidx);
                    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                    xv[u] = make_float4(lo.x, lo.y, hi.x, hi.y);
                } else {
                    xv[u] = __ldcs(static_cast<const float4*>(v.x) + gidx);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const IDX gidx = base + static_cast<IDX>(u) * stride;
            if (gidx < groups) {
                int64_t r, i0;
                locate<IDX>(v, groups_per_row, gidx, r, i0);
                const float inv = __fdiv_rn(1.0f, v.scale[r]);
                const float zp = load_zp(v, r);
                const uint32_t packed = quant_one<OUT_U8>(xv[u].x, inv, zp) | (quant_one<OUT_U8>(xv[u].y, inv, zp) << 8) |
                                        (quant_one<OUT_U8>(xv[u].z, inv, zp) << 16) |
                                        (quant_one<OUT_U8>(xv[u].w, inv, zp) << 24);
                __stcs(y + gidx, packed);
            }
        }
    }
}

template <bool IN_U8, bool Y_F16, typename IDX>
__global__ void __launch_bounds__(kThreads) dequantize_vec_kernel(const QuantView v, const IDX groups)
{
    const IDX groups_per_row = static_cast<IDX>(v.inner / 4);
    const IDX stride = static_cast<IDX>(gridDim.x) * kThreads;
    const int64_t body = v.inner - v.inner % 16;
    const uint32_t* x = static_cast<const uint32_t*>(v.x);
    for (IDX base = static_cast<IDX>(blockIdx.x) * kThreads + threadIdx.x; base < groups; base += stride * kUnroll) {
        uint32_t xv[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const IDX gidx = base + static_cast<IDX>(u) * stride;
            if (gidx < groups) {
                xv[u] = __ldcs(x + gidx);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const IDX gidx = base + static_cast<IDX>(u) * stride;
            if (gidx < groups) {
                int64_t r, i0;
                locate<IDX>(v, groups_per_row, gidx, r, i0);
                const float s = v.scale[r];
                const float zp = load_zp(v, r);
                const float neg_zs = __fmul_rn(-zp, s);
                const bool tail = i0 >= body;  // body is a multiple of 16, i0 of 4: all four agree
                const float f0 = dequant_one<IN_U8>(xv[u] & 0xFFu, s, zp, neg_zs, tail);
                const float f1 = dequant_one<IN_U8>((xv[u] >> 8) & 0xFFu, s, zp, neg_zs, tail);
                const float f2 = dequant_one<IN_U8>((xv[u] >> 16) & 0xFFu, s, zp, neg_zs, tail);
                const float f3 = dequant_one<IN_U8>(xv[u] >> 24, s, zp, neg_zs, tail);
                if constexpr (Y_F16) {
                    const __half2 h01 = __floats2half2_rn(f0, f1);
                    const __half2 h23 = __floats2half2_rn(f2, f3);
                    uint2 out;
                    out.x = *reinterpret_cast<const uint32_t*>(&h01);
                    out.y = *reinterpret_cast<const uint32_t*>(&h23);
                    __stcs(static_cast<uint2*>(v.y) + gidx, out);
                } else {
                    __stcs(static_cast<float4*>(v.y) + gidx, make_float4(f0, f1, f2, f3));
                }
            }
        }
    }
}

// Element-at-a-time forms for rows whose length is not a multiple of 4 or misaligned bases.
template <bool X_F16, bool OUT_U8>
__global__ void __launch_bounds__(kThreads) quantize_scalar_kernel(const QuantView v, const int64_t numel)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; e < numel; e += stride) {
        const int64_t row = e / v.inner;
        const int64_t r = row % v.rows;
        const float x = X_F16 ? __half2float(static_cast<const __half*>(v.x)[e]) : static_cast<const float*>(v.x)[e];
        static_cast<uint8_t*>(v.y)[e] =
            static_cast<uint8_t>(quant_one<OUT_U8>(x, __fdiv_rn(1.0f, v.scale[r]), load_zp(v, r)));
    }
}

template <bool IN_U8, bool Y_F16>
__global__ void __launch_bounds__(kThreads) dequantize_scalar_kernel(const QuantView v, const int64_t numel)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    const int64_t body = v.inner - v.inner % 16;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; e < numel; e += stride) {
        const int64_t row = e / v.inner;
        const int64_t r = row % v.rows;
        const int64_t i = e - row * v.inner;
        const float s = v.scale[r];
        const float zp = load_zp(v, r);
        const float f = dequant_one<IN_U8>(static_cast<const uint8_t*>(v.x)[e], s, zp, __fmul_rn(-zp, s), i >= body);
        if constexpr (Y_F16) {
            static_cast<__half*>(v.y)[e] = __float2half_rn(f);
        } else {
            static_cast<float*>(v.y)[e] = f;
        }
    }
}

unsigned grid_for(int64_t work_items, const DeviceInfo& dev)
{
    const int64_t per_block = static_cast<int64_t>(kThreads) * kUnroll;
    const int64_t want = (work_items + per_block - 1) / per_block;
    const int64_t cap = static_cast<int64_t>(dev.sm_count) * 16;  // a few waves of resident CTAs; the loop strides
    return static_cast<unsigned>(want < 1 ? 1 : (want > cap ? cap : want));
}

bool aligned_to(const void* p, uintptr_t a)
{
    return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

template <bool X_F16, bool OUT_U8>
int run_quantize(const QuantView& v, int64_t numel, bool vec, const DeviceInfo& dev, cudaStream_t stream)
{
    if (!vec) {
        quantize_scalar_kernel<X_F16, OUT_U8><<<grid_for(numel, dev), kThreads, 0, stream>>>(v, numel);
    } else if (numel / 4 <= 0x7FFFFFFF) {
        quantize_vec_kernel<X_F16, OUT_U8, uint32_t>
            <<<grid_for(numel / 4, dev), kThreads, 0, stream>>>(v, static_cast<uint32_t>(numel / 4));
    } else {
        quantize_vec_kernel<X_F16, OUT_U8, uint64_t>
            <<<grid_for(numel / 4, dev), kThreads, 0, stream>>>(v, static_cast<uint64_t>(numel / 4));
    }
    note_launch();
    return cuda_status(cudaGetLastError());
}

template <bool IN_U8, bool Y_F16>
int run_dequantize(const QuantView& v, int64_t numel, bool vec, const DeviceInfo& dev, cudaStream_t stream)
{
    if (!vec) {
        dequantize_scalar_kernel<IN_U8, Y_F16><<<grid_for(numel, dev), kThreads, 0, stream>>>(v, numel);
    } else if (numel / 4 <= 0x7FFFFFFF) {
        dequantize_vec_kernel<IN_U8, Y_F16, uint32_t>
            <<<grid_for(numel / 4, dev), kThreads, 0, stream>>>(v, static_cast<uint32_t>(numel / 4));
    } else {
        dequantize_vec_kernel<IN_U8, Y_F16, uint64_t>
            <<<grid_for(numel / 4, dev), kThreads, 0, stream>>>(v, static_cast<uint64_t>(numel / 4));
    }
    note_launch();
    return cuda_status(cudaGetLastError());
}

}  // namespace

int launch_quantize_linear(const nnb200_quant_linear_args& q, const DeviceInfo& dev, cudaStream_t stream)
{
    const QuantView v{q.x, q.y, q.outer, q.rows, q.inner, q.scale, q.zero_point, q.zp_unsigned};
    const int64_t numel = q.outer * q.rows * q.inner;
    const bool f16 = q.float_f16 != 0;
    const bool u8 = q.int_unsigned != 0;
    const bool vec = (q.inner % 4) == 0 && aligned_to(q.x, f16 ? 8 : 16) && aligned_to(q.y, 4);
    if (f16) {
        return u8 ? run_quantize<true, true>(v, numel, vec, dev, stream)
                  : run_quantize<true, false>(v, numel, vec, dev, stream);
    }
    return u8 ? run_quantize<false, true>(v, numel, vec, dev, stream)
              : run_quantize<false, false>(v, numel, vec, dev, stream);
}

int launch_dequantize_linear(const nnb200_quant_linear_args& q, const DeviceInfo& dev, cudaStream_t stream)
{
    const QuantView v{q.x, q.y, q.outer, q.rows, q.inner, q.scale, q.zero_point, q.zp_unsigned};
    const int64_t numel = q.outer * q.rows * q.inner;
    const bool f16 = q.float_f16 != 0;
    const bool u8 = q.int_unsigned != 0;
    const bool vec = (q.inner % 4) == 0 && aligned_to(q.x, 4) && aligned_to(q.y, f16 ? 8 : 16);
    if (u8) {
        return f16 ? run_dequantize<true, true>(v, numel, vec, dev, stream)
                   : run_dequantize<true, false>(v, numel, vec, dev, stream);
    }
    return f16 ? run_dequantize<false, true>(v, numel, vec, dev, stream)
               : run_dequantize<false, false>(v, numel, vec, dev, stream);
}

}  // namespace nnb200
