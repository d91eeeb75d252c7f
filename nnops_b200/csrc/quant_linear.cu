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
// Both kernels are pure streaming (5 bytes per element with f32, 3 with f16), so the budget is
// a handful of issue slots per element.  Every thread handles groups of 16 bytes of the
// floating side (4 f32 / 8 f16 elements): one 16-byte access there, one 4- or 8-byte access on
// the integer side, fully coalesced, kUnroll groups in flight before any is touched.  A group
// never straddles a row (the vector path needs inner % group == 0), so its scale / zero point
// are looked up once; the row of a group comes from a multiply-high division by the
// (launch-invariant) groups-per-row.  Rows that break the rule, or misaligned bases, run an
// element-at-a-time kernel with the same arithmetic.

#include <cuda_fp16.h>

#include <climits>
#include <type_traits>

#include "internal.cuh"

namespace nnb200 {

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

// floor(n / d) for n < 2^31 by one multiply-high: with s = ceil(log2 d) and
// m = floor(2^(31+s) / d) + 1, n * m >> (31 + s) is exact (the excess n * e / (d * 2^(31+s)),
// e <= d <= 2^s, stays below 1 / d).  d == 1 is flagged instead (it would need a shift by 31).
struct FastDiv {
    uint32_t mul;
    uint32_t shift;  // s - 1
    uint32_t is_one;
    uint32_t d;
};

FastDiv make_fast_div(uint32_t d)
{
    FastDiv f{0u, 0u, d <= 1u ? 1u : 0u, d};
    if (d > 1u) {
        uint32_t s = 0;
        while ((uint64_t{1} << s) < d) {
            ++s;
        }
        f.mul = static_cast<uint32_t>((uint64_t{1} << (31 + s)) / d + 1);
        f.shift = s - 1;
    }
    return f;
}

__device__ __forceinline__ uint32_t fast_div(uint32_t n, const FastDiv& f)
{
    return f.is_one ? n : (__umulhi(n, f.mul) >> f.shift);
}

struct QuantView {
    const void* x;
    void* y;
    int64_t outer, rows, inner;
    const float* scale;
    const void* zero_point;
    int32_t zp_unsigned;
};

// zp_unsigned carries NNB200_ZP_*: s8, u8 or int32 storage of the zero points.
__device__ __forceinline__ float load_zp(const QuantView& v, int64_t r)
{
    if (v.zp_unsigned == NNB200_ZP_S32) {
        return static_cast<float>(static_cast<const int32_t*>(v.zero_point)[r]);
    }
    return v.zp_unsigned == NNB200_ZP_U8 ? static_cast<float>(static_cast<const uint8_t*>(v.zero_point)[r])
                                         : static_cast<float>(static_cast<const int8_t*>(v.zero_point)[r]);
}

// fma, round-half-even with saturation to the 8-bit range in one conversion; the x86
// conversion sends NaN and anything at or above 2^31 to INT32_MIN, i.e. to the range's lower
// end, where a saturating conversion would give 0 / the upper end: patch those.
template <bool OUT_U8>
__device__ __forceinline__ uint32_t quant_one(float x, float inv, float zp)
{
    const float v = __fmaf_rn(x, inv, zp);
    int32_t q;
    if constexpr (OUT_U8) {
        asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(q) : "f"(v));
        q = (v < 2147483648.0f) ? q : 0;
    } else {
        asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(v));
        q = (v < 2147483648.0f) ? q : -128;
    }
    return static_cast<uint32_t>(q) & 0xFFu;
}

template <bool OUT_U8>
__device__ __forceinline__ uint32_t quant_four(float a, float b, float c, float d, float inv, float zp)
{
    return quant_one<OUT_U8>(a, inv, zp) | (quant_one<OUT_U8>(b, inv, zp) << 8) |
           (quant_one<OUT_U8>(c, inv, zp) << 16) | (quant_one<OUT_U8>(d, inv, zp) << 24);
}

template <bool IN_U8>
__device__ __forceinline__ float int8_to_float(uint32_t word, int byte)
{
    const uint32_t b = (word >> (8 * byte)) & 0xFFu;
    return IN_U8 ? static_cast<float>(b) : static_cast<float>(static_cast<int8_t>(b));
}

template <bool IN_U8>
__device__ __forceinline__ float dequant_one(uint32_t word, int byte, float scale, float zp, float neg_zs, bool tail)
{
    const float q = int8_to_float<IN_U8>(word, byte);
    return tail ? __fmul_rn(__fsub_rn(q, zp), scale) : __fmaf_rn(q, scale, neg_zs);
}

// Row parameter index r and in-row offset (in elements) of `group`.  IDX = uint32_t uses the
// multiply-high division (fewer than 2^31 groups); uint64_t divides.
template <typename IDX, int VEC>
__device__ __forceinline__ void locate(const QuantView& v, const FastDiv& per_row, const FastDiv& by_rows, IDX group,
                                       int64_t& r, int64_t& i0)
{
    if (v.rows == 1 && v.outer == 1) {
        r = 0;
        i0 = static_cast<int64_t>(group) * VEC;
        return;
    }
    if constexpr (std::is_same_v<IDX, uint32_t>) {
        const uint32_t row = fast_div(group, per_row);
        i0 = static_cast<int64_t>(group - row * per_row.d) * VEC;
        r = v.outer == 1 ? row : row - fast_div(row, by_rows) * by_rows.d;
    } else {
        const uint64_t gpr = static_cast<uint64_t>(v.inner / VEC);
        const uint64_t row = group / gpr;
        i0 = static_cast<int64_t>(group - row * gpr) * VEC;
        r = static_cast<int64_t>(row % static_cast<uint64_t>(v.rows));
    }
}

// VEC = elements per 16 bytes of x: 4 (f32) or 8 (f16).
template <bool X_F16, bool OUT_U8, typename IDX>
__global__ void __launch_bounds__(kThreads)
quantize_vec_kernel(const QuantView v, const IDX groups, const FastDiv per_row, const FastDiv by_rows)
{
    constexpr int VEC = X_F16 ? 8 : 4;
    const IDX stride = static_cast<IDX>(gridDim.x) * kThreads;
    for (IDX base = static_cast<IDX>(blockIdx.x) * kThreads + threadIdx.x; base < groups; base += stride * kUnroll) {
        uint4 raw[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const IDX gidx = base + static_cast<IDX>(u) * stride;
            if (gidx < groups) {
                raw[u] = __ldcs(static_cast<const uint4*>(v.x) + gidx);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const IDX gidx = base + static_cast<IDX>(u) * stride;
            if (gidx < groups) {
                int64_t r, i0;
                locate<IDX, VEC>(v, per_row, by_rows, gidx, r, i0);
                const float inv = __frcp_rn(v.scale[r]);  // correctly rounded: identical to 1.0f / scale
                const float zp = load_zp(v, r);
                if constexpr (X_F16) {
                    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw[u].x));
                    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw[u].y));
                    const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&raw[u].z));
                    const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&raw[u].w));
                    uint2 out;
                    out.x = quant_four<OUT_U8>(a.x, a.y, b.x, b.y, inv, zp);
                    out.y = quant_four<OUT_U8>(c.x, c.y, d.x, d.y, inv, zp);
                    __stcs(static_cast<uint2*>(v.y) + gidx, out);
                } else {
                    const uint32_t out = quant_four<OUT_U8>(__uint_as_float(raw[u].x), __uint_as_float(raw[u].y),
                                                            __uint_as_float(raw[u].z), __uint_as_float(raw[u].w), inv, zp);
                    __stcs(static_cast<uint32_t*>(v.y) + gidx, out);
                }
            }
        }
    }
}

// VEC = elements per 16 bytes of y: 4 (f32) or 8 (f16).
template <bool IN_U8, bool Y_F16, typename IDX>
__global__ void __launch_bounds__(kThreads)
dequantize_vec_kernel(const QuantView v, const IDX groups, const FastDiv per_row, const FastDiv by_rows)
{
    constexpr int VEC = Y_F16 ? 8 : 4;
    const IDX stride = static_cast<IDX>(gridDim.x) * kThreads;
    const int64_t body = v.inner - v.inner % 16;
    for (IDX base = static_cast<IDX>(blockIdx.x) * kThreads + threadIdx.x; base < groups; base += stride * kUnroll) {
        uint2 raw[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const IDX gidx = base + static_cast<IDX>(u) * stride;
            if (gidx < groups) {
                if constexpr (Y_F16) {
                    raw[u] = __ldcs(static_cast<const uint2*>(v.x) + gidx);
                } else {
                    raw[u] = make_uint2(__ldcs(static_cast<const uint32_t*>(v.x) + gidx), 0u);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const IDX gidx = base + static_cast<IDX>(u) * stride;
            if (gidx < groups) {
                int64_t r, i0;
                locate<IDX, VEC>(v, per_row, by_rows, gidx, r, i0);
                const float s = v.scale[r];
                const float zp = load_zp(v, r);
                const float neg_zs = __fmul_rn(-zp, s);
                const bool tail = i0 >= body;  // body is a multiple of 16, i0 of VEC: the whole group agrees
                float f[VEC];
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    f[j] = dequant_one<IN_U8>(j < 4 ? raw[u].x : raw[u].y, j & 3, s, zp, neg_zs, tail);
                }
                if constexpr (Y_F16) {
                    uint4 out;
                    const __half2 h0 = __floats2half2_rn(f[0], f[1]);
                    const __half2 h1 = __floats2half2_rn(f[2], f[3]);
                    const __half2 h2 = __floats2half2_rn(f[4 % VEC], f[5 % VEC]);
                    const __half2 h3 = __floats2half2_rn(f[6 % VEC], f[7 % VEC]);
                    out.x = *reinterpret_cast<const uint32_t*>(&h0);
                    out.y = *reinterpret_cast<const uint32_t*>(&h1);
                    out.z = *reinterpret_cast<const uint32_t*>(&h2);
                    out.w = *reinterpret_cast<const uint32_t*>(&h3);
                    __stcs(static_cast<uint4*>(v.y) + gidx, out);
                } else {
                    __stcs(static_cast<float4*>(v.y) + gidx, make_float4(f[0], f[1], f[2], f[3]));
                }
            }
        }
    }
}

// Element-at-a-time forms for rows whose length breaks the group rule or misaligned bases.
template <bool X_F16, bool OUT_U8>
__global__ void __launch_bounds__(kThreads) quantize_scalar_kernel(const QuantView v, const int64_t numel)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; e < numel; e += stride) {
        const int64_t row = e / v.inner;
        const int64_t r = row % v.rows;
        const float x = X_F16 ? __half2float(static_cast<const __half*>(v.x)[e]) : static_cast<const float*>(v.x)[e];
        static_cast<uint8_t*>(v.y)[e] = static_cast<uint8_t>(quant_one<OUT_U8>(x, __frcp_rn(v.scale[r]), load_zp(v, r)));
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
        const float f = dequant_one<IN_U8>(static_cast<const uint8_t*>(v.x)[e], 0, s, zp, __fmul_rn(-zp, s), i >= body);
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

// Divisors of the 32-bit path: groups per row, and rows (for the outer wrap).
void make_divisors(const QuantView& v, int vec, int64_t groups, FastDiv& per_row, FastDiv& by_rows)
{
    const bool small = groups <= 0x7FFFFFFF;
    per_row = make_fast_div(small ? static_cast<uint32_t>(v.inner / vec) : 1u);
    by_rows = make_fast_div(small && v.rows <= 0x7FFFFFFF ? static_cast<uint32_t>(v.rows) : 1u);
}

template <bool X_F16, bool OUT_U8>
int run_quantize(const QuantView& v, int64_t numel, bool vec_ok, const DeviceInfo& dev, cudaStream_t stream)
{
    constexpr int VEC = X_F16 ? 8 : 4;
    const int64_t groups = numel / VEC;
    FastDiv per_row, by_rows;
    make_divisors(v, VEC, groups, per_row, by_rows);
    if (!vec_ok) {
        quantize_scalar_kernel<X_F16, OUT_U8><<<grid_for(numel, dev), kThreads, 0, stream>>>(v, numel);
    } else if (groups <= 0x7FFFFFFF) {
        quantize_vec_kernel<X_F16, OUT_U8, uint32_t>
            <<<grid_for(groups, dev), kThreads, 0, stream>>>(v, static_cast<uint32_t>(groups), per_row, by_rows);
    } else {
        quantize_vec_kernel<X_F16, OUT_U8, uint64_t>
            <<<grid_for(groups, dev), kThreads, 0, stream>>>(v, static_cast<uint64_t>(groups), per_row, by_rows);
    }
    note_launch();
    return cuda_status(cudaGetLastError());
}

template <bool IN_U8, bool Y_F16>
int run_dequantize(const QuantView& v, int64_t numel, bool vec_ok, const DeviceInfo& dev, cudaStream_t stream)
{
    constexpr int VEC = Y_F16 ? 8 : 4;
    const int64_t groups = numel / VEC;
    FastDiv per_row, by_rows;
    make_divisors(v, VEC, groups, per_row, by_rows);
    if (!vec_ok) {
        dequantize_scalar_kernel<IN_U8, Y_F16><<<grid_for(numel, dev), kThreads, 0, stream>>>(v, numel);
    } else if (groups <= 0x7FFFFFFF) {
        dequantize_vec_kernel<IN_U8, Y_F16, uint32_t>
            <<<grid_for(groups, dev), kThreads, 0, stream>>>(v, static_cast<uint32_t>(groups), per_row, by_rows);
    } else {
        dequantize_vec_kernel<IN_U8, Y_F16, uint64_t>
            <<<grid_for(groups, dev), kThreads, 0, stream>>>(v, static_cast<uint64_t>(groups), per_row, by_rows);
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
    // 16 bytes of x per group: 4 f32 -> 4 bytes of y, 8 f16 -> 8 bytes of y.
    const bool vec = (q.inner % (f16 ? 8 : 4)) == 0 && aligned_to(q.x, 16) && aligned_to(q.y, f16 ? 8 : 4);
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
    const bool vec = (q.inner % (f16 ? 8 : 4)) == 0 && aligned_to(q.x, f16 ? 8 : 4) && aligned_to(q.y, 16);
    if (u8) {
        return f16 ? run_dequantize<true, true>(v, numel, vec, dev, stream)
                   : run_dequantize<true, false>(v, numel, vec, dev, stream);
    }
    return f16 ? run_dequantize<false, true>(v, numel, vec, dev, stream)
               : run_dequantize<false, false>(v, numel, vec, dev, stream);
}

}  // namespace nnb200
