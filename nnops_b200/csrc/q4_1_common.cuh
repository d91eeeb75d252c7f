// Q4_1 helpers shared by the decode, GEMV and GEMM kernels.  Block layout (20 bytes,
// 4-byte aligned): {f16 d, f16 m, 16 bytes qs}; byte j carries value j in its low nibble and
// value j+16 in its high nibble; w = d*q + m
// (reference include/nnops/detail/q4_1.hpp:53-79).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>

#include "epilogue.cuh"

namespace nnb200 {

constexpr int kQ4BlockBytes = 20;
constexpr int kQ4BlockElems = 32;
constexpr int kQ4BlockWords = 5;

// Output-side arithmetic of the fp routes: alpha, bias, clip, activation
// (reference matmul semantics: src/backend/cpu/matmul/matmul.cpp:443-483).
struct FpEpilogue {
    float alpha;
    const void* bias;  // output type
    int32_t activation;
    float act_alpha, act_beta;
    float min_clip, max_clip;
};

// True when the output arithmetic is the identity (alpha 1, no bias, no clip, no activation):
// callers test it once per tile and skip fp_epilogue_value altogether.
__device__ __forceinline__ bool fp_epilogue_is_identity(const FpEpilogue& e)
{
    return e.alpha == 1.0f && e.bias == nullptr && e.activation == NNB200_ACT_NONE && e.min_clip == -INFINITY &&
           e.max_clip == INFINITY;
}

template <bool OUT_F16>
__device__ __forceinline__ float fp_epilogue_value(const FpEpilogue& e, float acc, int64_t n)
{
    float v = acc;
    if (e.alpha != 1.0f) {
        v *= e.alpha;
    }
    if (e.bias != nullptr) {
        v += OUT_F16 ? __half2float(static_cast<const __half*>(e.bias)[n]) : static_cast<const float*>(e.bias)[n];
    }
    v = fminf(fmaxf(v, e.min_clip), e.max_clip);
    return act_apply(e.activation, e.act_alpha, e.act_beta, v);
}

// The same value with the run-time switches turned into operands, for loops over many elements:
// alpha is always multiplied in (x * 1.0f is x), a missing bias adds -0.0f (x + -0.0f is x for
// every x, -0 included), and the activation class -- 0 none, 1 Relu, 2 any other -- is a
// template argument chosen once outside the loop.
template <bool OUT_F16, int ACT>
__device__ __forceinline__ float fp_epilogue_value_flat(const FpEpilogue& e, float acc, int64_t n)
{
    float b = -0.0f;
    if (e.bias != nullptr) {
        b = OUT_F16 ? __half2float(static_cast<const __half*>(e.bias)[n]) : static_cast<const float*>(e.bias)[n];
    }
    float v = __fadd_rn(__fmul_rn(acc, e.alpha), b);
    v = fminf(fmaxf(v, e.min_clip), e.max_clip);
    if constexpr (ACT == 1) {
        v = fmaxf(v, 0.0f);
    } else if constexpr (ACT == 2) {
        v = act_apply(e.activation, e.act_alpha, e.act_beta, v);
    }
    return v;
}

// 32 consecutive columns of one row: accumulator bits in, output values (f32) out.  `identity`
// (fp_epilogue_is_identity, tested once per tile by the caller) passes the accumulator through.
template <bool OUT_F16>
__device__ __forceinline__ void fp_epilogue_chunk(const FpEpilogue& e, bool identity, const uint32_t (&v)[32], int n0,
                                                  int n_total, float (&o)[32])
{
    if (identity) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            o[j] = __uint_as_float(v[j]);
        }
        return;
    }
    const int act_class = e.activation == NNB200_ACT_NONE ? 0 : (e.activation == NNB200_ACT_RELU ? 1 : 2);
    if (act_class == 0) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            o[j] = fp_epilogue_value_flat<OUT_F16, 0>(e, __uint_as_float(v[j]), min(n0 + j, n_total - 1));
        }
    } else if (act_class == 1) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            o[j] = fp_epilogue_value_flat<OUT_F16, 1>(e, __uint_as_float(v[j]), min(n0 + j, n_total - 1));
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            o[j] = fp_epilogue_value_flat<OUT_F16, 2>(e, __uint_as_float(v[j]), min(n0 + j, n_total - 1));
        }
    }
}

// Two nibble-carrying words (8 bytes of qs) -> 8 consecutive f16 weights of the low nibbles
// and 8 of the high nibbles, each as a uint4 of four half2.
__device__ __forceinline__ void dequant_word_pair(uint32_t w0, uint32_t w1, __half2 d2, __half2 m2, uint4& lo,
                                                  uint4& hi)
{
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
    const uint32_t magic = 0x64646464u;
    uint32_t lo_out[4], hi_out[4];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const uint32_t w = i == 0 ? w0 : w1;
        const uint32_t x = w & 0x0F0F0F0Fu;
        const uint32_t y = (w >> 4) & 0x0F0F0F0Fu;
        // bytes (n0, 0x64, n1, 0x64) = half2(1024 + n0, 1024 + n1)
        const uint32_t x01 = __byte_perm(x, magic, 0x4140);
        const uint32_t x23 = __byte_perm(x, magic, 0x4342);
        const uint32_t y01 = __byte_perm(y, magic, 0x4140);
        const uint32_t y23 = __byte_perm(y, magic, 0x4342);
        const __half2 q0 = __hsub2(*reinterpret_cast<const __half2*>(&x01), k1024);
        const __half2 q1 = __hsub2(*reinterpret_cast<const __half2*>(&x23), k1024);
        const __half2 q2 = __hsub2(*reinterpret_cast<const __half2*>(&y01), k1024);
        const __half2 q3 = __hsub2(*reinterpret_cast<const __half2*>(&y23), k1024);
        const __half2 r0 = __hfma2(q0, d2, m2);
        const __half2 r1 = __hfma2(q1, d2, m2);
        const __half2 r2 = __hfma2(q2, d2, m2);
        const __half2 r3 = __hfma2(q3, d2, m2);
        lo_out[2 * i] = *reinterpret_cast<const uint32_t*>(&r0);
        lo_out[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&r1);
        hi_out[2 * i] = *reinterpret_cast<const uint32_t*>(&r2);
        hi_out[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&r3);
    }
    lo = make_uint4(lo_out[0], lo_out[1], lo_out[2], lo_out[3]);
    hi = make_uint4(hi_out[0], hi_out[1], hi_out[2], hi_out[3]);
}

}  // namespace nnb200
