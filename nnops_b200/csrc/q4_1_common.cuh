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

}  // namespace nnb200
