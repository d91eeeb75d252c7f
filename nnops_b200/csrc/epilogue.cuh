// The int8 route's output arithmetic, shared by every int8 engine so they cannot drift
// apart.  It restates, step for step, the reference's CPU epilogue
// (src/backend/cpu/simd_kernel/simd_epilogue.hpp:129-160, 341-467): every f32 operation is
// spelled with an explicit round-to-nearest intrinsic so the compiler cannot contract a
// multiply and an add into an FMA -- integer outputs are compared byte for byte.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/nnb200.h"

namespace nnb200 {

// Everything an engine's epilogue needs besides the accumulator, by value in kernel params.
struct I8Epilogue {
    void* out;
    int64_t ldc;            // elements
    int32_t out_kind;       // NNB200_OUT_*
    const void* bias;       // int32 (integer destinations) | f32 | f16
    int32_t relu;
    int32_t activation;
    float act_alpha, act_beta;
    float min_clip, max_clip;
    const float* scale_a;   // [m] or null
    const float* scale_w;   // [n] or null
    const int32_t* zp_a;    // [m] or null
    const int32_t* zp_w;    // [n] or null
    float scale_a_scalar, scale_w_scalar;
    int32_t zp_a_scalar, zp_w_scalar;
    int32_t compensate;     // any zero point may be non-zero: r_a / r_w are valid
    const int32_t* r_a;     // [m]  sum_k A[m][k]; may be null when every weight zero point is 0
    const int32_t* r_w;     // [n]  sum_k W[n][k]; may be null when every activation zero point is 0
    int32_t k;
    float out_scale;
    int32_t out_zp;
    // Column-sharded output written straight into every rank's full matrix: `out` is this
    // rank's own copy, `peer_out[i]` the same window (same pitch) inside the other ranks'
    // buffers, mapped into this process for peer-to-peer stores.  8-bit destinations only.
    int32_t num_peers;
    void* peer_out[7];
    // The same window inside a multicast mapping bound to every rank's copy (this rank's too):
    // tiles are stored once with multimem.st and replicated by the switch; peer_out is unused.
    void* mc_out;
    // Set by the tensor-core launcher, not by callers: this many entries of peer_out are written
    // with plain 32-byte stores from the ordinary epilogue (two-rank shards on the CTA-pair
    // kernel), and num_peers is 0.
    int32_t direct_peers;
};

__device__ __forceinline__ float act_apply(int32_t act, float alpha, float beta, float x)
{
    switch (act) {
    case NNB200_ACT_RELU: return fmaxf(x, 0.0f);
    case NNB200_ACT_RELU6: return fminf(fmaxf(x, 0.0f), 6.0f);
    case NNB200_ACT_LEAKY_RELU: return x > 0.0f ? x : alpha * x;
    case NNB200_ACT_SIGMOID: return 1.0f / (1.0f + expf(-x));
    case NNB200_ACT_TANH: return tanhf(x);
    case NNB200_ACT_GELU: {
        const float c = 0.7978845608028654f;
        return 0.5f * x * (1.0f + tanhf(c * (x + 0.044715f * x * x * x)));
    }
    case NNB200_ACT_SILU: return x / (1.0f + expf(-x));
    case NNB200_ACT_HARD_SWISH: {
        const float r = fminf(fmaxf(x + 3.0f, 0.0f), 6.0f);
        return x * r * (beta / 6.0f);
    }
    case NNB200_ACT_ELU: return x > 0.0f ? x : alpha * (expf(x) - 1.0f);
    default: return x;
    }
}

// raw - zp_a*R_w[n] - zp_w*R_a[m] + K*zp_a*zp_w, wrapping int32 (matmul_int8_compensate).
__device__ __forceinline__ int32_t i8_compensate(int32_t raw, int32_t zpa, int32_t zpw, int32_t ra, int32_t rw,
                                                 int32_t k)
{
    uint32_t v = static_cast<uint32_t>(raw);
    v -= static_cast<uint32_t>(zpa) * static_cast<uint32_t>(rw);
    v -= static_cast<uint32_t>(zpw) * static_cast<uint32_t>(ra);
    v += static_cast<uint32_t>(k) * static_cast<uint32_t>(zpa) * static_cast<uint32_t>(zpw);
    return static_cast<int32_t>(v);
}

// Requantise: f32 product, f32 clamp, x + copysign(0.5, x) rounded in f32, truncate, + zp.
// lo / hi are the destination range already shifted by the zero point.
__device__ __forceinline__ int32_t i8_requant(int32_t v, float req, float lo, float hi, int32_t zp_out)
{
    float x = __fmul_rn(__int2float_rn(v), req);
    x = fminf(fmaxf(x, lo), hi);
    const float r = truncf(__fadd_rn(x, copysignf(0.5f, x)));
    return static_cast<int32_t>(r) + zp_out;
}

// Per-row constants of the epilogue.
struct I8RowTerms {
    int32_t zpa;
    int32_t ra;
    float s_a;
    float row_k;  // s_a / out_scale, one f32 division per row
};

__device__ __forceinline__ I8RowTerms i8_row_terms(const I8Epilogue& e, int64_t m)
{
    I8RowTerms t;
    t.zpa = e.zp_a != nullptr ? e.zp_a[m] : e.zp_a_scalar;
    t.ra = (e.compensate && e.r_a != nullptr) ? e.r_a[m] : 0;   // null: every weight zero point is 0
    t.s_a = e.scale_a != nullptr ? e.scale_a[m] : e.scale_a_scalar;
    t.row_k = __fdiv_rn(t.s_a, e.out_scale);
    return t;
}

// Integer value of one element after compensation, bias and Relu.
__device__ __forceinline__ int32_t i8_int_value(const I8Epilogue& e, const I8RowTerms& t, int32_t raw, int32_t zpw,
                                                int32_t rw, int32_t bias)
{
    int32_t v = raw;
    if (e.compensate) {
        v = i8_compensate(raw, t.zpa, zpw, t.ra, rw, e.k);
    }
    v = static_cast<int32_t>(static_cast<uint32_t>(v) + static_cast<uint32_t>(bias));
    if (e.relu && v < 0) {
        v = 0;
    }
    return v;
}

// fp destination value: dequantise, add a non-zero bias, clip, activate.
__device__ __forceinline__ float i8_fp_value(const I8Epilogue& e, const I8RowTerms& t, int32_t raw, int32_t zpw,
                                             int32_t rw, float s_w, float bias)
{
    int32_t v = raw;
    if (e.compensate) {
        v = i8_compensate(raw, t.zpa, zpw, t.ra, rw, e.k);
    }
    float f = __fmul_rn(__int2float_rn(v), __fmul_rn(t.s_a, s_w));
    if (bias != 0.0f) {
        f = __fadd_rn(f, bias);
    }
    f = fminf(fmaxf(f, e.min_clip), e.max_clip);
    return act_apply(e.activation, e.act_alpha, e.act_beta, f);
}

// One element, loads its own column terms, scalar store.  The slow-path form used by the
// generic and narrow engines and by ragged edges of the tensor-core engine.
__device__ __forceinline__ void i8_store_element(const I8Epilogue& e, const I8RowTerms& t, int64_t m, int64_t n,
                                                 int32_t raw)
{
    const int32_t zpw = e.zp_w != nullptr ? e.zp_w[n] : e.zp_w_scalar;
    const int32_t rw = (e.compensate && e.r_w != nullptr) ? e.r_w[n] : 0;
    const float s_w = e.scale_w != nullptr ? e.scale_w[n] : e.scale_w_scalar;
    const int64_t idx = m * e.ldc + n;
    if (e.out_kind <= NNB200_OUT_U8) {
        const int32_t b = e.bias != nullptr ? static_cast<const int32_t*>(e.bias)[n] : 0;
        const int32_t v = i8_int_value(e, t, raw, zpw, rw, b);
        if (e.out_kind == NNB200_OUT_S32) {
            static_cast<int32_t*>(e.out)[idx] = v;
        } else {
            const float req = __fmul_rn(t.row_k, s_w);
            const float zpf = static_cast<float>(e.out_zp);
            if (e.out_kind == NNB200_OUT_S8) {
                static_cast<int8_t*>(e.out)[idx] =
                    static_cast<int8_t>(i8_requant(v, req, -128.0f - zpf, 127.0f - zpf, e.out_zp));
            } else {
                static_cast<uint8_t*>(e.out)[idx] =
                    static_cast<uint8_t>(i8_requant(v, req, 0.0f - zpf, 255.0f - zpf, e.out_zp));
            }
        }
    } else {
        float b = 0.0f;
        if (e.bias != nullptr) {
            b = e.out_kind == NNB200_OUT_F32 ? static_cast<const float*>(e.bias)[n]
                                             : __half2float(static_cast<const __half*>(e.bias)[n]);
        }
        const float f = i8_fp_value(e, t, raw, zpw, rw, s_w, b);
        if (e.out_kind == NNB200_OUT_F32) {
            static_cast<float*>(e.out)[idx] = f;
        } else {
            static_cast<__half*>(e.out)[idx] = __float2half_rn(f);
        }
    }
}

}  // namespace nnb200
