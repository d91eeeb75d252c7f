// C entry points around the UNMODIFIED nnops reference CPU route.  TEST INFRASTRUCTURE
// ONLY: built by oracle/build.py into oracle/_ref/libnnops_ref_<isa>.so from the reference's
// own sources (read in place, never copied), and used to (1) validate the plain-C
// restatement in nnops_oracle.c, (2) generate tests/golden/ fixtures, and (3) serve as the
// timed host-CPU baseline ("kind": "reference").  The shipped CUDA path never loads it.
//
// Everything here goes through the reference's public operator API exactly as a caller
// would: Linear::create / MatMul::create / Conv2D::create(attrs, Backend::CPU) ->
// compute(out, inputs, ctx), with an OpenMP parallel_for injected through ComputeContext::cpu.

#include "nnops/core/openmp_backend.hpp"
#include "nnops/ops/conv2d.hpp"
#include "nnops/ops/linear.hpp"
#include "nnops/ops/matmul.hpp"
#include "nnops/ops/quant_linear.hpp"
#include "nnops/detail/q4_1.hpp"

#include <cstdint>
#include <cstring>

using namespace nnops;

namespace {

// Field-for-field twin of oracle_gemm_i8_args in nnops_oracle.c.
struct GemmI8Args {
    const void* a;
    const int8_t* w;
    void* out;
    int64_t m, n, k;
    int64_t a_stride_m, a_stride_k, w_stride_n, w_stride_k, ldc;
    int32_t a_unsigned;
    int32_t out_kind;
    const void* bias;
    int32_t relu;
    const float* scale_a;
    const float* scale_w;
    const int32_t* zp_a;
    const int32_t* zp_w;
    float scale_a_scalar, scale_w_scalar;
    int32_t zp_a_scalar, zp_w_scalar;
    float out_scale;
    int32_t out_zp;
    float min_clip, max_clip;
};

DataType out_dtype(int kind)
{
    switch (kind) {
    case 0: return DataType::s32;
    case 1: return DataType::s8;
    case 2: return DataType::u8;
    case 3: return DataType::f32;
    default: return DataType::f16;
    }
}

QuantParams make_qp(const float* s, const int32_t* z, float s0, int32_t z0, int64_t count,
                    QuantGranularity g)
{
    QuantParams q;
    q.scale = s0;
    q.zero_point = z0;
    if (s != nullptr || z != nullptr) {
        q.granularity = g;
        q.scale_data = s;
        q.zero_point_data = z;
        q.num_scales = count;
    }
    return q;
}

ComputeContext make_ctx(int threads)
{
    ComputeContext ctx;
    if (threads > 1) {
        ctx.cpu = openmp_backend(threads);
    }
    return ctx;
}

} // namespace

extern "C" {

/// int8 Linear / MatMul through the reference op.  use_linear != 0 requires the NT pose
/// (A [M,K], W [N,K]) and calls Linear; otherwise MatMul with the transposes the strides imply.
int ref_gemm_i8(const GemmI8Args* p, int use_linear, int threads)
{
    const bool ta = p->a_stride_k != 1;   // A stored [K, M]
    const bool tb = p->w_stride_k == 1;   // W stored [N, K]
    const int64_t a_shape[2] = {ta ? p->k : p->m, ta ? p->m : p->k};
    const int64_t w_shape[2] = {tb ? p->n : p->k, tb ? p->k : p->n};
    const int64_t o_shape[2] = {p->m, p->n};
    // a_unsigned doubles as the activation dtype selector: 0 = s8, 1 = u8, 2 = f32, 3 = f16 (the
    // fp-activation route: A is quantised on the fly with the parameters given for A).
    const DataType adt = p->a_unsigned == 3 ? DataType::f16
                         : p->a_unsigned == 2 ? DataType::f32
                         : p->a_unsigned == 1 ? DataType::u8
                                              : DataType::s8;
    const int64_t a_elem = int64_t(data_type_size(adt));
    const DataType odt = out_dtype(p->out_kind);

    TensorView a(a_shape, adt, const_cast<void*>(p->a), (ta ? p->a_stride_k : p->a_stride_m) * a_elem,
                 TensorLayout::Dense,
                 make_qp(p->scale_a, p->zp_a, p->scale_a_scalar, p->zp_a_scalar, p->m,
                         QuantGranularity::PerToken));
    TensorView w(w_shape, DataType::s8, const_cast<int8_t*>(p->w), tb ? p->w_stride_n : p->w_stride_k,
                 TensorLayout::Dense,
                 make_qp(p->scale_w, p->zp_w, p->scale_w_scalar, p->zp_w_scalar, p->n,
                         QuantGranularity::PerChannel));
    QuantParams oq;
    oq.scale = p->out_scale;
    oq.zero_point = p->out_zp;
    TensorView out(o_shape, odt, p->out, p->ldc * int64_t(data_type_size(odt)), TensorLayout::Dense, oq);

    const int64_t b_shape[1] = {p->n};
    const DataType bdt = p->out_kind <= 2 ? DataType::s32 : odt;
    TensorView bias(b_shape, bdt, const_cast<void*>(p->bias));

    Epilogue ep;
    ep.type = p->relu ? EpilogueActivateType::Relu : EpilogueActivateType::None;
    ep.min_clip = p->min_clip;
    ep.max_clip = p->max_clip;

    const ComputeContext ctx = make_ctx(threads);
    TensorView ins[3] = {a, w, bias};
    const std::span<const TensorView> in_span(ins, p->bias ? 3 : 2);

    Status st;
    if (use_linear) {
        if (ta || !tb) {
            return int(Status::invalid_argument);
        }
        LinearAttributes attrs;
        attrs.output_dtype = odt;
        attrs.epilogue = ep;
        auto op = Linear::create(attrs, Backend::CPU);
        st = op->compute(out, in_span, ctx, nullptr);
    } else {
        MatMulAttributes attrs;
        attrs.transpose_a = ta;
        attrs.transpose_b = tb;
        attrs.output_dtype = odt;
        attrs.epilogue = ep;
        auto op = MatMul::create(attrs, Backend::CPU);
        st = op->compute(out, in_span, ctx, nullptr);
    }
    return int(st);
}

/// Linear(f32|f16 activations x q4_1 weights [N,K]) through the reference op.  The output
/// dtype equals the activation dtype (the reference's only fp pose).
int ref_linear_q4_1(const void* x, int x_is_f16, int64_t m, int64_t k, int64_t x_pitch_bytes,
                    const void* w_blocks, int64_t n, int64_t w_pitch_bytes, const void* bias,
                    void* out, int64_t out_pitch_bytes, int threads)
{
    const DataType dt = x_is_f16 ? DataType::f16 : DataType::f32;
    const int64_t x_shape[2] = {m, k};
    const int64_t w_shape[2] = {n, k};
    const int64_t o_shape[2] = {m, n};
    const int64_t b_shape[1] = {n};
    TensorView xv(x_shape, dt, const_cast<void*>(x), x_pitch_bytes);
    TensorView wv(w_shape, DataType::q4_1, const_cast<void*>(w_blocks), w_pitch_bytes);
    TensorView ov(o_shape, dt, out, out_pitch_bytes);
    TensorView bv(b_shape, dt, const_cast<void*>(bias));
    LinearAttributes attrs;
    attrs.output_dtype = dt;
    auto op = Linear::create(attrs, Backend::CPU);
    const ComputeContext ctx = make_ctx(threads);
    TensorView ins[3] = {xv, wv, bv};
    return int(op->compute(ov, std::span<const TensorView>(ins, bias ? 3 : 2), ctx, nullptr));
}

/// Reference Q4_1 codec, for pinning the restated codec.
void ref_q4_1_decode(const void* blocks, int64_t count, float* out) { pack_q4<float>(blocks, count, out); }
void ref_q4_1_quantize(const float* src, int64_t count, void* blocks) { quantize_q4<float>(src, count, blocks); }

/// QuantizeLinear / DequantizeLinear through the reference ops.  `shape`/`rank` describe the
/// dense tensor, `axis` and `param_count` select the granularity exactly as the op does
/// (count 1 = per tensor, axis < 0 = one parameter per innermost row, else per index of axis).
int ref_quantize_linear(const void* x, int x_is_f16, const int64_t* shape, int rank, int64_t axis,
                        const float* scale, const void* zero_point, int zp_is_u8, int64_t param_count,
                        void* y, int y_is_u8, int threads)
{
    const std::span<const int64_t> sh(shape, size_t(rank));
    const int64_t p_shape[1] = {param_count};
    TensorView xv(sh, x_is_f16 ? DataType::f16 : DataType::f32, const_cast<void*>(x));
    TensorView sv(p_shape, DataType::f32, const_cast<float*>(scale));
    TensorView zv(p_shape, zp_is_u8 ? DataType::u8 : DataType::s8, const_cast<void*>(zero_point));
    TensorView yv(sh, y_is_u8 ? DataType::u8 : DataType::s8, y);
    QuantLinearAttributes attrs;
    attrs.axis = axis;
    attrs.output_dtype = y_is_u8 ? DataType::u8 : DataType::s8;
    auto op = QuantizeLinear::create(attrs, Backend::CPU);
    const ComputeContext ctx = make_ctx(threads);
    TensorView ins[3] = {xv, sv, zv};
    return int(op->compute(yv, std::span<const TensorView>(ins, 3), ctx, nullptr));
}

int ref_dequantize_linear(const void* x, int x_is_u8, const int64_t* shape, int rank, int64_t axis,
                          const float* scale, const void* zero_point, int zp_is_u8, int64_t param_count,
                          void* y, int y_is_f16, int threads)
{
    const std::span<const int64_t> sh(shape, size_t(rank));
    const int64_t p_shape[1] = {param_count};
    TensorView xv(sh, x_is_u8 ? DataType::u8 : DataType::s8, const_cast<void*>(x));
    TensorView sv(p_shape, DataType::f32, const_cast<float*>(scale));
    TensorView zv(p_shape, zp_is_u8 ? DataType::u8 : DataType::s8, const_cast<void*>(zero_point));
    TensorView yv(sh, y_is_f16 ? DataType::f16 : DataType::f32, y);
    QuantLinearAttributes attrs;
    attrs.axis = axis;
    attrs.output_dtype = y_is_f16 ? DataType::f16 : DataType::f32;
    auto op = DequantizeLinear::create(attrs, Backend::CPU);
    const ComputeContext ctx = make_ctx(threads);
    TensorView ins[3] = {xv, sv, zv};
    return int(op->compute(yv, std::span<const TensorView>(ins, 3), ctx, nullptr));
}

/// int8 Conv2D through the reference op: dense NHWC u8/s8 activation [n, ih, iw, ic], dense s8
/// HWIO filter [kh, kw, ic/groups, oc], dense NHWC output.  geom = {n, ih, iw, ic, oc, kh, kw,
/// stride_h, stride_w, dil_h, dil_w, pad_h, pad_w, groups, oh, ow}.  The call pattern is the
/// reference's own CUDA-vs-CPU test (tests/test_cuda_conv2d.cpp:327-400).
int ref_conv2d_i8(const void* x, int x_unsigned, const int8_t* w, const void* bias, void* out, int out_kind,
                  const int64_t* geom, float scale_x, int32_t zp_x, const float* scale_w, const int32_t* zp_w,
                  float scale_w_scalar, int32_t zp_w_scalar, float out_scale, int32_t out_zp, int relu,
                  float min_clip, float max_clip, int threads)
{
    const int64_t n = geom[0], ih = geom[1], iw = geom[2], ic = geom[3], oc = geom[4], kh = geom[5], kw = geom[6];
    const int64_t groups = geom[13], oh = geom[14], ow = geom[15];
    const DataType odt = out_dtype(out_kind);
    const bool int_out = out_kind <= 2;

    QuantParams qa;
    qa.scale = scale_x;
    qa.zero_point = zp_x;
    QuantParams qw = make_qp(scale_w, zp_w, scale_w_scalar, zp_w_scalar, oc, QuantGranularity::PerChannel);
    QuantParams qc;
    qc.scale = out_scale;
    qc.zero_point = out_zp;

    const int64_t a_shape[4] = {n, ih, iw, ic};
    const int64_t w_shape[4] = {kh, kw, ic / groups, oc};
    const int64_t o_shape[4] = {n, oh, ow, oc};
    const int64_t b_shape[1] = {oc};
    TensorView av(a_shape, x_unsigned ? DataType::u8 : DataType::s8, const_cast<void*>(x), TensorLayout::NHWC, qa);
    TensorView wv(w_shape, DataType::s8, const_cast<int8_t*>(w), TensorLayout::HWIO, qw);
    TensorView ov(o_shape, odt, out, TensorLayout::NHWC, qc);
    TensorView bv(b_shape, int_out ? DataType::s32 : odt, const_cast<void*>(bias), TensorLayout::Dense);

    Conv2DAttributes attrs;
    attrs.kernel_size = {kh, kw};
    attrs.stride = {geom[7], geom[8]};
    attrs.dilation = {geom[9], geom[10]};
    attrs.padding = {geom[11], geom[12]};
    attrs.groups = groups;
    attrs.output_dtype = odt;
    attrs.epilogue.type = relu ? EpilogueActivateType::Relu : EpilogueActivateType::None;
    attrs.epilogue.min_clip = min_clip;
    attrs.epilogue.max_clip = max_clip;

    auto op = Conv2D::create(attrs, Backend::CPU);
    const ComputeContext ctx = make_ctx(threads);
    TensorView ins[3] = {av, wv, bv};
    return int(op->compute(ov, std::span<const TensorView>(ins, bias ? 3 : 2), ctx, nullptr));
}

void ref_release_scratch() { release_scratch_memory(); }

} // extern "C"
