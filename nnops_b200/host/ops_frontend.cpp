// Stand-alone front end of Linear, MatMul, QuantizeLinear, DequantizeLinear and Conv2D (quantized route) for builds
// without the nnops source tree: create / getOutputTensorDesc / validate / compute with the
// reference's argument checks and status codes (src/ops/linear.cpp:26-120,
// src/ops/matmul.cpp:36-152, src/ops/quant_linear.cpp:54-175,
// include/nnops/detail/validate.hpp:70-126, include/nnops/detail/shape_inference.hpp:453-526,713-742),
// dispatching to the CUDA backend.  There is no CPU route here: an operator created for
// another backend answers Status::unsupported.

#include "nnops_b200/nnops_api.hpp"

#include <algorithm>

namespace nnops {

const char* to_string(Status s) noexcept
{
    switch (s) {
    case Status::ok: return "ok";
    case Status::invalid_argument: return "invalid_argument";
    case Status::unsupported: return "unsupported";
    case Status::not_initialized: return "not_initialized";
    case Status::out_of_memory: return "out_of_memory";
    case Status::internal: return "internal";
    }
    return "unknown";
}

namespace {

Status check_counts(size_t n_in, size_t n_out, size_t min_in, size_t max_in, size_t want_out)
{
    return (n_in >= min_in && n_in <= max_in && n_out == want_out) ? Status::ok : Status::invalid_argument;
}

// Counts, then "every view has storage": a call with a null view is rejected before any work.
Status check_views(std::span<TensorView> outputs, std::span<const TensorView> inputs, size_t min_in, size_t max_in)
{
    if (check_counts(inputs.size(), outputs.size(), min_in, max_in, 1) != Status::ok) {
        return Status::invalid_argument;
    }
    for (const auto& v : inputs) {
        if (v.is_empty() && v.numel() != 0) {
            return Status::invalid_argument;
        }
    }
    for (const auto& v : outputs) {
        if (v.is_empty() && v.numel() != 0) {
            return Status::invalid_argument;
        }
    }
    return Status::ok;
}

template <class Op>
Status validate_views(const Op& op, std::span<TensorView> outputs, std::span<const TensorView> inputs)
{
    std::vector<TensorDesc> in_d, out_d;
    for (const auto& v : inputs) in_d.push_back(v.desc());
    for (const auto& v : outputs) out_d.push_back(v.desc());
    return op.validate(in_d, out_d);
}

}  // namespace

// ---- Linear -----------------------------------------------------------------------------

std::unique_ptr<Linear> Linear::create(const LinearAttributes& attrs, Backend backend)
{
    return std::unique_ptr<Linear>(new Linear(attrs, backend));  // never fails
}

std::vector<TensorDesc> Linear::getOutputTensorDesc(std::span<const TensorDesc> inputs) const
{
    const TensorDesc& x = inputs[0];
    const TensorDesc& w = inputs[1];
    TensorDesc out = x;  // [.., K] -> [.., N], activation dtype
    out.row_stride_elems = 0;
    if (out.rank >= 1 && w.rank == 2) {
        out.dims[static_cast<size_t>(out.rank - 1)] = attrs_.gated ? w.dims[0] / 2 : w.dims[0];
    }
    if (is_int8_matmul(x.dtype, w.dtype)) {
        const DataType odt = attrs_.output_dtype;
        const bool known = odt == DataType::f16 || odt == DataType::f32 || odt == DataType::s32 ||
                           odt == DataType::s8 || odt == DataType::u8;
        out.dtype = known ? odt : DataType::f32;
    }
    return {out};
}

Status Linear::validate(std::span<const TensorDesc> inputs, std::span<const TensorDesc> outputs) const
{
    if (check_counts(inputs.size(), outputs.size(), 2, 3, 1) != Status::ok) {
        return Status::invalid_argument;
    }
    if (backend_ == Backend::CUDA && inputs[0].rank > 6) {
        return Status::unsupported;
    }
    if (attrs_.add_to && attrs_.residual_pre_activation && (attrs_.gated || backend_ != Backend::CPU)) {
        return Status::unsupported;
    }
    return Status::ok;
}

Status Linear::compute(std::span<TensorView> outputs, std::span<const TensorView> inputs, const ComputeContext& ctx,
                       void* workspace)
{
    if (const Status s = check_views(outputs, inputs, 2, 3); s != Status::ok) {
        return s;
    }
    if (const Status s = validate_views(*this, outputs, inputs); s != Status::ok) {
        return s;
    }
    if (backend_ != Backend::CUDA) {
        return Status::unsupported;
    }
    return backend::cuda::linear_cuda(attrs_, outputs[0], inputs, ctx, workspace);
}

void Linear::prepackWeights(std::span<const TensorView> inputs, std::span<TensorView> outputs,
                            const ComputeContext& ctx)
{
    if (backend_ != Backend::CUDA || inputs.empty() || outputs.empty()) {
        return;
    }
    if (inputs[0].data_type() == DataType::q4_1) {
        backend::cuda::prepack_q4_1_cuda(inputs[0], outputs[0], ctx);
        return;
    }
    backend::cuda::prepack_i8_cuda(inputs[0], true, outputs[0], ctx);
}

// ---- MatMul -----------------------------------------------------------------------------

std::unique_ptr<MatMul> MatMul::create(const MatMulAttributes& attrs, Backend backend)
{
    return std::unique_ptr<MatMul>(new MatMul(attrs, backend));
}

std::vector<TensorDesc> MatMul::getOutputTensorDesc(std::span<const TensorDesc> inputs) const
{
    const TensorDesc& a = inputs[0];
    const TensorDesc& b = inputs[1];
    const int64_t ra = a.rank, rb = b.rank;
    const bool b_is_nk = attrs_.transpose_b || b.layout == TensorLayout::PackedI8B200;  // a packed B stands for [N, K]
    const int64_t M = attrs_.transpose_a ? a.dims[static_cast<size_t>(ra - 1)] : a.dims[static_cast<size_t>(ra - 2)];
    const int64_t N = b_is_nk ? b.dims[static_cast<size_t>(rb - 2)] : b.dims[static_cast<size_t>(rb - 1)];
    // numpy broadcast of the leading axes, right-aligned.
    const int64_t la = ra - 2, lb = rb - 2, lr = std::max(la, lb);
    TensorDesc out;
    out.layout = a.layout;
    out.dtype = is_int8_matmul(a.dtype, b.dtype) ? attrs_.output_dtype : a.dtype;
    out.rank = lr + 2;
    for (int64_t d = 0; d < lr; ++d) {
        const int64_t ai = la - 1 - d, bi = lb - 1 - d;
        const int64_t ad = ai >= 0 ? a.dims[static_cast<size_t>(ai)] : 1;
        const int64_t bd = bi >= 0 ? b.dims[static_cast<size_t>(bi)] : 1;
        out.dims[static_cast<size_t>(lr - 1 - d)] = std::max(ad, bd);
    }
    out.dims[static_cast<size_t>(lr)] = M;
    out.dims[static_cast<size_t>(lr + 1)] = N;
    return {out};
}

Status MatMul::validate(std::span<const TensorDesc> inputs, std::span<const TensorDesc> outputs) const
{
    if (check_counts(inputs.size(), outputs.size(), 2, 3, 1) != Status::ok) {
        return Status::invalid_argument;
    }
    if (attrs_.residual_pre_activation && backend_ != Backend::CPU) {
        return Status::unsupported;
    }
    const TensorDesc& a = inputs[0];
    const TensorDesc& b = inputs[1];
    if (a.rank < 2 || b.rank < 2) {
        return Status::invalid_argument;
    }
    if (backend_ == Backend::CUDA && (a.rank > 6 || b.rank > 6)) {
        return Status::unsupported;
    }
    const int64_t k_a = attrs_.transpose_a ? a.dims[static_cast<size_t>(a.rank - 2)] : a.dims[static_cast<size_t>(a.rank - 1)];
    const bool b_is_nk = attrs_.transpose_b || b.layout == TensorLayout::PackedI8B200;
    const int64_t k_b = b_is_nk ? b.dims[static_cast<size_t>(b.rank - 1)] : b.dims[static_cast<size_t>(b.rank - 2)];
    return k_a == k_b ? Status::ok : Status::invalid_argument;
}

Status MatMul::compute(std::span<TensorView> outputs, std::span<const TensorView> inputs, const ComputeContext& ctx,
                       void* workspace)
{
    if (const Status s = check_views(outputs, inputs, 2, 3); s != Status::ok) {
        return s;
    }
    if (const Status s = validate_views(*this, outputs, inputs); s != Status::ok) {
        return s;
    }
    if (backend_ != Backend::CUDA) {
        return Status::unsupported;
    }
    return backend::cuda::matmul_cuda(attrs_, outputs[0], inputs, ctx, workspace);
}

void MatMul::prepackWeights(std::span<const TensorView> inputs, std::span<TensorView> outputs,
                            const ComputeContext& ctx)
{
    if (backend_ != Backend::CUDA || inputs.empty() || outputs.empty()) {
        return;
    }
    backend::cuda::prepack_i8_cuda(inputs[0], attrs_.transpose_b, outputs[0], ctx);
}

// ---- QuantizeLinear / DequantizeLinear -----------------------------------------------------

namespace {

TensorDesc same_shape_as(const TensorDesc& x, DataType dt)
{
    TensorDesc out;
    out.rank = x.rank;
    out.layout = x.layout;
    out.dtype = dt;
    out.dims = x.dims;
    return out;
}

bool rows_compact(const TensorDesc& d)
{
    return d.rank < 2 || d.row_stride_elems == 0 || d.row_stride_elems == d.dims[static_cast<size_t>(d.rank - 1)];
}

// A float side (f32/f16), an s8/u8 side, an f32 scale and an s8/u8 zero point; rows packed.
Status check_quant_linear(std::span<const TensorDesc> inputs, std::span<const TensorDesc> outputs, bool quantize)
{
    if (check_counts(inputs.size(), outputs.size(), 3, 3, 1) != Status::ok) {
        return Status::invalid_argument;
    }
    const DataType flt = quantize ? inputs[0].dtype : outputs[0].dtype;
    const DataType qnt = quantize ? outputs[0].dtype : inputs[0].dtype;
    if (flt != DataType::f32 && flt != DataType::f16) {
        return Status::unsupported;
    }
    if (qnt != DataType::s8 && qnt != DataType::u8) {
        return Status::invalid_argument;
    }
    if (inputs[1].dtype != DataType::f32) {
        return Status::invalid_argument;
    }
    if (inputs[2].dtype != DataType::s8 && inputs[2].dtype != DataType::u8) {
        return Status::invalid_argument;
    }
    if (!rows_compact(inputs[0]) || !rows_compact(outputs[0])) {
        return Status::unsupported;
    }
    return Status::ok;
}

}  // namespace

std::unique_ptr<QuantizeLinear> QuantizeLinear::create(const QuantLinearAttributes& attrs, Backend backend)
{
    return std::unique_ptr<QuantizeLinear>(new QuantizeLinear(attrs, backend));
}

std::vector<TensorDesc> QuantizeLinear::getOutputTensorDesc(std::span<const TensorDesc> inputs) const
{
    return {same_shape_as(inputs[0], attrs_.output_dtype)};
}

Status QuantizeLinear::validate(std::span<const TensorDesc> inputs, std::span<const TensorDesc> outputs) const
{
    return check_quant_linear(inputs, outputs, true);
}

Status QuantizeLinear::compute(std::span<TensorView> outputs, std::span<const TensorView> inputs,
                               const ComputeContext& ctx, void* workspace)
{
    if (const Status s = check_views(outputs, inputs, 3, 3); s != Status::ok) {
        return s;
    }
    if (const Status s = validate_views(*this, outputs, inputs); s != Status::ok) {
        return s;
    }
    if (backend_ != Backend::CUDA) {
        return Status::unsupported;
    }
    return backend::cuda::quantize_linear_cuda(attrs_, outputs[0], inputs, ctx, workspace);
}

std::unique_ptr<DequantizeLinear> DequantizeLinear::create(const QuantLinearAttributes& attrs, Backend backend)
{
    return std::unique_ptr<DequantizeLinear>(new DequantizeLinear(attrs, backend));
}

std::vector<TensorDesc> DequantizeLinear::getOutputTensorDesc(std::span<const TensorDesc> inputs) const
{
    return {same_shape_as(inputs[0], attrs_.output_dtype)};
}

Status DequantizeLinear::validate(std::span<const TensorDesc> inputs, std::span<const TensorDesc> outputs) const
{
    return check_quant_linear(inputs, outputs, false);
}

Status DequantizeLinear::compute(std::span<TensorView> outputs, std::span<const TensorView> inputs,
                                 const ComputeContext& ctx, void* workspace)
{
    if (const Status s = check_views(outputs, inputs, 3, 3); s != Status::ok) {
        return s;
    }
    if (const Status s = validate_views(*this, outputs, inputs); s != Status::ok) {
        return s;
    }
    if (backend_ != Backend::CUDA) {
        return Status::unsupported;
    }
    return backend::cuda::dequantize_linear_cuda(attrs_, outputs[0], inputs, ctx, workspace);
}

// ---- Conv2D (quantized route) -----------------------------------------------------------

namespace {

int64_t ceil_div_i64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// include/nnops/detail/shape_inference.hpp:55-83.
int64_t spatial_out(int64_t in, int64_t kernel, int64_t stride, int64_t dilation, int64_t padding, int auto_pad)
{
    const int64_t eff = dilation * (kernel - 1) + 1;
    switch (auto_pad) {
    case 0: return (in + 2 * padding - eff) / stride + 1;
    case 1: return ceil_div_i64(in, stride);
    case 2: return in > 0 ? (in - 1) / stride + 1 : 1;
    case 3: return (in - eff) / stride + 1;
    default: return 0;
    }
}

// include/nnops/detail/shape_inference.hpp:87-108: only the leading half is a kernel argument.
int64_t leading_padding(int64_t in, int64_t kernel, int64_t stride, int64_t dilation, int64_t padding, int auto_pad)
{
    if (auto_pad == 1 || auto_pad == 2) {
        const int64_t eff = dilation * (kernel - 1) + 1;
        const int64_t total = std::max<int64_t>(0, (ceil_div_i64(in, stride) - 1) * stride + eff - in);
        return auto_pad == 1 ? total / 2 : total - total / 2;
    }
    return auto_pad == 3 ? 0 : padding;
}

}  // namespace

std::unique_ptr<Conv2D> Conv2D::create(const Conv2DAttributes& attrs, Backend backend)
{
    return std::unique_ptr<Conv2D>(new Conv2D(attrs, backend));
}

std::vector<TensorDesc> Conv2D::getOutputTensorDesc(std::span<const TensorDesc> inputs) const
{
    const TensorDesc& in = inputs[0];
    const TensorDesc& wt = inputs[1];
    const int ap = static_cast<int>(attrs_.auto_pad);
    TensorDesc out;
    out.rank = 4;
    out.layout = in.layout;
    out.dtype = in.dtype;
    out.dims[0] = in.dims[0];
    out.dims[1] = spatial_out(in.dims[1], attrs_.kernel_size[0], attrs_.stride[0], attrs_.dilation[0], attrs_.padding[0], ap);
    out.dims[2] = spatial_out(in.dims[2], attrs_.kernel_size[1], attrs_.stride[1], attrs_.dilation[1], attrs_.padding[1], ap);
    // HWIO's last axis is OC; a packed blob's descriptor leads with it.
    out.dims[3] = wt.layout == TensorLayout::PackedHWIOCuda ? wt.dims[0] : wt.dims[3];
    if (is_quantized_conv2d(wt.dtype)) {
        // src/ops/conv2d.cpp:168-178: a pre-quantized activation takes output_dtype.
        const bool fp_act = in.dtype == DataType::f32 || in.dtype == DataType::f16;
        const DataType odt = attrs_.output_dtype;
        const bool int_out = odt == DataType::s8 || odt == DataType::u8;
        out.dtype = (int_out || !fp_act) ? odt : in.dtype;
    }
    return {out};
}

Status Conv2D::validate(std::span<const TensorDesc> inputs, std::span<const TensorDesc> outputs) const
{
    if (check_counts(inputs.size(), outputs.size(), 2, 3, 1) != Status::ok) {
        return Status::invalid_argument;
    }
    if (inputs[0].layout != TensorLayout::NHWC && inputs[0].layout != TensorLayout::Dense) {
        return Status::invalid_argument;
    }
    if (inputs[1].layout != TensorLayout::HWIO && inputs[1].layout != TensorLayout::PackedHWIOCuda) {
        return Status::invalid_argument;
    }
    if (attrs_.add_to && attrs_.residual_pre_activation) {
        return Status::unsupported;
    }
    return Status::ok;
}

Status Conv2D::compute(std::span<TensorView> outputs, std::span<const TensorView> inputs, const ComputeContext& ctx,
                       void* workspace)
{
    if (const Status s = check_views(outputs, inputs, 2, 3); s != Status::ok) {
        return s;
    }
    if (const Status s = validate_views(*this, outputs, inputs); s != Status::ok) {
        return s;
    }
    if (backend_ != Backend::CUDA) {
        return Status::unsupported;
    }
    // auto_pad lives in the descriptor; the kernel sees explicit leading padding (src/ops/conv2d.cpp:246-256).
    Conv2DAttributes attrs = attrs_;
    if (attrs.auto_pad != Conv2DAttributes::AutoPad::NOTSET) {
        const int ap = static_cast<int>(attrs.auto_pad);
        attrs.padding[0] = leading_padding(inputs[0].shape(1), attrs.kernel_size[0], attrs.stride[0], attrs.dilation[0],
                                           attrs.padding[0], ap);
        attrs.padding[1] = leading_padding(inputs[0].shape(2), attrs.kernel_size[1], attrs.stride[1], attrs.dilation[1],
                                           attrs.padding[1], ap);
        attrs.auto_pad = Conv2DAttributes::AutoPad::NOTSET;
    }
    return backend::cuda::conv2d_cuda(attrs, outputs[0], inputs, ctx, workspace);
}

void Conv2D::prepackWeights(std::span<const TensorView> inputs, std::span<TensorView> outputs, const ComputeContext& ctx)
{
    if (backend_ != Backend::CUDA || inputs.empty() || outputs.empty()) {
        return;
    }
    const TensorView& weight = inputs[0];
    const TensorDesc d = backend::cuda::conv_i8_packed_weight_desc(attrs_, weight.desc());
    if (d.rank == 0) {
        return;   // no packed form
    }
    if (outputs[0].is_empty()) {
        const int64_t shape[2] = {d.dims[0], d.dims[1]};
        outputs[0] = TensorView(std::span<const int64_t>(shape, 2), d.dtype, nullptr, d.row_stride_elems, d.layout,
                                weight.quant_params());
        return;
    }
    (void)backend::cuda::conv_i8_packed_weight_pack(attrs_, weight, outputs[0], ctx);
}

}  // namespace nnops
