// nnops::backend::cuda::conv2d_cuda for the B200 backend -- the quantized route only -- and the
// packed-filter pair Conv2D::prepackWeights drives.  C++23, no CUDA headers: the work is calls
// into the C ABI (include/nnb200.h).
//
// These are the symbols nnops' Conv2D front end resolves when it is built with CUDA
// (src/ops/conv2d.cpp:86-90 dispatch, :312-340 prepack).  They replace conv2d_cuda's quantized
// branch (src/backend/cuda/conv/conv2d.cu:822-836 -> conv2d_i8_cuda,
// src/backend/cuda/conv/conv2d_i8.cu:910-1100) and conv_i8_packed_weight_desc / _pack
// (src/backend/cuda/conv/conv2d_i8.cu:1108-1170).  Refusals mirror the reference's: anything but
// a u8/s8 NHWC activation against an s8 HWIO (or PackedHWIOCuda) filter, a Winograd request, a
// residual add, an s32 destination -> Status::unsupported.  Floating-point convolutions are not
// part of this backend and answer unsupported as well.

#ifdef NNB200_USE_NNOPS_HEADERS
#include "nnops/ops/conv2d.hpp"
#else
#include "nnops_b200/nnops_api.hpp"
#endif

#include "nnb200.h"
#include "staging.hpp"

#include <cstring>

namespace nnops::backend::cuda {

using namespace b200_detail;

namespace {

// Shape of the packed blob as a [OC, bytes / OC] s8 view (OC first so that shape inference still
// reads the channel count, as the reference's descriptor does).
int64_t packed_row_bytes(int64_t kh, int64_t kw, int64_t icg, int64_t oc)
{
    const int64_t total = static_cast<int64_t>(nnb200_conv2d_i8_pack_bytes(kh, kw, icg, oc));
    return (total + oc - 1) / oc;
}

}  // namespace

Status conv2d_cuda(const Conv2DAttributes& attrs, TensorView& output, std::span<const TensorView> inputs,
                   const ComputeContext& ctx, void*)
{
    if (inputs.size() < 2) {
        return Status::invalid_argument;
    }
    const TensorView& act = inputs[0];
    const TensorView& wgt = inputs[1];
    const TensorView* bias = inputs.size() > 2 && !inputs[2].is_empty() ? &inputs[2] : nullptr;
    if (!is_quantized_conv2d(wgt.data_type())) {
        return Status::unsupported;   // fp convolutions: not on this backend
    }
    if (output.numel() == 0) {
        return Status::ok;
    }
    const DataType adt = act.data_type();
    if ((adt != DataType::u8 && adt != DataType::s8) || attrs.algorithm == ConvAlgorithm::Winograd || attrs.add_to) {
        return Status::unsupported;
    }
    const bool packed = wgt.layout() == TensorLayout::PackedHWIOCuda;
    if (act.rank() != 4 || output.rank() != 4 || (packed ? wgt.rank() != 2 : wgt.rank() != 4) ||
        (!packed && wgt.layout() != TensorLayout::HWIO)) {
        return Status::unsupported;
    }
    int kind = 0;
    if (!out_kind_of(output.data_type(), kind) || kind == NNB200_OUT_S32) {
        return Status::unsupported;
    }
    if (attrs.groups <= 0 || act.shape(3) % attrs.groups != 0 || output.shape(3) % attrs.groups != 0) {
        return Status::invalid_argument;
    }

    nnb200_conv2d_i8_args c;
    std::memset(&c, 0, sizeof(c));
    c.input = act.ptr<void>();
    c.weight = wgt.ptr<void>();
    c.out = output.ptr<void>();
    c.batch = act.shape(0); c.ih = act.shape(1); c.iw = act.shape(2); c.ic = act.shape(3);
    c.oh = output.shape(1); c.ow = output.shape(2); c.oc = output.shape(3);
    c.kh = attrs.kernel_size[0]; c.kw = attrs.kernel_size[1];
    c.stride_h = attrs.stride[0]; c.stride_w = attrs.stride[1];
    c.dil_h = attrs.dilation[0]; c.dil_w = attrs.dilation[1];
    c.pad_h = attrs.padding[0]; c.pad_w = attrs.padding[1];
    c.groups = attrs.groups;
    c.in_stride_n = act.stride_elems(0); c.in_stride_h = act.stride_elems(1);
    c.in_stride_w = act.stride_elems(2); c.in_stride_c = act.stride_elems(3);
    c.out_stride_n = output.stride_elems(0); c.out_stride_h = output.stride_elems(1);
    c.out_stride_w = output.stride_elems(2);
    if (output.stride_elems(3) != 1) {
        return Status::unsupported;
    }
    c.weight_packed = packed;
    if (packed) {
        if (wgt.shape(0) != c.oc ||
            wgt.numel() < static_cast<int64_t>(nnb200_conv2d_i8_pack_bytes(c.kh, c.kw, c.ic / c.groups, c.oc))) {
            return Status::unsupported;
        }
    } else {
        if (wgt.shape(0) != c.kh || wgt.shape(1) != c.kw || wgt.shape(2) != c.ic / c.groups || wgt.shape(3) != c.oc) {
            return Status::invalid_argument;
        }
        c.w_stride_kh = wgt.stride_elems(0); c.w_stride_kw = wgt.stride_elems(1);
        c.w_stride_ic = wgt.stride_elems(2); c.w_stride_oc = wgt.stride_elems(3);
    }
    c.a_unsigned = adt == DataType::u8;
    c.out_kind = kind;
    const bool int_out = kind <= NNB200_OUT_U8;
    c.relu = int_out && attrs.epilogue.type == EpilogueActivateType::Relu;
    c.activation = static_cast<int32_t>(attrs.epilogue.type);
    c.act_alpha = attrs.epilogue.alpha;
    c.act_beta = attrs.epilogue.beta;
    c.min_clip = attrs.epilogue.min_clip;
    c.max_clip = attrs.epilogue.max_clip;
    c.bias = bias != nullptr ? bias->ptr<void>() : nullptr;

    // The activation is per-tensor; element 0 of an array form is read on the host
    // (conv2d_i8.cu:1010-1013).  The filter's per-channel arrays are host arrays by contract and
    // staged per call; device arrays are used in place.
    const QuantParams& qa = act.quant_params();
    const QuantParams& qw = wgt.quant_params();
    if ((qa.scale_data != nullptr && nnb200_is_device_pointer(qa.scale_data)) ||
        (qa.zero_point_data != nullptr && nnb200_is_device_pointer(qa.zero_point_data))) {
        return Status::unsupported;
    }
    c.scale_x = qa.scale_data != nullptr ? qa.scale_data[0] : qa.scale;
    c.zp_x = qa.zero_point_data != nullptr ? qa.zero_point_data[0] : qa.zero_point;
    c.scale_w_scalar = qw.scale;
    c.zp_w_scalar = qw.zero_point;
    c.out_scale = 1.0f;
    if (int_out) {
        const QuantParams& qc = output.quant_params();
        if ((qc.scale_data != nullptr && nnb200_is_device_pointer(qc.scale_data)) ||
            (qc.zero_point_data != nullptr && nnb200_is_device_pointer(qc.zero_point_data))) {
            return Status::unsupported;
        }
        c.out_scale = qc.scale_data != nullptr ? qc.scale_data[0] : qc.scale;
        c.out_zp = qc.zero_point_data != nullptr ? qc.zero_point_data[0] : qc.zero_point;
    }

    Staging st(ctx.cuda_stream);
    const size_t oc_bytes = static_cast<size_t>(c.oc) * 4;
    st.reserve(qw.scale_data, oc_bytes);
    st.reserve(qw.zero_point_data, oc_bytes);
    // The scratch size depends on whether zero points are present, not on their addresses: ask with
    // stand-in pointers, then fill in the real ones.
    c.scale_w = qw.scale_data;
    c.zp_w = qw.zero_point_data;
    c.zp_w_nonzero = qw.zero_point_data != nullptr;
    const size_t scratch = nnb200_conv2d_i8_workspace_bytes(&c);
    st.reserve_raw(scratch);
    if (const int e = st.allocate(); e != NNB200_OK) {
        return to_status(e);
    }
    DeviceArray sw, zw;
    for (const int e : {st.place(qw.scale_data, oc_bytes, false, sw), st.place(qw.zero_point_data, oc_bytes, true, zw)}) {
        if (e != NNB200_OK) {
            return to_status(e);
        }
    }
    c.scale_w = static_cast<const float*>(sw.ptr);
    c.zp_w = static_cast<const int32_t*>(zw.ptr);
    // Keep the promise conservative: the scratch was sized for "may be non-zero".
    c.zp_w_nonzero = zw.ptr != nullptr;
    if (scratch > 0) {
        c.workspace = st.take_raw(scratch);
        c.workspace_bytes = scratch;
        if (c.workspace == nullptr) {
            return Status::internal;
        }
    }
    return to_status(nnb200_conv2d_i8(&c, ctx.cuda_stream));
}

TensorDesc conv_i8_packed_weight_desc(const Conv2DAttributes& attrs, const TensorDesc& weight)
{
    TensorDesc d;
    if (weight.rank != 4 || weight.dtype != DataType::s8 || weight.layout != TensorLayout::HWIO ||
        attrs.algorithm == ConvAlgorithm::Winograd || attrs.groups <= 0 || weight.dims[3] % attrs.groups != 0) {
        return d;   // rank 0: no packed form
    }
    const int64_t oc = weight.dims[3];
    d.rank = 2;
    d.layout = TensorLayout::PackedHWIOCuda;
    d.dtype = DataType::s8;
    d.dims.resize(2);
    d.dims[0] = oc;
    d.dims[1] = packed_row_bytes(weight.dims[0], weight.dims[1], weight.dims[2], oc);
    d.row_stride_elems = d.dims[1];
    return d;
}

Status conv_i8_packed_weight_pack(const Conv2DAttributes& attrs, const TensorView& weight, TensorView& out,
                                  const ComputeContext& ctx)
{
    if (weight.rank() != 4 || weight.data_type() != DataType::s8 || weight.layout() != TensorLayout::HWIO ||
        attrs.groups <= 0 || weight.shape(3) % attrs.groups != 0) {
        return Status::unsupported;
    }
    const int64_t kh = weight.shape(0), kw = weight.shape(1), icg = weight.shape(2), oc = weight.shape(3);
    if (out.rank() != 2 || out.data_type() != DataType::s8 || out.layout() != TensorLayout::PackedHWIOCuda ||
        out.shape(0) != oc || out.numel() < static_cast<int64_t>(nnb200_conv2d_i8_pack_bytes(kh, kw, icg, oc))) {
        return Status::unsupported;
    }
    return to_status(nnb200_conv2d_i8_pack(weight.ptr<void>(), weight.stride_elems(0), weight.stride_elems(1),
                                           weight.stride_elems(2), weight.stride_elems(3), kh, kw, icg, oc,
                                           attrs.groups, out.ptr<void>(), ctx.cuda_stream));
}

}  // namespace nnops::backend::cuda
