// nnops::backend::cuda::quantize_linear_cuda / dequantize_linear_cuda for the B200 backend.
//
// The operator front end resolves these two symbols when it is built with CUDA (declared at
// src/ops/quant_linear.cpp:21-28 of the reference); the reference defines them as
// Status::unsupported stubs (src/backend/cuda/not_implemented.cu:28-37), so in an nnops tree
// this file takes their place in that translation unit's stead.  Behaviour follows the CPU
// route (src/backend/cpu/quant_linear.cpp:80-305): the tensor is a flat row-major array, the
// granularity comes from the scale's element count and `axis`, scale is f32 and the zero
// point s8 or u8 by its own dtype.  All three inputs are device tensors on this backend.
//
// C++23, no CUDA headers: the work is two calls into the C ABI (include/nnb200.h).

#ifdef NNB200_USE_NNOPS_HEADERS
#include "nnops/ops/quant_linear.hpp"
#else
#include "nnops_b200/nnops_api.hpp"
#endif

#include "nnb200.h"

#include <cstring>

namespace nnops::backend::cuda {

namespace {

Status to_status(int code)
{
    return code >= 0 && code <= 5 ? static_cast<Status>(code) : Status::internal;
}

// [outer][rows][inner] view of x for the granularity the operator resolves.
bool decompose(const QuantLinearAttributes& attrs, const TensorView& x, const TensorView& scale,
               nnb200_quant_linear_args& q)
{
    const int64_t rank = x.rank();
    const int64_t numel = x.numel();
    switch (resolve_quant_granularity(scale, attrs.axis)) {
    case QuantGranularity::PerTensor:
        q.outer = 1;
        q.rows = 1;
        q.inner = numel;
        return true;
    case QuantGranularity::PerToken: {
        if (rank < 1) {
            return false;
        }
        const int64_t last = x.shape(rank - 1);
        q.outer = 1;
        q.rows = last > 0 ? numel / last : 0;
        q.inner = last;
        return scale.numel() == q.rows;
    }
    case QuantGranularity::PerChannel: {
        if (attrs.axis >= rank) {
            return false;
        }
        q.outer = 1;
        q.inner = 1;
        for (int64_t d = 0; d < attrs.axis; ++d) {
            q.outer *= x.shape(d);
        }
        for (int64_t d = attrs.axis + 1; d < rank; ++d) {
            q.inner *= x.shape(d);
        }
        q.rows = x.shape(attrs.axis);
        return scale.numel() == q.rows;
    }
    }
    return false;
}

Status run(const QuantLinearAttributes& attrs, TensorView& output, std::span<const TensorView> inputs,
           const ComputeContext& ctx, bool quantize)
{
    if (inputs.size() != 3) {
        return Status::invalid_argument;
    }
    const TensorView& x = inputs[0];
    const TensorView& scale = inputs[1];
    const TensorView& zp = inputs[2];
    if (output.numel() == 0) {
        return Status::ok;
    }
    const DataType flt = quantize ? x.data_type() : output.data_type();
    const DataType qnt = quantize ? output.data_type() : x.data_type();
    if ((flt != DataType::f32 && flt != DataType::f16) || (qnt != DataType::s8 && qnt != DataType::u8) ||
        scale.data_type() != DataType::f32 || (zp.data_type() != DataType::s8 && zp.data_type() != DataType::u8)) {
        return Status::unsupported;
    }
    if (x.numel() != output.numel() || zp.numel() != scale.numel()) {
        return Status::invalid_argument;
    }
    nnb200_quant_linear_args q;
    std::memset(&q, 0, sizeof(q));
    if (!decompose(attrs, x, scale, q)) {
        return Status::invalid_argument;
    }
    q.x = x.ptr<void>();
    q.y = output.ptr<void>();
    q.scale = scale.ptr<float>();
    q.zero_point = zp.ptr<void>();
    q.zp_unsigned = zp.data_type() == DataType::u8;
    q.float_f16 = flt == DataType::f16;
    q.int_unsigned = qnt == DataType::u8;
    return to_status(quantize ? nnb200_quantize_linear(&q, ctx.cuda_stream)
                              : nnb200_dequantize_linear(&q, ctx.cuda_stream));
}

}  // namespace

Status quantize_linear_cuda(const QuantLinearAttributes& attrs, TensorView& output, std::span<const TensorView> inputs,
                            const ComputeContext& ctx, void*)
{
    return run(attrs, output, inputs, ctx, true);
}

Status dequantize_linear_cuda(const QuantLinearAttributes& attrs, TensorView& output,
                              std::span<const TensorView> inputs, const ComputeContext& ctx, void*)
{
    return run(attrs, output, inputs, ctx, false);
}

}  // namespace nnops::backend::cuda
