// Entry points nnops' Conv2D front end references when it is built with CUDA but which this
// backend does not serve: they answer Status::unsupported, the pattern of the reference's own
// stub unit (src/backend/cuda/not_implemented.cu:21-37).  Only built into the drop-in library
// (against the nnops headers); the stand-alone front end never refers to them.

#include "nnops/core/compute_context.hpp"
#include "nnops/core/tensor_view.hpp"
#include "nnops/ops/depthwise_conv.hpp"

#include <span>

namespace nnops::backend::cuda {

// Floating-point depthwise convolution (src/ops/conv2d.cpp:263-283 reroutes depthwise-shaped fp
// Conv2D calls here; the quantized route never does).
Status depthwise_conv_cuda(const DepthwiseConvAttributes&, TensorView&, std::span<const TensorView>,
                           const ComputeContext&, void*)
{
    return Status::unsupported;
}

}  // namespace nnops::backend::cuda
