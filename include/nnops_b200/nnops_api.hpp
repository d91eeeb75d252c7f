// Stand-alone mirror of the slice of the nnops operator API that the quantized-matmul path
// uses: the boundary types (DataType, Status, QuantParams, Epilogue, TensorDesc, TensorView,
// ComputeContext), the two matmul operators (Linear, MatMul) and the two elementwise operators
// either side of them in a W8A8 graph (QuantizeLinear, DequantizeLinear).  Names, argument meaning and error
// behaviour follow the reference so that code written against nnops compiles against this
// header unchanged:
//
//   reference                                   here
//   include/nnops/core/data_type.hpp:23         DataType (same numbering, q4_1 = 11)
//   include/nnops/core/status.hpp:19            Status
//   include/nnops/core/quant_params.hpp:36      QuantParams
//   include/nnops/core/epilogue.hpp:23-91       EpilogueActivateType, Epilogue
//   include/nnops/core/tensor_view.hpp:38,124   TensorDesc, TensorView (pitched, non-owning)
//   include/nnops/core/compute_context.hpp:24   ComputeContext (cuda_stream)
//   include/nnops/core/op_base.hpp:30           OpBase
//   include/nnops/ops/linear.hpp:41-142         LinearAttributes, Linear
//   include/nnops/ops/matmul.hpp:37-135         MatMulAttributes, MatMul
//   include/nnops/ops/quant_linear.hpp:24-141   QuantLinearAttributes, QuantizeLinear, DequantizeLinear
//
// It is NOT a copy of those headers: only what this path needs exists, written from the
// documented behaviour.  When the real nnops headers are available the CUDA backend glue
// (nnops_b200/host/cuda_backend.cpp) is compiled against them instead and this file is unused.
#pragma once

#include <array>
#include <cstddef>
#include <cstdint>
#include <limits>
#include <memory>
#include <span>
#include <vector>

namespace nnops {

enum class Backend : uint8_t { CPU = 0, CUDA = 1, Vulkan = 2, Metal = 3 };

enum class Status : uint8_t { ok = 0, invalid_argument, unsupported, not_initialized, out_of_memory, internal };
constexpr bool is_ok(Status s) noexcept { return s == Status::ok; }
const char* to_string(Status s) noexcept;

enum class DataType : uint8_t { f32 = 0, f16, bf16, s8, u8, s32, s64, f8_e4m3, f8_e5m2, s4, u4, q4_1 };

inline constexpr int64_t q4_1_block_elems = 32;
inline constexpr size_t q4_1_block_bytes = 20;

/// Bytes of one element; 0 for sub-byte and block-packed types.
constexpr size_t data_type_size(DataType dt) noexcept
{
    switch (dt) {
    case DataType::f32: case DataType::s32: return 4;
    case DataType::f16: case DataType::bf16: return 2;
    case DataType::s8: case DataType::u8: case DataType::f8_e4m3: case DataType::f8_e5m2: return 1;
    case DataType::s64: return 8;
    default: return 0;
    }
}
/// The unit row strides are counted in: the element, or the 20-byte block for q4_1.
constexpr size_t data_type_stride_unit(DataType dt) noexcept
{
    return dt == DataType::q4_1 ? q4_1_block_bytes : data_type_size(dt);
}
/// Bytes of a row of `cols` logical elements.
constexpr size_t data_type_row_bytes(DataType dt, int64_t cols) noexcept
{
    if (cols <= 0) return 0;
    if (dt == DataType::q4_1) return static_cast<size_t>((cols + q4_1_block_elems - 1) / q4_1_block_elems) * q4_1_block_bytes;
    if (dt == DataType::s4 || dt == DataType::u4) return static_cast<size_t>((cols + 1) / 2);
    return static_cast<size_t>(cols) * data_type_size(dt);
}

enum class QuantGranularity : uint8_t { PerTensor = 0, PerToken = 1, PerChannel = 2 };

/// Quantization of a view.  scale_data / zero_point_data may be HOST arrays (the reference
/// contract) or device arrays (used in place, no staging).
struct QuantParams {
    QuantGranularity granularity = QuantGranularity::PerTensor;
    float scale = 1.0f;
    int32_t zero_point = 0;
    const float* scale_data = nullptr;
    const int32_t* zero_point_data = nullptr;
    int64_t num_scales = 0;
    bool is_active() const noexcept
    {
        return scale_data != nullptr || zero_point_data != nullptr || scale != 1.0f || zero_point != 0;
    }
};

enum class EpilogueActivateType : uint8_t {
    None = 0, Relu, Gelu, Sigmoid, Tanh, LeakyRelu, Silu, HardSwish, Elu, Relu6
};
enum class EpilogueQuantType : uint8_t { None = 0, Requantize = 1, Dequantize = 2 };

struct Epilogue {
    EpilogueActivateType type = EpilogueActivateType::None;
    float alpha = 0.0f;
    float beta = 1.0f;
    float min_clip = -std::numeric_limits<float>::infinity();
    float max_clip = std::numeric_limits<float>::infinity();
    EpilogueQuantType quant = EpilogueQuantType::None;
    const float* quant_scales = nullptr;
    const int32_t* quant_zero_points = nullptr;
    int64_t quant_param_count = 0;
    int64_t quant_axis = 0;
};

/// The layouts this path uses.  nnops numbers its tags append-only (include/nnops/core/tensor_layout.hpp).
/// Tag values follow include/nnops/core/tensor_layout.hpp of nnops where a tag exists there (NHWC 2,
/// HWIO 5, Dense 12, PackedHWIOCuda 14); the two packed matmul forms of this backend take the next
/// free values after the highest one nnops uses (17).
enum class TensorLayout : uint8_t {
    NHWC = 2,
    HWIO = 5,
    Dense = 12,
    PackedHWIOCuda = 14,
    PackedI8B200 = 18,
    PackedQ4_1B200 = 19,
};

/// Fixed-capacity dimension list (the reference uses an inline small vector of 8).
struct Dims {
    std::array<int64_t, 8> v{};
    int64_t& operator[](size_t i) noexcept { return v[i]; }
    const int64_t& operator[](size_t i) const noexcept { return v[i]; }
    int64_t* data() noexcept { return v.data(); }
    const int64_t* data() const noexcept { return v.data(); }
    void resize(size_t) noexcept {}
};

struct TensorDesc {
    static constexpr int64_t kMaxRank = 8;
    Dims dims;
    int64_t rank = 0;
    DataType dtype = DataType::f32;
    TensorLayout layout = TensorLayout::Dense;
    int64_t row_stride_elems = 0;

    int64_t numel() const noexcept
    {
        int64_t n = 1;
        for (int64_t i = 0; i < rank; ++i) n *= dims[static_cast<size_t>(i)];
        return n;
    }
    /// Suggested row pitch in bytes, rounded up to `alignment`.
    int64_t row_pitch(int64_t alignment = 32) const noexcept
    {
        if (rank < 2) return static_cast<int64_t>(data_type_stride_unit(dtype));
        const int64_t bytes = static_cast<int64_t>(data_type_row_bytes(dtype, dims[static_cast<size_t>(rank - 1)]));
        return (bytes + alignment - 1) / alignment * alignment;
    }
    size_t storage_bytes(int64_t alignment = 32) const noexcept
    {
        if (rank < 2) return data_type_row_bytes(dtype, numel());
        int64_t rows = 1;
        for (int64_t i = 0; i + 1 < rank; ++i) rows *= dims[static_cast<size_t>(i)];
        return static_cast<size_t>(rows * row_pitch(alignment));
    }
};

/// Non-owning, pitched view of a tensor: rows of the last dimension, `pitch` bytes apart; all
/// leading dimensions are dense multiples of the row pitch.
class TensorView {
public:
    static constexpr int64_t kMaxRank = 8;
    TensorView() = default;
    TensorView(std::span<const int64_t> shape, DataType dtype, void* data,
               TensorLayout layout = TensorLayout::Dense, QuantParams qp = {})
        : data_(data), dtype_(dtype), layout_(layout), qp_(qp)
    {
        set_shape(shape);
        pitch_ = rank_ >= 2 ? static_cast<int64_t>(data_type_row_bytes(dtype, shape_[static_cast<size_t>(rank_ - 1)]))
                            : (rank_ == 1 ? static_cast<int64_t>(data_type_stride_unit(dtype)) : 0);
    }
    TensorView(std::span<const int64_t> shape, DataType dtype, void* data, int64_t pitch,
               TensorLayout layout = TensorLayout::Dense, QuantParams qp = {})
        : data_(data), pitch_(pitch), dtype_(dtype), layout_(layout), qp_(qp)
    {
        set_shape(shape);
    }

    int64_t rank() const noexcept { return rank_; }
    int64_t shape(int64_t d) const noexcept { return shape_[static_cast<size_t>(d)]; }
    const int64_t* shape() const noexcept { return shape_.data(); }
    int64_t pitch() const noexcept { return pitch_; }
    DataType data_type() const noexcept { return dtype_; }
    TensorLayout layout() const noexcept { return layout_; }
    const QuantParams& quant_params() const noexcept { return qp_; }
    bool is_empty() const noexcept { return data_ == nullptr; }
    template <class T> T* ptr() noexcept { return static_cast<T*>(data_); }
    template <class T> const T* ptr() const noexcept { return static_cast<const T*>(data_); }

    int64_t numel() const noexcept
    {
        if (rank_ == 0) return data_ != nullptr ? 1 : 0;
        int64_t n = 1;
        for (int64_t i = 0; i < rank_; ++i) n *= shape_[static_cast<size_t>(i)];
        return n;
    }
    /// Row stride in storage units (elements, or 20-byte blocks for q4_1).
    int64_t row_stride_elems() const noexcept
    {
        if (rank_ < 2) return 1;
        const int64_t unit = static_cast<int64_t>(data_type_stride_unit(dtype_));
        return unit > 0 ? pitch_ / unit : 0;
    }
    int64_t stride_elems(int64_t dim) const noexcept
    {
        if (dim == rank_ - 1) return 1;
        int64_t s = row_stride_elems();
        for (int64_t i = rank_ - 2; i > dim; --i) s *= shape_[static_cast<size_t>(i)];
        return s;
    }
    TensorDesc desc() const noexcept
    {
        TensorDesc d;
        d.rank = rank_;
        for (int64_t i = 0; i < rank_; ++i) d.dims[static_cast<size_t>(i)] = shape_[static_cast<size_t>(i)];
        d.dtype = dtype_;
        d.layout = layout_;
        d.row_stride_elems = rank_ >= 2 ? row_stride_elems() : 0;
        return d;
    }

private:
    void set_shape(std::span<const int64_t> shape) noexcept
    {
        rank_ = static_cast<int64_t>(shape.size() <= 8 ? shape.size() : 8);
        for (int64_t i = 0; i < rank_; ++i) shape_[static_cast<size_t>(i)] = shape[static_cast<size_t>(i)];
    }
    std::array<int64_t, 8> shape_{};
    void* data_ = nullptr;
    int64_t pitch_ = 0;
    DataType dtype_ = DataType::f32;
    TensorLayout layout_ = TensorLayout::Dense;
    QuantParams qp_;
    int64_t rank_ = 0;
};

/// Per-call execution context.  Only the CUDA stream matters on this path.
struct ComputeContext {
    Backend expected_backend = Backend::CPU;
    void* cuda_stream = nullptr;  ///< cudaStream_t, opaque; nullptr = default stream
};

enum class OpType : uint8_t { Linear = 0, MatMul = 1, QuantizeLinear = 2, DequantizeLinear = 3, Conv2D = 4 };

class OpBase {
public:
    virtual ~OpBase() = default;
    virtual std::vector<TensorDesc> getOutputTensorDesc(std::span<const TensorDesc> inputs) const = 0;
    virtual size_t getWorkspaceSize(std::span<const TensorDesc>, std::span<const TensorDesc>) const { return 0; }
    virtual Status validate(std::span<const TensorDesc>, std::span<const TensorDesc>) const { return Status::ok; }
    virtual Status compute(std::span<TensorView> outputs, std::span<const TensorView> inputs,
                           const ComputeContext& ctx = {}, void* workspace = nullptr) = 0;
    Status compute(TensorView& output, std::span<const TensorView> inputs, const ComputeContext& ctx = {},
                   void* workspace = nullptr)
    {
        TensorView outs[] = {output};
        return compute(std::span<TensorView>(outs), inputs, ctx, workspace);
    }
    /// Two-step contract: an empty outputs[0] asks for the packed form's geometry; this
    /// backend reads raw weights in place and leaves it empty ("no packed form").
    virtual void prepackWeights(std::span<const TensorView>, std::span<TensorView>, const ComputeContext& = {}) {}
    virtual OpType getOpType() const = 0;
    virtual Backend getBackend() const = 0;
};

struct LinearAttributes {
    Epilogue epilogue{};
    bool add_to = false;
    bool residual_pre_activation = false;
    DataType output_dtype = DataType::f32;
    bool gated = false;
    EpilogueActivateType gate_activation = EpilogueActivateType::Silu;
    float gate_alpha = 1.0f;
    float gate_beta = 0.0f;
    float gate_limit = std::numeric_limits<float>::infinity();
};

/// y[.., N] = epilogue(x[.., K] * W[N, K]^T + bias).  Quantized route: x s8/u8, W s8, output
/// dtype = attributes.output_dtype; weight-decode route: x f16/f32, W q4_1.
class Linear : public OpBase {
public:
    static std::unique_ptr<Linear> create(const LinearAttributes& attrs, Backend backend = Backend::CPU);
    std::vector<TensorDesc> getOutputTensorDesc(std::span<const TensorDesc> inputs) const override;
    Status validate(std::span<const TensorDesc> inputs, std::span<const TensorDesc> outputs) const override;
    using OpBase::compute;
    Status compute(std::span<TensorView> outputs, std::span<const TensorView> inputs, const ComputeContext& ctx = {},
                   void* workspace = nullptr) override;
    /// int8 weights on CUDA: the query answers a [N, K] s8 view tagged TensorLayout::PackedI8B200
    /// whose pitch makes N * pitch the blob size; the second call fills it.  compute() accepts
    /// the packed view in place of W.  q4_1 weights: a [N, K] q4_1 view tagged
    /// TensorLayout::PackedQ4_1B200 (separate nibble and (d, m) planes), same two steps.  Other
    /// weights answer "no packed form".
    void prepackWeights(std::span<const TensorView> inputs, std::span<TensorView> outputs,
                        const ComputeContext& ctx = {}) override;
    OpType getOpType() const override { return OpType::Linear; }
    Backend getBackend() const override { return backend_; }
    const LinearAttributes& attributes() const noexcept { return attrs_; }

private:
    Linear(const LinearAttributes& a, Backend b) : attrs_(a), backend_(b) {}
    LinearAttributes attrs_;
    Backend backend_;
};

struct MatMulAttributes {
    bool transpose_a = false;
    bool transpose_b = false;
    float alpha = 1.0f;
    float beta = 0.0f;
    bool residual_pre_activation = false;
    DataType output_dtype = DataType::s32;
    DataType act_quant_dtype = DataType::s8;
    Epilogue epilogue{};
};

inline constexpr bool is_int8_matmul(DataType a, DataType b) noexcept
{
    return (a == DataType::s8 || a == DataType::u8) && b == DataType::s8;
}

/// C[.., M, N] = epilogue(op(A) * op(B) + bias) with numpy batch broadcasting.
class MatMul : public OpBase {
public:
    static std::unique_ptr<MatMul> create(const MatMulAttributes& attrs = {}, Backend backend = Backend::CPU);
    std::vector<TensorDesc> getOutputTensorDesc(std::span<const TensorDesc> inputs) const override;
    Status validate(std::span<const TensorDesc> inputs, std::span<const TensorDesc> outputs) const override;
    using OpBase::compute;
    Status compute(std::span<TensorView> outputs, std::span<const TensorView> inputs, const ComputeContext& ctx = {},
                   void* workspace = nullptr) override;
    /// As Linear::prepackWeights, for a 2-D B operand in either pose; the packed view stands for
    /// the [N, K] form, so compute() reads it as if transpose_b were set.
    void prepackWeights(std::span<const TensorView> inputs, std::span<TensorView> outputs,
                        const ComputeContext& ctx = {}) override;
    OpType getOpType() const override { return OpType::MatMul; }
    Backend getBackend() const override { return backend_; }
    const MatMulAttributes& attributes() const noexcept { return attrs_; }

private:
    MatMul(const MatMulAttributes& a, Backend b) : attrs_(a), backend_(b) {}
    MatMulAttributes attrs_;
    Backend backend_;
};

struct QuantLinearAttributes {
    /// -1: one parameter per innermost row (per token); >= 0: one per index along `axis` (per
    /// channel).  A one-element scale is per tensor whatever the axis.
    int64_t axis = -1;
    /// QuantizeLinear: s8 / u8.  DequantizeLinear: f32 / f16 (anything else means f32).
    DataType output_dtype = DataType::s8;
};

inline QuantGranularity resolve_quant_granularity(const TensorView& scale, int64_t axis)
{
    if (scale.numel() <= 1) return QuantGranularity::PerTensor;
    return axis < 0 ? QuantGranularity::PerToken : QuantGranularity::PerChannel;
}

/// inputs {x (f32/f16), y_scale (f32), y_zero_point (s8/u8)} -> y (s8/u8):
/// y = saturate(round_half_even(x / scale) + zero_point).
class QuantizeLinear : public OpBase {
public:
    static std::unique_ptr<QuantizeLinear> create(const QuantLinearAttributes& attrs = {}, Backend backend = Backend::CPU);
    static std::unique_ptr<QuantizeLinear> create(Backend backend) { return create(QuantLinearAttributes{}, backend); }
    std::vector<TensorDesc> getOutputTensorDesc(std::span<const TensorDesc> inputs) const override;
    Status validate(std::span<const TensorDesc> inputs, std::span<const TensorDesc> outputs) const override;
    using OpBase::compute;
    Status compute(std::span<TensorView> outputs, std::span<const TensorView> inputs, const ComputeContext& ctx = {},
                   void* workspace = nullptr) override;
    OpType getOpType() const override { return OpType::QuantizeLinear; }
    Backend getBackend() const override { return backend_; }
    const QuantLinearAttributes& attributes() const noexcept { return attrs_; }

private:
    QuantizeLinear(const QuantLinearAttributes& a, Backend b) : attrs_(a), backend_(b) {}
    QuantLinearAttributes attrs_;
    Backend backend_;
};

/// inputs {x (s8/u8), x_scale (f32), x_zero_point (s8/u8)} -> y (f32/f16): y = (x - zero_point) * scale.
class DequantizeLinear : public OpBase {
public:
    static std::unique_ptr<DequantizeLinear> create(const QuantLinearAttributes& attrs = {}, Backend backend = Backend::CPU);
    static std::unique_ptr<DequantizeLinear> create(Backend backend) { return create(QuantLinearAttributes{}, backend); }
    std::vector<TensorDesc> getOutputTensorDesc(std::span<const TensorDesc> inputs) const override;
    Status validate(std::span<const TensorDesc> inputs, std::span<const TensorDesc> outputs) const override;
    using OpBase::compute;
    Status compute(std::span<TensorView> outputs, std::span<const TensorView> inputs, const ComputeContext& ctx = {},
                   void* workspace = nullptr) override;
    OpType getOpType() const override { return OpType::DequantizeLinear; }
    Backend getBackend() const override { return backend_; }
    const QuantLinearAttributes& attributes() const noexcept { return attrs_; }

private:
    DequantizeLinear(const QuantLinearAttributes& a, Backend b) : attrs_(a), backend_(b)
    {
        if (attrs_.output_dtype != DataType::f32 && attrs_.output_dtype != DataType::f16) {
            attrs_.output_dtype = DataType::f32;
        }
    }
    QuantLinearAttributes attrs_;
    Backend backend_;
};

enum class ConvAlgorithm : uint8_t { ImplicitGemm = 0, Winograd, Auto };

inline constexpr bool is_quantized_conv2d(DataType weight_dtype) noexcept { return weight_dtype == DataType::s8; }

/// Field for field the attributes of nnops' Conv2D (include/nnops/ops/conv2d.hpp:51-130); this backend
/// serves the quantized route only (s8 HWIO filter, pre-quantized u8/s8 NHWC activation).
struct Conv2DAttributes {
    std::array<int64_t, 2> kernel_size = {1, 1};
    std::array<int64_t, 2> stride = {1, 1};
    std::array<int64_t, 2> dilation = {1, 1};
    std::array<int64_t, 2> padding = {0, 0};
    int64_t groups = 1;
    enum class AutoPad : uint8_t { NOTSET = 0, SAME_UPPER, SAME_LOWER, VALID };
    AutoPad auto_pad = AutoPad::NOTSET;
    Epilogue epilogue{};
    bool add_to = false;
    bool residual_pre_activation = false;
    DataType output_dtype = DataType::f32;
    DataType act_quant_dtype = DataType::s8;
    ConvAlgorithm algorithm = ConvAlgorithm::Auto;
    int64_t winograd_order = 0;
};

/// y[N, OH, OW, OC] = epilogue(conv(x[N, IH, IW, IC], w[KH, KW, IC/G, OC]) + bias), channel-last.
class Conv2D : public OpBase {
public:
    static std::unique_ptr<Conv2D> create(const Conv2DAttributes& attrs, Backend backend = Backend::CPU);
    std::vector<TensorDesc> getOutputTensorDesc(std::span<const TensorDesc> inputs) const override;
    Status validate(std::span<const TensorDesc> inputs, std::span<const TensorDesc> outputs) const override;
    using OpBase::compute;
    Status compute(std::span<TensorView> outputs, std::span<const TensorView> inputs, const ComputeContext& ctx = {},
                   void* workspace = nullptr) override;
    /// s8 HWIO filter on CUDA: the query answers an [OC, bytes / OC] s8 view tagged
    /// TensorLayout::PackedHWIOCuda; the second call fills it; compute() accepts it in place of the filter.
    void prepackWeights(std::span<const TensorView> inputs, std::span<TensorView> outputs,
                        const ComputeContext& ctx = {}) override;
    OpType getOpType() const override { return OpType::Conv2D; }
    Backend getBackend() const override { return backend_; }
    const Conv2DAttributes& attributes() const noexcept { return attrs_; }

private:
    Conv2D(const Conv2DAttributes& a, Backend b) : attrs_(a), backend_(b) {}
    Conv2DAttributes attrs_;
    Backend backend_;
};

namespace backend::cuda {
/// The two backend entry points the operator front end dispatches to (the reference declares
/// them at src/ops/linear.cpp:24 and src/ops/matmul.cpp:35).
Status linear_cuda(const LinearAttributes& attrs, TensorView& output, std::span<const TensorView> inputs,
                   const ComputeContext& ctx, void* workspace);
Status matmul_cuda(const MatMulAttributes& attrs, TensorView& output, std::span<const TensorView> inputs,
                   const ComputeContext& ctx, void* workspace);
/// Two-step prepack of a 2-D int8 weight (w_is_nk: stored [N, K], else [K, N]); see Linear::prepackWeights.
void prepack_i8_cuda(const TensorView& weight, bool w_is_nk, TensorView& packed, const ComputeContext& ctx);
/// Two-step prepack of a 2-D q4_1 weight stored [N, K] into separated nibble and (d, m) planes.
void prepack_q4_1_cuda(const TensorView& weight, TensorView& packed, const ComputeContext& ctx);
/// ... and the two of QuantizeLinear / DequantizeLinear (declared at src/ops/quant_linear.cpp:21-28).
Status quantize_linear_cuda(const QuantLinearAttributes& attrs, TensorView& output, std::span<const TensorView> inputs,
                            const ComputeContext& ctx, void* workspace);
Status dequantize_linear_cuda(const QuantLinearAttributes& attrs, TensorView& output,
                              std::span<const TensorView> inputs, const ComputeContext& ctx, void* workspace);
/// Conv2D's entry (dispatched at src/ops/conv2d.cpp:86-90 of the reference) and the packed-filter pair its
/// prepackWeights drives (src/backend/cuda/conv/conv2d_pack.h:30-37).
Status conv2d_cuda(const Conv2DAttributes& attrs, TensorView& output, std::span<const TensorView> inputs,
                   const ComputeContext& ctx, void* workspace);
TensorDesc conv_i8_packed_weight_desc(const Conv2DAttributes& attrs, const TensorDesc& weight);
Status conv_i8_packed_weight_pack(const Conv2DAttributes& attrs, const TensorView& weight, TensorView& out,
                                  const ComputeContext& ctx);
}  // namespace backend::cuda

}  // namespace nnops
