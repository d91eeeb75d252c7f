// nnops::backend::cuda::linear_cuda / matmul_cuda for the B200 backend: the host side of the
// drop-in boundary.  C++23, no CUDA headers -- everything device-side goes through the C ABI
// in include/nnb200.h, with the stream taken from ComputeContext.
//
// These are the two symbols nnops' operator front end resolves when it is built with CUDA
// (declared at src/ops/linear.cpp:24 and src/ops/matmul.cpp:35 of the reference, dispatched by
// src/ops/dispatch.hpp:42-96).  They replace src/backend/cuda/matmul/linear.cu:94-163 and
// src/backend/cuda/matmul/matmul.cu:99-160 for the quantized routes:
//
//   * s8/u8 x s8 -> s32 | s8 | u8 | f32 | f16 with the fused epilogue (every pose, batch
//     broadcast over up to four leading axes);
//   * f16/f32 x q4_1 [N,K] -> f16/f32, which the reference serves on the CPU only;
//   * f16/f32 activations carrying QuantParams x s8 weights -> the activation dtype: quantize
//     on the fly, int8 GEMM, dequantizing epilogue (CPU-only in the reference,
//     src/backend/cpu/matmul/matmul_i8.cpp:389-464).
//
// Compiled against the real nnops headers when NNB200_USE_NNOPS_HEADERS is defined (the
// maintainer's integration), else against the stand-alone mirror.
//
// Semantics kept from the reference: integer destinations honour only Relu and ignore
// alpha/beta and the clip bounds; a rejected call writes nothing; an empty output is ok;
// QuantParams arrays may be host memory (staged per call, stream-ordered, like the reference
// launcher does) or device memory (used in place).

#ifdef NNB200_USE_NNOPS_HEADERS
#include "nnops/ops/linear.hpp"
#include "nnops/ops/matmul.hpp"
#else
#include "nnops_b200/nnops_api.hpp"
#endif

#include "nnb200.h"
#include "staging.hpp"

#include <algorithm>
#include <array>
#include <cstring>
#include <vector>

namespace nnops::backend::cuda {

using namespace b200_detail;

namespace {

constexpr int kMaxBatchRank = 4;          // rank-6 operands: four broadcastable batch axes
constexpr int64_t kMaxBatchCount = 65535; // the reference refuses larger flattened batches

// Batch geometry after numpy-style broadcasting of the leading axes of a and b.
struct BatchLayout {
    int rank = 0;
    int64_t size[kMaxBatchRank] = {1, 1, 1, 1};
    int64_t a_stride[kMaxBatchRank] = {0, 0, 0, 0};
    int64_t b_stride[kMaxBatchRank] = {0, 0, 0, 0};
    int64_t c_stride[kMaxBatchRank] = {0, 0, 0, 0};
    int64_t count = 1;
};

bool batch_layout(const TensorView& a, const TensorView& b, const TensorView& c, BatchLayout& L)
{
    const int64_t al = std::max<int64_t>(a.rank() - 2, 0);
    const int64_t bl = std::max<int64_t>(b.rank() - 2, 0);
    const int64_t rank = std::max(al, bl);
    if (rank > kMaxBatchRank) {
        return false;
    }
    L.rank = static_cast<int>(rank);
    for (int64_t d = 0; d < rank; ++d) {
        const int64_t ai = al - 1 - d, bi = bl - 1 - d, ci = c.rank() - 3 - d;
        const int64_t ad = ai >= 0 ? a.shape(ai) : 1;
        const int64_t bd = bi >= 0 ? b.shape(bi) : 1;
        if (ad != bd && ad != 1 && bd != 1) {
            return false;
        }
        const int64_t slot = rank - 1 - d;
        L.size[slot] = std::max(ad, bd);
        L.a_stride[slot] = ad == 1 ? 0 : a.stride_elems(ai);
        L.b_stride[slot] = bd == 1 ? 0 : b.stride_elems(bi);
        L.c_stride[slot] = ci >= 0 ? c.stride_elems(ci) : 0;
        if (L.size[slot] > kMaxBatchCount) {
            return false;
        }
        L.count *= L.size[slot];
        if (L.count > kMaxBatchCount) {
            return false;
        }
    }
    return true;
}

// True for a weight view that holds nnb200_i8_pack's blob (stand-alone API only: the reference's
// layout enumeration has no such tag, and its CUDA operators answer "no packed form").
bool is_packed_i8(const TensorView& w)
{
#ifdef NNB200_USE_NNOPS_HEADERS
    (void)w;
    return false;
#else
    return w.layout() == TensorLayout::PackedI8B200;
#endif
}

struct I8Call {
    const TensorView* a;
    const TensorView* w;
    const TensorView* bias;
    TensorView* out;
    bool transpose_a;   // A stored [K, M]
    bool w_is_nk;       // W stored [N, K] (Linear, or MatMul with transpose_b)
    const Epilogue* ep;
    int kind;
};

Status run_i8(const I8Call& c, const ComputeContext& ctx)
{
    const TensorView& a = *c.a;
    const TensorView& w = *c.w;
    TensorView& out = *c.out;
    if (a.rank() < 2 || w.rank() < 2 || out.rank() < 2) {
        return Status::invalid_argument;
    }
    const int64_t M = c.transpose_a ? a.shape(a.rank() - 1) : a.shape(a.rank() - 2);
    const int64_t Ka = c.transpose_a ? a.shape(a.rank() - 2) : a.shape(a.rank() - 1);
    const int64_t Kb = c.w_is_nk ? w.shape(w.rank() - 1) : w.shape(w.rank() - 2);
    const int64_t N = c.w_is_nk ? w.shape(w.rank() - 2) : w.shape(w.rank() - 1);
    if (Ka != Kb) {
        return Status::invalid_argument;
    }
    BatchLayout L;
    if (!batch_layout(a, w, out, L)) {
        return Status::unsupported;
    }

    nnb200_gemm_i8_args g;
    std::memset(&g, 0, sizeof(g));
    g.m = M;
    g.n = N;
    g.k = Ka;
    g.a_stride_m = c.transpose_a ? 1 : a.row_stride_elems();
    g.a_stride_k = c.transpose_a ? a.row_stride_elems() : 1;
    g.w_stride_n = c.w_is_nk ? w.row_stride_elems() : 1;
    g.w_stride_k = c.w_is_nk ? 1 : w.row_stride_elems();
    nnb200_i8_packed pk{};
    const bool packed = is_packed_i8(w);
    if (packed) {
        // The blob holds W as [N][pitch], its per-channel arrays and its row sums on the device.
        if (nnb200_i8_packed_view(w.ptr<void>(), N, Ka, &pk) != NNB200_OK) {
            return Status::invalid_argument;
        }
        g.w_stride_n = pk.pitch;
        g.w_stride_k = 1;
        g.r_w = pk.r_w;
    }
    g.ldc = out.row_stride_elems();
    g.batch = 1;
    g.a_unsigned = a.data_type() == DataType::u8;
    g.out_kind = c.kind;
    const bool int_out = c.kind <= NNB200_OUT_U8;
    g.relu = int_out && c.ep->type == EpilogueActivateType::Relu;
    g.activation = static_cast<int32_t>(c.ep->type);
    g.act_alpha = c.ep->alpha;
    g.act_beta = c.ep->beta;
    g.min_clip = c.ep->min_clip;
    g.max_clip = c.ep->max_clip;

    const QuantParams& qa = a.quant_params();
    const QuantParams& qw = w.quant_params();
    g.scale_a_scalar = qa.scale;
    g.scale_w_scalar = qw.scale;
    g.zp_a_scalar = qa.zero_point;
    g.zp_w_scalar = qw.zero_point;
    g.out_scale = 1.0f;
    if (int_out) {
        // Output parameters are per-tensor; element 0 of an array form is read on the host.
        const QuantParams& qc = out.quant_params();
        if ((qc.scale_data != nullptr && nnb200_is_device_pointer(qc.scale_data)) ||
            (qc.zero_point_data != nullptr && nnb200_is_device_pointer(qc.zero_point_data))) {
            return Status::unsupported;
        }
        g.out_scale = qc.scale_data != nullptr ? qc.scale_data[0] : qc.scale;
        g.out_zp = qc.zero_point_data != nullptr ? qc.zero_point_data[0] : qc.zero_point;
    }
    g.bias = c.bias != nullptr ? c.bias->ptr<void>() : nullptr;

    // Stage host-side arrays, then size the kernels' scratch with the final argument block.
    Staging st(ctx.cuda_stream);
    const size_t m_bytes = static_cast<size_t>(M) * 4, n_bytes = static_cast<size_t>(N) * 4;
    st.reserve(qa.scale_data, m_bytes);
    st.reserve(qa.zero_point_data, m_bytes);
    if (!packed) {
        st.reserve(qw.scale_data, n_bytes);
        st.reserve(qw.zero_point_data, n_bytes);
    }
    // Scratch for the two zero-point sweeps, only when some zero point can be non-zero.
    if (qa.zero_point != 0 || qw.zero_point != 0 || qa.zero_point_data != nullptr || qw.zero_point_data != nullptr) {
        st.reserve_raw(((m_bytes + 255) & ~size_t(255)) + ((n_bytes + 255) & ~size_t(255)));
    }
    // Optional scratch with which the few-row engine shares K evenly among the SMs.  The library
    // sizes it from shapes and pointers alone (zero points do not enter), so the block as filled
    // so far is enough to ask.
    g.a = a.ptr<void>();
    g.w = w.ptr<void>();
    g.out = out.ptr<void>();
    st.reserve_raw(nnb200_gemm_i8_workspace_bytes(&g) - nnb200_gemm_i8_min_workspace_bytes(&g));
    if (const int e = st.allocate(); e != NNB200_OK) {
        return to_status(e);
    }
    DeviceArray sa, za, sw, zw;
    for (const int e : {st.place(qa.scale_data, m_bytes, false, sa), st.place(qa.zero_point_data, m_bytes, true, za)}) {
        if (e != NNB200_OK) {
            return to_status(e);
        }
    }
    if (packed) {
        // Per-channel arrays were copied into the blob at pack time; the view's own (host) arrays
        // only tell which of them are in use, and whether any zero point is non-zero.
        if (qw.scale_data != nullptr) {
            sw.ptr = pk.scale_w;
        }
        if (qw.zero_point_data != nullptr) {
            zw.ptr = pk.zp_w;
            zw.any_nonzero = nnb200_is_device_pointer(qw.zero_point_data) != 0 ||
                             std::any_of(qw.zero_point_data, qw.zero_point_data + N, [](int32_t x) { return x != 0; });
        }
    } else {
        for (const int e : {st.place(qw.scale_data, n_bytes, false, sw), st.place(qw.zero_point_data, n_bytes, true, zw)}) {
            if (e != NNB200_OK) {
                return to_status(e);
            }
        }
    }
    g.scale_a = static_cast<const float*>(sa.ptr);
    g.zp_a = static_cast<const int32_t*>(za.ptr);
    g.scale_w = static_cast<const float*>(sw.ptr);
    g.zp_w = static_cast<const int32_t*>(zw.ptr);
    g.zp_a_nonzero = za.ptr != nullptr && za.any_nonzero;
    g.zp_w_nonzero = zw.ptr != nullptr && zw.any_nonzero;
    g.a = a.ptr<void>();
    g.w = w.ptr<void>();
    g.out = out.ptr<void>();
    // Zero-point scratch is sized from the argument block; reserve it now that the block is final.
    const size_t need = nnb200_gemm_i8_workspace_bytes(&g);
    if (need > 0) {
        g.workspace = st.take_raw(need);
        g.workspace_bytes = need;
        if (g.workspace == nullptr) {
            return Status::internal;
        }
    }

    // Walk the broadcast batch; each slice is one 2-D call.
    const size_t out_elem = data_type_size(out.data_type());
    std::array<int64_t, kMaxBatchRank> idx{};
    for (int64_t b = 0; b < L.count; ++b) {
        int64_t ao = 0, wo = 0, co = 0;
        for (int d = 0; d < L.rank; ++d) {
            ao += idx[static_cast<size_t>(d)] * L.a_stride[d];
            wo += idx[static_cast<size_t>(d)] * L.b_stride[d];
            co += idx[static_cast<size_t>(d)] * L.c_stride[d];
        }
        g.a = a.ptr<char>() + ao;  // 1-byte elements
        g.w = w.ptr<char>() + wo;
        g.out = out.ptr<char>() + co * static_cast<int64_t>(out_elem);
        if (const int e = nnb200_gemm_i8(&g, ctx.cuda_stream); e != NNB200_OK) {
            return to_status(e);
        }
        for (int d = L.rank - 1; d >= 0; --d) {
            if (++idx[static_cast<size_t>(d)] < L.size[d]) {
                break;
            }
            idx[static_cast<size_t>(d)] = 0;
        }
    }
    return Status::ok;
}

// f32/f16 activations with active per-tensor / per-token QuantParams x s8 weights: A is
// quantised with ITS parameters (fma(x, 1/scale, zp), round-half-even, saturate to
// act_dtype -- the QuantizeLinear arithmetic), the int8 GEMM runs on the result and its
// dequantizing epilogue writes A's dtype.  Per-token arrays are indexed by the global row over
// all leading axes, as the reference's dequantizing route does (matmul_tile_impl.h:454-463).
Status run_dq_from_fp(const TensorView& a, const TensorView& w, const TensorView* bias, TensorView& out,
                      bool transpose_a, bool w_is_nk, DataType act_dtype, const Epilogue& ep,
                      const ComputeContext& ctx)
{
    const QuantParams& qp = a.quant_params();
    const bool quantized = qp.is_active() && (qp.granularity == QuantGranularity::PerTensor ||
                                              qp.granularity == QuantGranularity::PerToken);
    if (!quantized) {
        return Status::invalid_argument;  // a float A without parameters is not a quantized tensor
    }
    if (transpose_a || out.data_type() != a.data_type()) {
        return Status::unsupported;
    }
    if (act_dtype != DataType::s8 && act_dtype != DataType::u8) {
        return Status::unsupported;
    }
    if (a.rank() < 2 || w.rank() != 2 || out.rank() != a.rank()) {
        return Status::unsupported;  // batched weights are not served on this route
    }
    const int64_t K = a.shape(a.rank() - 1);
    const int64_t rows = K > 0 ? a.numel() / K : 0;
    if (a.row_stride_elems() != K) {
        return Status::unsupported;  // the quantising pass walks A as one dense array
    }
    const bool per_token = qp.scale_data != nullptr || qp.zero_point_data != nullptr;
    const int64_t count = per_token ? rows : 1;

    // Scratch: A_q, then scale / zero-point arrays when they are not already on the device.
    Staging st(ctx.cuda_stream);
    st.reserve_raw(static_cast<size_t>(rows * K));
    const size_t p_bytes = static_cast<size_t>(count) * 4;
    const bool scale_dev = qp.scale_data != nullptr && nnb200_is_device_pointer(qp.scale_data) != 0;
    const bool zp_dev = qp.zero_point_data != nullptr && nnb200_is_device_pointer(qp.zero_point_data) != 0;
    if (!scale_dev) {
        st.reserve_raw(p_bytes);
    }
    if (!zp_dev) {
        st.reserve_raw(p_bytes);
    }
    if (const int e = st.allocate(); e != NNB200_OK) {
        return to_status(e);
    }
    void* aq = st.take_raw(static_cast<size_t>(rows * K));
    std::vector<float> scale_h;
    std::vector<int32_t> zp_h;
    const float* scale_d = qp.scale_data;
    const void* zp_d = qp.zero_point_data;
    if (!scale_dev) {
        if (qp.scale_data != nullptr) {
            scale_h.assign(qp.scale_data, qp.scale_data + count);
        } else {
            scale_h.assign(static_cast<size_t>(count), qp.scale);
        }
        void* d = st.take_raw(p_bytes);
        if (const int e = nnb200_copy_h2d_async(d, scale_h.data(), p_bytes, ctx.cuda_stream); e != NNB200_OK) {
            return to_status(e);
        }
        scale_d = static_cast<const float*>(d);
    }
    if (!zp_dev) {
        if (qp.zero_point_data != nullptr) {
            zp_h.assign(qp.zero_point_data, qp.zero_point_data + count);
        } else {
            zp_h.assign(static_cast<size_t>(count), qp.zero_point);
        }
        void* d = st.take_raw(p_bytes);
        if (const int e = nnb200_copy_h2d_async(d, zp_h.data(), p_bytes, ctx.cuda_stream); e != NNB200_OK) {
            return to_status(e);
        }
        zp_d = d;
    }
    // The staged host vectors are pageable memory: the copies above have completed from the
    // host's point of view when the calls return (pageable cudaMemcpyAsync stages first).

    nnb200_quant_linear_args q;
    std::memset(&q, 0, sizeof(q));
    q.x = a.ptr<void>();
    q.y = aq;
    q.outer = 1;
    q.rows = per_token ? rows : 1;
    q.inner = per_token ? K : rows * K;
    q.scale = scale_d;
    q.zero_point = zp_d;
    q.zp_unsigned = NNB200_ZP_S32;
    q.float_f16 = a.data_type() == DataType::f16;
    q.int_unsigned = act_dtype == DataType::u8;
    if (const int e = nnb200_quantize_linear(&q, ctx.cuda_stream); e != NNB200_OK) {
        return to_status(e);
    }

    // The int8 GEMM over A_q as one tall [rows, K] matrix with A's parameters.
    const int64_t a2[] = {rows, K};
    const int64_t o2[] = {rows, out.shape(out.rank() - 1)};
    QuantParams aq_qp = qp;
    if (per_token) {
        aq_qp.scale_data = qp.scale_data != nullptr ? scale_d : nullptr;
        aq_qp.zero_point_data = qp.zero_point_data != nullptr ? static_cast<const int32_t*>(zp_d) : nullptr;
    }
    TensorView aq_view(a2, act_dtype, aq, TensorLayout::Dense, aq_qp);
    TensorView out2(o2, out.data_type(), out.ptr<void>(), out.pitch(), TensorLayout::Dense, out.quant_params());
    int kind;
    if (!out_kind_of(out.data_type(), kind)) {
        return Status::unsupported;
    }
    const I8Call call{&aq_view, &w, bias, &out2, false, w_is_nk, &ep, kind};
    return run_i8(call, ctx);
}

// f16/f32 activations x q4_1 weights stored [N, K].
Status run_q4_1(const TensorView& x, const TensorView& w, const TensorView* bias, TensorView& out, float alpha,
                const Epilogue& ep, const ComputeContext& ctx)
{
    if (w.rank() != 2 || x.rank() < 2 || out.rank() < 2) {
        return Status::unsupported;
    }
    const DataType xdt = x.data_type();
    const DataType odt = out.data_type();
    if ((xdt != DataType::f16 && xdt != DataType::f32) || (odt != DataType::f16 && odt != DataType::f32)) {
        return Status::unsupported;
    }
    if (xdt == DataType::f32 && odt == DataType::f16) {
        return Status::unsupported;  // the output is at least as wide as the activations
    }
    const int64_t K = x.shape(x.rank() - 1);
    const int64_t N = w.shape(0);
    if (w.shape(1) != K) {
        return Status::invalid_argument;
    }
    if (bias != nullptr && bias->data_type() != odt) {
        return Status::invalid_argument;
    }
    // Leading axes of x are rows of one tall matrix when they are densely pitched.
    int64_t rows = 1;
    for (int64_t d = 0; d + 1 < x.rank(); ++d) {
        rows *= x.shape(d);
    }
    nnb200_q4_1_args q;
    std::memset(&q, 0, sizeof(q));
    q.a = x.ptr<void>();
    q.w_blocks = w.ptr<void>();
    q.out = out.ptr<void>();
    q.m = rows;
    q.n = N;
    q.k = K;
    q.lda = x.row_stride_elems();
    q.ldw_blocks = w.row_stride_elems();
#ifndef NNB200_USE_NNOPS_HEADERS
    if (w.layout() == TensorLayout::PackedQ4_1B200) {
        // A prepacked weight: the view's data is nnb200_q4_1_pack's blob.
        nnb200_q4_1_packed planes;
        if (nnb200_q4_1_packed_view(w.ptr<void>(), N, K, &planes) != NNB200_OK) {
            return Status::invalid_argument;
        }
        q.w_blocks = planes.qs;
        q.ldw_blocks = planes.qs_pitch;
        q.w_dm = planes.dm;
        q.ld_dm = planes.dm_pitch;
    }
#endif
    q.ldc = out.row_stride_elems();
    q.a_f16 = xdt == DataType::f16;
    q.out_f16 = odt == DataType::f16;
    q.bias = bias != nullptr ? bias->ptr<void>() : nullptr;
    q.activation = static_cast<int32_t>(ep.type);
    q.act_alpha = ep.alpha;
    q.act_beta = ep.beta;
    q.min_clip = ep.min_clip;
    q.max_clip = ep.max_clip;
    q.alpha = alpha;
    // Tall problems run faster with scratch for the expanded weights (stream-ordered, freed
    // right after the launch is enqueued).
    Staging st(ctx.cuda_stream);
    if (const size_t need = nnb200_q4_1_workspace_bytes(&q); need > 0) {
        st.reserve_raw(need);
        if (st.allocate() == NNB200_OK) {
            q.workspace = st.take_raw(need);
            q.workspace_bytes = need;
        }
    }
    return to_status(nnb200_linear_q4_1(&q, ctx.cuda_stream));
}

}  // namespace

Status linear_cuda(const LinearAttributes& attrs, TensorView& output, std::span<const TensorView> inputs,
                   const ComputeContext& ctx, void*)
{
    const TensorView& x = inputs[0];
    const TensorView& w = inputs[1];
    const TensorView* bias = inputs.size() > 2 ? &inputs[2] : nullptr;
    if (attrs.gated) {
        return Status::unsupported;  // the gated combine has no CUDA route (reference linear.cu:102)
    }
    if (is_int8_matmul(x.data_type(), w.data_type())) {
        if (output.numel() == 0) {
            return Status::ok;
        }
        int kind;
        if (!out_kind_of(output.data_type(), kind)) {
            return Status::unsupported;
        }
        if (attrs.add_to) {
            return Status::unsupported;  // no residual on the integer route (reference linear.cu:34)
        }
        if (w.rank() != 2) {
            return Status::invalid_argument;
        }
        const I8Call call{&x, &w, bias, &output, false, true, &attrs.epilogue, kind};
        return run_i8(call, ctx);
    }
    if (w.data_type() == DataType::q4_1) {
        if (output.numel() == 0) {
            return Status::ok;
        }
        if (attrs.add_to) {
            return Status::unsupported;
        }
        return run_q4_1(x, w, bias, output, 1.0f, attrs.epilogue, ctx);
    }
    if ((x.data_type() == DataType::f32 || x.data_type() == DataType::f16) && w.data_type() == DataType::s8) {
        if (output.numel() == 0) {
            return Status::ok;
        }
        if (attrs.add_to) {
            return Status::unsupported;
        }
        return run_dq_from_fp(x, w, bias, output, false, true, DataType::s8, attrs.epilogue, ctx);
    }
    return Status::unsupported;  // dense fp Linear is outside this backend
}

#ifndef NNB200_USE_NNOPS_HEADERS
// Two-step prepack of a 2-D s8 weight: an empty `packed` is set to the geometry of the blob (a
// [N, K] s8 view tagged PackedI8B200 whose pitch gives N * pitch = the blob's bytes, carrying the
// weight's QuantParams); a populated one is filled on the stream.  Anything else answers
// "no packed form" by leaving `packed` alone.
void prepack_i8_cuda(const TensorView& weight, bool w_is_nk, TensorView& packed, const ComputeContext& ctx)
{
    if (weight.data_type() != DataType::s8 || weight.rank() != 2) {
        return;
    }
    const int64_t n = w_is_nk ? weight.shape(0) : weight.shape(1);
    const int64_t k = w_is_nk ? weight.shape(1) : weight.shape(0);
    if (n <= 0 || k <= 0) {
        return;
    }
    const int64_t pitch = static_cast<int64_t>(nnb200_i8_pack_bytes(n, k)) / n;
    const int64_t shape[2] = {n, k};
    if (packed.is_empty()) {
        packed = TensorView(shape, DataType::s8, nullptr, pitch, TensorLayout::PackedI8B200, weight.quant_params());
        return;
    }
    if (packed.layout() != TensorLayout::PackedI8B200 || packed.rank() != 2 || packed.shape(0) != n ||
        packed.shape(1) != k || packed.pitch() != pitch) {
        return;  // not the geometry the query gave
    }
    const QuantParams& q = weight.quant_params();
    nnb200_i8_pack(weight.ptr<void>(), n, k, w_is_nk ? weight.row_stride_elems() : 1,
                   w_is_nk ? 1 : weight.row_stride_elems(), q.scale_data, q.scale, q.zero_point_data, q.zero_point,
                   packed.ptr<void>(), static_cast<size_t>(n * pitch), ctx.cuda_stream);
}
#endif

#ifndef NNB200_USE_NNOPS_HEADERS
// Two-step prepack of a 2-D q4_1 weight stored [N, K]: an empty `packed` is set to the geometry of
// the blob (a [N, K] q4_1 view tagged PackedQ4_1B200 whose pitch, a whole number of 20-byte
// units, makes N * pitch cover the blob); a populated one is filled on the stream.
void prepack_q4_1_cuda(const TensorView& weight, TensorView& packed, const ComputeContext& ctx)
{
    if (weight.data_type() != DataType::q4_1 || weight.rank() != 2) {
        return;
    }
    const int64_t n = weight.shape(0), k = weight.shape(1);
    if (n <= 0 || k <= 0) {
        return;
    }
    const size_t bytes = nnb200_q4_1_pack_bytes(n, k);
    const int64_t per_row = static_cast<int64_t>(bytes / static_cast<size_t>(n));
    const int64_t pitch = (per_row + 19) / 20 * 20;
    const int64_t shape[2] = {n, k};
    if (packed.is_empty()) {
        packed = TensorView(shape, DataType::q4_1, nullptr, pitch, TensorLayout::PackedQ4_1B200, QuantParams{});
        return;
    }
    if (packed.layout() != TensorLayout::PackedQ4_1B200 || packed.rank() != 2 || packed.shape(0) != n ||
        packed.shape(1) != k || packed.pitch() != pitch) {
        return;  // not the geometry the query gave
    }
    nnb200_q4_1_pack(weight.ptr<void>(), weight.row_stride_elems(), n, k, packed.ptr<void>(),
                     static_cast<size_t>(n * pitch), ctx.cuda_stream);
}
#endif

Status matmul_cuda(const MatMulAttributes& attrs, TensorView& output, std::span<const TensorView> inputs,
                   const ComputeContext& ctx, void*)
{
    const TensorView& a = inputs[0];
    const TensorView& b = inputs[1];
    const TensorView* bias = inputs.size() > 2 ? &inputs[2] : nullptr;
    if (is_int8_matmul(a.data_type(), b.data_type())) {
        if (output.numel() == 0) {
            return Status::ok;
        }
        int kind;
        if (!out_kind_of(output.data_type(), kind)) {
            return Status::unsupported;
        }
        const I8Call call{&a, &b, bias, &output, attrs.transpose_a, attrs.transpose_b || is_packed_i8(b), &attrs.epilogue,
                          kind};
        return run_i8(call, ctx);
    }
    if (b.data_type() == DataType::q4_1) {
        if (output.numel() == 0) {
            return Status::ok;
        }
        // Only the [N, K] weight pose with row-major activations is served; no accumulate into C.
        if (!attrs.transpose_b || attrs.transpose_a || attrs.beta != 0.0f) {
            return Status::unsupported;
        }
        return run_q4_1(a, b, bias, output, attrs.alpha, attrs.epilogue, ctx);
    }
    if ((a.data_type() == DataType::f32 || a.data_type() == DataType::f16) && b.data_type() == DataType::s8) {
        if (output.numel() == 0) {
            return Status::ok;
        }
        if (attrs.beta != 0.0f) {
            return Status::unsupported;
        }
        return run_dq_from_fp(a, b, bias, output, attrs.transpose_a, attrs.transpose_b, attrs.act_quant_dtype,
                              attrs.epilogue, ctx);
    }
    return Status::unsupported;
}

}  // namespace nnops::backend::cuda
