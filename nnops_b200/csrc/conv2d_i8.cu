// int8 Conv2D (NHWC u8/s8 activation x s8 HWIO filter) as a gather pass + the int8 GEMM.
//
// Counterpart of the reference's quantized convolution route
// (src/backend/cuda/conv/conv2d_i8.cu:358-785 kernel, :910-1100 host entry): pixels on M, output
// channels of one group on N, k = (tap, channel) tap-major.  There the gather runs inside an
// mma.sync tile kernel; here the product itself belongs to the tcgen05 GEMM (gemm_i8_umma.cu and
// the small-M engines behind nnb200_gemm_i8), and what is convolution-specific is done by two
// streaming kernels in front of it:
//
//   conv_gather_i8_kernel     activation -> column matrix  col[g][pixel][k], 16 bytes per thread
//                             where a group's channels allow it.  A tap that falls into the
//                             padding carries the activation's zero point (the real value 0),
//                             which is what the reference's CPU and CUDA gathers store
//                             (conv2d_i8.cu:112-121) so that the zero-point compensation cancels it.
//   conv_filter_kmajor_kernel HWIO filter -> [g][oc/g][k] with k contiguous (the Linear pose every
//                             GEMM engine accepts); conv_filter_sums_kernel adds the per-channel
//                             sums R_w.  Run per call on a raw filter (it is small), or once by
//                             nnb200_conv2d_i8_pack.
//
// Convolutions with strides of 1 or 2 over whole 128-channel blocks per group with symmetric weights skip the
// gather altogether (the implicit-GEMM form, launch_conv_i8_umma in gemm_i8_umma.cu): the GEMM's
// producer reads the activation itself, one 4-D TMA box {128 channels, bw, bh, 1 image} per
// k-block (tap, channel block) at the patch's origin shifted by the tap -- out-of-image parts are
// filled with zeros by the copy engine -- and the epilogue adds the zero point's share back for
// rows whose window overhangs: zp_x times the filter's channel sums over the lost taps, one of a
// few rows of a small table (conv_border_table_kernel) picked by the row's border class.
//
// A 1x1 / stride 1 / unpadded convolution over a dense activation needs no gather: the activation
// IS the [pixels, channels] matrix.  The epilogue is the GEMM's (compensation, int32 bias, Relu,
// requantisation; or dequantisation, fp bias, clip, activation): the reference's CPU convolution
// calls the same epilogue routine as its matmul (src/backend/cpu/conv/conv2d_implicit_gemm_i8.cpp:
// 906-980), and results are compared with that route bit for bit.

#include <cstring>

#include "internal.cuh"
#include "epilogue.cuh"

namespace nnb200 {

namespace {

struct ConvGeom {
    int64_t batch, ih, iw, ic, oh, ow, oc;
    int64_t kh, kw, sh, sw, dh, dw, ph, pw, groups;
    int64_t icg, ocg, k, kp;   // k = kh*kw*icg; kp = k rounded up to 16 (row pitch of the column matrix)
    int64_t pixels;            // batch * oh * ow
};

struct GatherParams {
    const uint8_t* in;
    uint8_t* col;
    int64_t in_n, in_h, in_w, in_c;   // element strides of the activation
    int32_t batch, ih, iw, oh, ow;
    int32_t kh, kw, sh, sw, dh, dw, ph, pw, groups, icg;
    int32_t k, kp;
    int64_t pixels;
    uint32_t pad_byte;   // the activation's zero point as a byte
};

// One thread per 16-byte piece of the column matrix (16 consecutive k of one pixel and group);
// a block takes `rows_per_block` rows (pixel, group) at a time.  What a piece needs to know about
// its tap (input offset of the tap, first channel) and about its row (image and group base,
// window origin) is decoded once per block into shared memory, so the per-piece work is one
// 32-bit division, two table reads, the bounds test, one load and one store.
// VEC: the 16 k are 16 consecutive channels of one tap (icg % 16 == 0, dense channel axis,
// 16-byte aligned rows), one 128-bit load; otherwise each byte finds its own tap.
template <bool VEC>
__global__ void __launch_bounds__(256) conv_gather_i8_kernel(const GatherParams p, const int rows_per_block)
{
    extern __shared__ __align__(8) uint8_t gather_smem[];
    const int cpr = p.kp >> 4;   // pieces per row
    int64_t* row_base = reinterpret_cast<int64_t*>(gather_smem);          // [rows_per_block]
    int32_t* row_ih0 = reinterpret_cast<int32_t*>(row_base + rows_per_block);
    int32_t* row_iw0 = row_ih0 + rows_per_block;
    int32_t* tap_dh = row_iw0 + rows_per_block;                            // [cpr] of the piece's first k
    int32_t* tap_dw = tap_dh + cpr;
    int32_t* tap_c = tap_dw + cpr;
    int32_t* tap_id = tap_c + cpr;                                         // kh * kw_count + kw (byte-wise path)

    for (int c = threadIdx.x; c < cpr; c += blockDim.x) {
        const int32_t k0 = c << 4;
        const int32_t tap = k0 / p.icg;
        const int32_t kh = tap / p.kw;
        const int32_t kw = tap - kh * p.kw;
        tap_dh[c] = kh * p.dh;
        tap_dw[c] = kw * p.dw;
        tap_c[c] = k0 - tap * p.icg;
        tap_id[c] = tap;
    }
    const int64_t rows_total = static_cast<int64_t>(p.groups) * p.pixels;
    const int32_t plane = p.oh * p.ow;
    for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * rows_per_block; row0 < rows_total;
         row0 += static_cast<int64_t>(gridDim.x) * rows_per_block) {
        __syncthreads();   // the previous batch's readers are done (and the tap table is written)
        for (int r = threadIdx.x; r < rows_per_block; r += blockDim.x) {
            const int64_t row = row0 + r;
            if (row < rows_total) {
                const int32_t g = static_cast<int32_t>(row / p.pixels);
                const int32_t pixel = static_cast<int32_t>(row - static_cast<int64_t>(g) * p.pixels);
                const int32_t n = pixel / plane;
                const int32_t rem = pixel - n * plane;
                const int32_t oh = rem / p.ow;
                const int32_t ow = rem - oh * p.ow;
                row_base[r] = static_cast<int64_t>(n) * p.in_n + static_cast<int64_t>(g) * p.icg * p.in_c;
                row_ih0[r] = oh * p.sh - p.ph;
                row_iw0[r] = ow * p.sw - p.pw;
            }
        }
        __syncthreads();
        // A warp walks the pieces of one row at a time (lanes = consecutive pieces: coalesced and
        // no division); rows shorter than a warp share one, `rows_per_warp` at a time.
        const int lane = threadIdx.x & 31;
        const int warp = threadIdx.x >> 5;
        const int rows_per_warp = cpr >= 32 ? 1 : 32 / cpr;
        const int sub_row = cpr >= 32 ? 0 : lane / cpr;
        const int c_first = cpr >= 32 ? lane : lane - sub_row * cpr;
        const int c_step = cpr >= 32 ? 32 : cpr;   // short rows: one piece per lane, the loop below runs once
        for (int r = warp * rows_per_warp + sub_row; r < rows_per_block && sub_row < rows_per_warp;
             r += 8 * rows_per_warp) {
          for (int c = c_first; c < cpr; c += c_step) {
            const int64_t row = row0 + r;
            if (row >= rows_total) {
                break;
            }
            const uint8_t* base = p.in + row_base[r];
            uint4 v;
            if constexpr (VEC) {
                const int32_t ih = row_ih0[r] + tap_dh[c];
                const int32_t iw = row_iw0[r] + tap_dw[c];
                const uint32_t pad4 = p.pad_byte * 0x01010101u;
                v = make_uint4(pad4, pad4, pad4, pad4);
                if (static_cast<uint32_t>(ih) < static_cast<uint32_t>(p.ih) &&
                    static_cast<uint32_t>(iw) < static_cast<uint32_t>(p.iw)) {
                    v = __ldg(reinterpret_cast<const uint4*>(base + static_cast<int64_t>(ih) * p.in_h +
                                                             static_cast<int64_t>(iw) * p.in_w + tap_c[c]));
                }
            } else {
                uint32_t w[4] = {0u, 0u, 0u, 0u};
                int32_t k = c << 4;
                int32_t ch = tap_c[c];
                int32_t kh = tap_id[c] / p.kw;
                int32_t kw = tap_id[c] - kh * p.kw;
#pragma unroll
                for (int j = 0; j < 16; ++j, ++k) {
                    uint32_t byte = 0u;
                    if (k < p.k) {
                        const int32_t ih = row_ih0[r] + kh * p.dh;
                        const int32_t iw = row_iw0[r] + kw * p.dw;
                        byte = p.pad_byte;
                        if (static_cast<uint32_t>(ih) < static_cast<uint32_t>(p.ih) &&
                            static_cast<uint32_t>(iw) < static_cast<uint32_t>(p.iw)) {
                            byte = base[static_cast<int64_t>(ih) * p.in_h + static_cast<int64_t>(iw) * p.in_w +
                                        static_cast<int64_t>(ch) * p.in_c];
                        }
                    }
                    w[j >> 2] |= byte << ((j & 3) * 8);
                    if (++ch == p.icg) {
                        ch = 0;
                        if (++kw == p.kw) {
                            kw = 0;
                            ++kh;
                        }
                    }
                }
                v = make_uint4(w[0], w[1], w[2], w[3]);
            }
            reinterpret_cast<uint4*>(p.col)[row * cpr + c] = v;
          }
        }
    }
}

struct FilterParams {
    const int8_t* w;       // HWIO, element strides below
    int8_t* wt;            // [groups][ocg][kp]
    int64_t w_kh, w_kw, w_ic, w_oc;
    int32_t kh, kw, icg, ocg, groups, k, kp;
};

// 32 x 32 tiles through shared memory: the HWIO filter is read along oc (its contiguous axis),
// the k-major rows are written along k.  Columns k >= K of the padded rows are written as zeros.
__global__ void __launch_bounds__(256) conv_filter_kmajor_kernel(const FilterParams p)
{
    __shared__ int8_t tile[32][33];
    const int tx = threadIdx.x & 31;
    const int ty = threadIdx.x >> 5;   // 0..7
    const int64_t oc = static_cast<int64_t>(p.groups) * p.ocg;
    const int k0 = blockIdx.x * 32;
    const int64_t c0 = static_cast<int64_t>(blockIdx.y) * 32;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int k = k0 + ty * 4 + r;
        const int64_t channel = c0 + tx;
        int8_t v = 0;
        if (k < p.k && channel < oc) {
            const int32_t tap = k / p.icg;
            const int32_t c = k - tap * p.icg;
            const int32_t kh = tap / p.kw;
            const int32_t kw = tap - kh * p.kw;
            v = p.w[kh * p.w_kh + kw * p.w_kw + c * p.w_ic + channel * p.w_oc];
        }
        tile[ty * 4 + r][tx] = v;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int64_t channel = c0 + ty * 4 + r;
        const int k = k0 + tx;
        if (channel < oc && k < p.kp) {
            p.wt[channel * p.kp + k] = tile[tx][ty * 4 + r];   // [g][n] rows are consecutive: g * ocg + n == channel
        }
    }
}

// Channel sums of the k-major filter, one warp per channel (coalesced 4-byte reads; kp is a
// multiple of 16 and the padding is zero).
__global__ void __launch_bounds__(256) conv_filter_sums_kernel(const int8_t* __restrict__ wt, const int64_t oc,
                                                               const int32_t kp, int32_t* __restrict__ r_w)
{
    const int lane = threadIdx.x & 31;
    const int64_t channel = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (channel >= oc) {
        return;
    }
    const int32_t* row = reinterpret_cast<const int32_t*>(wt + channel * kp);
    int32_t sum = 0;
    for (int32_t i = lane; i < kp / 4; i += 32) {
        sum = __dp4a(row[i], 0x01010101, sum);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
    }
    if (lane == 0) {
        r_w[channel] = sum;
    }
}

// Per-tap channel sums of the k-major filter: wtap[tap][channel] = sum over the tap's icg
// weights (icg a multiple of 4: the implicit-GEMM form, which is what reads them, has whole
// 128-channel blocks).  One warp per channel, coalesced 4-byte reads, one reduction per tap.
__global__ void __launch_bounds__(256) conv_filter_tap_sums_kernel(const int8_t* __restrict__ wt, const int64_t oc,
                                                                   const int32_t kp, const int32_t icg, const int32_t taps,
                                                                   int32_t* __restrict__ wtap)
{
    const int lane = threadIdx.x & 31;
    const int64_t channel = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (channel >= oc) {
        return;
    }
    const int32_t* row = reinterpret_cast<const int32_t*>(wt + channel * kp);
    const int32_t words = icg >> 2;
    for (int32_t tap = 0; tap < taps; ++tap) {
        int32_t sum = 0;
        for (int32_t i = lane; i < words; i += 32) {
            sum = __dp4a(row[tap * words + i], 0x01010101, sum);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
        }
        if (lane == 0) {
            wtap[static_cast<int64_t>(tap) * oc + channel] = sum;
        }
    }
}

// Border-class table of the implicit-GEMM form: row (i, j) = sum of the per-tap channel sums
// over the taps (a, b) with a in mask_h[i - 1] or b in mask_w[j - 1] (index 0 = no tap lost).
struct BorderParams {
    const int32_t* wtap;   // [kh * kw][oc]
    int32_t* table;        // [(nh + 1) * (nw + 1)][oc]
    int32_t oc, kh, kw, nh, nw;
    uint32_t mask_h[8], mask_w[8];
};

__global__ void __launch_bounds__(256) conv_border_table_kernel(const BorderParams p)
{
    const int classes = (p.nh + 1) * (p.nw + 1);
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<int64_t>(classes) * p.oc) {
        return;
    }
    const int cls = static_cast<int>(idx / p.oc);
    const int ch = static_cast<int>(idx - static_cast<int64_t>(cls) * p.oc);
    const int i = cls / (p.nw + 1), j = cls - i * (p.nw + 1);
    const uint32_t mh = i > 0 ? p.mask_h[i - 1] : 0u;
    const uint32_t mw = j > 0 ? p.mask_w[j - 1] : 0u;
    int32_t sum = 0;
    for (int a = 0; a < p.kh; ++a) {
        for (int b = 0; b < p.kw; ++b) {
            if (((mh >> a) | (mw >> b)) & 1u) {
                sum += p.wtap[static_cast<int64_t>(a * p.kw + b) * p.oc + ch];
            }
        }
    }
    p.table[idx] = sum;
}

int64_t round_up_i64(int64_t v, int64_t a)
{
    return (v + a - 1) / a * a;
}

// Fills the derived geometry; false when the arguments do not describe a convolution.
bool conv_geometry(const nnb200_conv2d_i8_args* a, ConvGeom* g)
{
    if (a == nullptr || a->batch < 0 || a->ih <= 0 || a->iw <= 0 || a->ic <= 0 || a->oc <= 0 || a->kh <= 0 ||
        a->kw <= 0 || a->stride_h <= 0 || a->stride_w <= 0 || a->dil_h <= 0 || a->dil_w <= 0 || a->pad_h < 0 ||
        a->pad_w < 0 || a->groups <= 0 || a->ic % a->groups != 0 || a->oc % a->groups != 0) {
        return false;
    }
    g->batch = a->batch; g->ih = a->ih; g->iw = a->iw; g->ic = a->ic; g->oc = a->oc;
    g->kh = a->kh; g->kw = a->kw; g->sh = a->stride_h; g->sw = a->stride_w; g->dh = a->dil_h; g->dw = a->dil_w;
    g->ph = a->pad_h; g->pw = a->pad_w; g->groups = a->groups;
    // pad_h / pad_w are the LEADING paddings; the output extent is the caller's (an auto-padded
    // convolution pads the trailing edge by a different amount).  Taps beyond any edge read the
    // zero point; an output extent whose last window would start more than the leading padding
    // plus one filter span past the image is not a convolution of this input.
    const int64_t oh = a->oh, ow = a->ow;
    const int64_t span_h = (a->kh - 1) * a->dil_h + 1, span_w = (a->kw - 1) * a->dil_w + 1;
    if (oh <= 0 || ow <= 0 || (oh - 1) * a->stride_h - a->pad_h > a->ih - 1 + a->pad_h + span_h ||
        (ow - 1) * a->stride_w - a->pad_w > a->iw - 1 + a->pad_w + span_w) {
        return false;
    }
    g->oh = oh; g->ow = ow;
    g->icg = a->ic / a->groups;
    g->ocg = a->oc / a->groups;
    g->k = a->kh * a->kw * g->icg;
    g->kp = round_up_i64(g->k, 16);
    g->pixels = a->batch * oh * ow;
    const int64_t lim = int64_t(1) << 31;
    return g->k < lim && g->pixels < lim && a->ih < 32768 * 16 && a->iw < 32768 * 16 && g->oc < (int64_t(1) << 21);
}

// The activation can be handed to the GEMM as it lies: 1x1, stride 1, no padding, channels
// contiguous, one uniform pixel pitch.
bool pointwise_in_place(const nnb200_conv2d_i8_args* a, const ConvGeom& g)
{
    return g.kh == 1 && g.kw == 1 && g.sh == 1 && g.sw == 1 && g.ph == 0 && g.pw == 0 && a->in_stride_c == 1 &&
           a->in_stride_h == g.iw * a->in_stride_w && (g.batch == 1 || a->in_stride_n == g.ih * a->in_stride_h) &&
           a->in_stride_w % 16 == 0 && reinterpret_cast<uintptr_t>(a->input) % 16 == 0 && g.icg % 16 == 0;
}

struct ConvScratch {
    size_t col_bytes;      // gathered activation, 0 for the in-place pointwise case and the implicit form
    size_t filter_bytes;   // k-major filter, 0 when the caller passed a packed one
    size_t sums_bytes;     // R_w of every channel and the per-tap sums, 0 when packed
    size_t gemm_bytes;     // what one group's GEMM asks for
    size_t total;
};

// The implicit-GEMM form (no gathered copy; launch_conv_i8_umma) takes convolutions with strides of
// 1 or 2 (a stride is the tensor map's element stride along that axis) over whole 128-channel blocks per group whose weights have no zero points, when TMA can
// address the activation (dense channels, 16-byte aligned pitches and base).
bool implicit_form(const nnb200_conv2d_i8_args* a, const ConvGeom& g)
{
    if (knob(NNB200_KNOB_CONV_FORM) == 1) {
        return false;   // measurement switch: always the gather pass + GEMM
    }
    const bool any_size = knob(NNB200_KNOB_CONV_FORM) == 2;   // ... or this form wherever it can run
    const bool zp_w_zero = a->zp_w_scalar == 0 && (a->zp_w == nullptr || a->zp_w_nonzero == 0);
    // Patches of 128 pixels must not pad a small image by more than half again of its pixels.
    int64_t padded = 0;
    conv_patch_log2(static_cast<int>(g.oh), static_cast<int>(g.ow), &padded);
    // ... and small planes (14 x 14 measured a little slower than the gather form, 28 x 28 the
    // same, 56 x 56 1.4x and 112 x 112 1.7x faster) stay on the gather form.
    if (g.oh > 65536 || g.ow > 65536 || (!any_size && (padded * 2 > g.oh * g.ow * 3 || g.oh * g.ow < 700))) {
        return false;
    }
    if (a->zp_x != 0 && g.kh <= 32 && g.kw <= 32) {
        uint32_t masks[8];
        if (conv_border_masks(static_cast<int>(g.oh), static_cast<int>(g.ih), static_cast<int>(g.kh), static_cast<int>(g.sh),
                              static_cast<int>(g.dh), static_cast<int>(g.ph), masks) < 0 ||
            conv_border_masks(static_cast<int>(g.ow), static_cast<int>(g.iw), static_cast<int>(g.kw), static_cast<int>(g.sw),
                              static_cast<int>(g.dw), static_cast<int>(g.pw), masks) < 0) {
            return false;   // more than eight kinds of overhang along an axis
        }
    }
    return g.sh >= 1 && g.sh <= 2 && g.sw >= 1 && g.sw <= 2 && g.icg % 128 == 0 && g.kh <= 32 && g.kw <= 32 && zp_w_zero && a->in_stride_c == 1 &&
           a->in_stride_w % 16 == 0 && a->in_stride_h % 16 == 0 && a->in_stride_n % 16 == 0 &&
           reinterpret_cast<uintptr_t>(a->input) % 16 == 0 && a->in_stride_w >= g.ic && g.oh <= 65536 && g.ow <= 65536 &&
           (g.kh - 1) * g.dh < 32768 && (g.kw - 1) * g.dw < 32768 && g.ph < 32768 && g.pw < 32768;
}

size_t align256(size_t v)
{
    return (v + 255) & ~size_t(255);
}

// One group's GEMM, as nnb200_gemm_i8 arguments (pointers of group 0; the caller offsets them).
void group_gemm_args(const nnb200_conv2d_i8_args* a, const ConvGeom& g, bool in_place, nnb200_gemm_i8_args* q)
{
    *q = nnb200_gemm_i8_args{};
    q->m = g.pixels;
    q->n = g.ocg;
    q->k = g.k;
    q->a_stride_m = in_place ? a->in_stride_w : g.kp;
    q->a_stride_k = 1;
    q->w_stride_n = g.kp;
    q->w_stride_k = 1;
    q->ldc = a->out_stride_w;
    q->batch = 1;
    q->a_unsigned = a->a_unsigned;
    q->out_kind = a->out_kind;
    q->relu = a->relu;
    q->activation = a->activation;
    q->act_alpha = a->act_alpha;
    q->act_beta = a->act_beta;
    q->min_clip = a->min_clip;
    q->max_clip = a->max_clip;
    q->scale_a_scalar = a->scale_x;
    q->scale_w_scalar = a->scale_w_scalar;
    q->zp_a_scalar = a->zp_x;
    q->zp_w_scalar = a->zp_w_scalar;
    q->scale_w = a->scale_w;
    q->zp_w = a->zp_w;
    q->bias = a->bias;
    q->zp_w_nonzero = a->zp_w != nullptr ? a->zp_w_nonzero : 0;
    q->out_scale = a->out_scale;
    q->out_zp = a->out_zp;
    q->force_engine = NNB200_ENGINE_AUTO;
}

bool needs_compensation(const nnb200_conv2d_i8_args* a)
{
    return a->zp_x != 0 || a->zp_w_scalar != 0 || (a->zp_w != nullptr && a->zp_w_nonzero != 0);
}

bool plan_scratch(const nnb200_conv2d_i8_args* a, const ConvGeom& g, bool in_place, ConvScratch* s)
{
    const bool implicit = !in_place && implicit_form(a, g);
    s->col_bytes = (in_place || implicit) ? 0 : align256(static_cast<size_t>(g.groups) * static_cast<size_t>(g.pixels) *
                                                         static_cast<size_t>(g.kp));
    s->filter_bytes = a->weight_packed ? 0 : align256(static_cast<size_t>(g.oc) * static_cast<size_t>(g.kp));
    s->sums_bytes = a->weight_packed ? 0 : align256(static_cast<size_t>(g.oc) * 4) +
                                               align256(static_cast<size_t>(g.oc) * static_cast<size_t>(g.kh * g.kw) * 4);
    if (implicit) {
        // gemm_bytes holds the border-class table here: at most 9 x 9 rows of oc sums.
        s->gemm_bytes = a->zp_x != 0 ? align256(static_cast<size_t>(81) * static_cast<size_t>(g.oc) * 4) : 0;
        s->total = s->filter_bytes + s->sums_bytes + s->gemm_bytes;
        return true;
    }
    nnb200_gemm_i8_args q;
    group_gemm_args(a, g, in_place, &q);
    // Pointers only decide alignment-dependent engine choices: stand-ins with the alignment the
    // real operands will have (scratch sections are 256-byte aligned).
    q.a = in_place ? a->input : reinterpret_cast<const void*>(uintptr_t(4096));
    q.w = reinterpret_cast<const void*>(uintptr_t(4096));
    q.out = a->out;
    s->gemm_bytes = align256(nnb200_gemm_i8_workspace_bytes(&q));
    s->total = s->col_bytes + s->filter_bytes + s->sums_bytes + s->gemm_bytes;
    return true;
}

int out_elem_bytes(int32_t kind)
{
    switch (kind) {
    case NNB200_OUT_S8:
    case NNB200_OUT_U8: return 1;
    case NNB200_OUT_F16: return 2;
    default: return 4;
    }
}

}  // namespace

// Byte size of the packed filter: [oc][kp] k-major rows, then (each section 256-byte aligned)
// int32 sums per channel and int32 sums per (tap, channel).
size_t conv_pack_bytes(int64_t oc, int64_t kp, int64_t taps)
{
    return align256(static_cast<size_t>(oc) * static_cast<size_t>(kp)) + align256(static_cast<size_t>(oc) * 4) +
           static_cast<size_t>(oc) * static_cast<size_t>(taps) * 4;
}

int launch_conv_filter_kmajor(const void* w, int64_t w_kh, int64_t w_kw, int64_t w_ic, int64_t w_oc, int64_t kh,
                              int64_t kw, int64_t icg, int64_t ocg, int64_t groups, void* wt, int32_t* r_w,
                              int32_t* wtap, cudaStream_t stream)
{
    FilterParams f;
    f.w = static_cast<const int8_t*>(w);
    f.wt = static_cast<int8_t*>(wt);
    f.w_kh = w_kh; f.w_kw = w_kw; f.w_ic = w_ic; f.w_oc = w_oc;
    f.kh = static_cast<int32_t>(kh); f.kw = static_cast<int32_t>(kw);
    f.icg = static_cast<int32_t>(icg); f.ocg = static_cast<int32_t>(ocg); f.groups = static_cast<int32_t>(groups);
    f.k = static_cast<int32_t>(kh * kw * icg);
    f.kp = static_cast<int32_t>(round_up_i64(f.k, 16));
    const int64_t oc = ocg * groups;
    const dim3 grid(static_cast<unsigned>((f.kp + 31) / 32), static_cast<unsigned>((oc + 31) / 32));
    conv_filter_kmajor_kernel<<<grid, 256, 0, stream>>>(f);
    note_launch();
    if (r_w != nullptr) {
        conv_filter_sums_kernel<<<static_cast<unsigned>((oc + 7) / 8), 256, 0, stream>>>(f.wt, oc, f.kp, r_w);
        note_launch();
    }
    if (wtap != nullptr) {
        conv_filter_tap_sums_kernel<<<static_cast<unsigned>((oc + 7) / 8), 256, 0, stream>>>(
            f.wt, oc, f.kp, f.icg, static_cast<int32_t>(kh * kw), wtap);
        note_launch();
    }
    return cuda_status(cudaGetLastError());
}

}  // namespace nnb200

using namespace nnb200;

extern "C" {

size_t nnb200_conv2d_i8_workspace_bytes(const nnb200_conv2d_i8_args* a)
{
    ConvGeom g;
    if (!conv_geometry(a, &g)) {
        return 0;
    }
    ConvScratch s;
    plan_scratch(a, g, pointwise_in_place(a, g), &s);
    return s.total;
}

size_t nnb200_conv2d_i8_pack_bytes(int64_t kh, int64_t kw, int64_t ic_per_group, int64_t oc)
{
    if (kh <= 0 || kw <= 0 || ic_per_group <= 0 || oc <= 0) {
        return 0;
    }
    return conv_pack_bytes(oc, round_up_i64(kh * kw * ic_per_group, 16), kh * kw);
}

int nnb200_conv2d_i8_pack(const void* weight, int64_t w_stride_kh, int64_t w_stride_kw, int64_t w_stride_ic,
                          int64_t w_stride_oc, int64_t kh, int64_t kw, int64_t ic_per_group, int64_t oc,
                          int64_t groups, void* blob, void* stream)
{
    if (weight == nullptr || blob == nullptr || kh <= 0 || kw <= 0 || ic_per_group <= 0 || oc <= 0 || groups <= 0 ||
        oc % groups != 0 || oc >= (int64_t(1) << 21) || reinterpret_cast<uintptr_t>(blob) % 16 != 0 ||
        kh * kw * ic_per_group >= (int64_t(1) << 31)) {
        return NNB200_INVALID_ARGUMENT;
    }
    const int64_t kp = round_up_i64(kh * kw * ic_per_group, 16);
    uint8_t* after = static_cast<uint8_t*>(blob) + align256(static_cast<size_t>(oc * kp));
    int32_t* sums = reinterpret_cast<int32_t*>(after);
    int32_t* wtap = reinterpret_cast<int32_t*>(after + align256(static_cast<size_t>(oc) * 4));
    // The per-tap sums serve the implicit-GEMM form only (whole 128-channel blocks per group).
    return launch_conv_filter_kmajor(weight, w_stride_kh, w_stride_kw, w_stride_ic, w_stride_oc, kh, kw, ic_per_group,
                                     oc / groups, groups, blob, sums, ic_per_group % 128 == 0 ? wtap : nullptr,
                                     static_cast<cudaStream_t>(stream));
}

int nnb200_conv2d_i8(const nnb200_conv2d_i8_args* a, void* stream_v)
{
    ConvGeom g;
    if (!conv_geometry(a, &g) || a->input == nullptr || a->weight == nullptr || a->out == nullptr) {
        return NNB200_INVALID_ARGUMENT;
    }
    if (a->out_kind != NNB200_OUT_S8 && a->out_kind != NNB200_OUT_U8 && a->out_kind != NNB200_OUT_F32 &&
        a->out_kind != NNB200_OUT_F16) {
        return NNB200_UNSUPPORTED;   // no s32 destination, as in the reference (conv2d_i8.cu:941-944)
    }
    // The GEMM writes [pixels, oc/g] windows at one row pitch.
    if (a->out_stride_h != g.ow * a->out_stride_w || (g.batch > 1 && a->out_stride_n != g.oh * a->out_stride_h) ||
        a->out_stride_w < g.oc) {
        return NNB200_UNSUPPORTED;
    }
    if (a->weight_packed && reinterpret_cast<uintptr_t>(a->weight) % 16 != 0) {
        return NNB200_INVALID_ARGUMENT;
    }
    // Natural alignment of the arrays the kernels read as 2- or 4-byte words: refused here
    // instead of faulting on the GPU.
    const auto misaligned = [](const void* q, uintptr_t to) { return (reinterpret_cast<uintptr_t>(q) & (to - 1)) != 0; };
    if (misaligned(a->scale_w, 4) || misaligned(a->zp_w, 4) ||
        misaligned(a->bias, a->out_kind == NNB200_OUT_F16 ? 2 : 4)) {
        return NNB200_INVALID_ARGUMENT;
    }
    if (g.pixels == 0) {
        return NNB200_OK;
    }
    const bool in_place = pointwise_in_place(a, g);
    const bool implicit = !in_place && implicit_form(a, g);   // the same decision plan_scratch takes
    if (!in_place && !implicit && g.kp / 16 > 2048) {
        return NNB200_UNSUPPORTED;   // the gather's tap table is sized for K <= 32768
    }
    ConvScratch plan;
    plan_scratch(a, g, in_place, &plan);
    if (plan.total > 0 && (a->workspace == nullptr || a->workspace_bytes < plan.total ||
                           reinterpret_cast<uintptr_t>(a->workspace) % 16 != 0)) {
        return NNB200_INVALID_ARGUMENT;
    }
    const cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    uint8_t* ws = static_cast<uint8_t*>(a->workspace);
    uint8_t* col = ws;
    int8_t* wt = reinterpret_cast<int8_t*>(ws + plan.col_bytes);
    int32_t* r_w = reinterpret_cast<int32_t*>(ws + plan.col_bytes + plan.filter_bytes);
    int32_t* wtap = reinterpret_cast<int32_t*>(ws + plan.col_bytes + plan.filter_bytes + align256(static_cast<size_t>(g.oc) * 4));
    uint8_t* gemm_ws = ws + plan.col_bytes + plan.filter_bytes + plan.sums_bytes;
    const bool comp = needs_compensation(a);

    if (a->weight_packed) {
        wt = static_cast<int8_t*>(const_cast<void*>(a->weight));
        uint8_t* after = reinterpret_cast<uint8_t*>(wt) + align256(static_cast<size_t>(g.oc * g.kp));
        r_w = reinterpret_cast<int32_t*>(after);
        wtap = reinterpret_cast<int32_t*>(after + align256(static_cast<size_t>(g.oc) * 4));
    } else {
        const int st = launch_conv_filter_kmajor(a->weight, a->w_stride_kh, a->w_stride_kw, a->w_stride_ic,
                                                 a->w_stride_oc, g.kh, g.kw, g.icg, g.ocg, g.groups, wt,
                                                 comp ? r_w : nullptr, (implicit && a->zp_x != 0) ? wtap : nullptr, stream);
        if (st != NNB200_OK) {
            return st;
        }
    }
    if (implicit) {
        // One launch per group on the tensor-core engine, the activation read in place.
        const DeviceInfo* dev = current_device_info();
        if (dev == nullptr) {
            return NNB200_INTERNAL;
        }
        if (dev->cc_major != 10) {
            return NNB200_UNSUPPORTED;
        }
        const bool int_out = a->out_kind <= NNB200_OUT_U8;
        const int64_t out_esz = out_elem_bytes(a->out_kind);
        const int64_t bias_esz = a->out_kind == NNB200_OUT_F16 ? 2 : 4;
        BorderParams bp;
        std::memset(&bp, 0, sizeof(bp));
        int32_t* border = reinterpret_cast<int32_t*>(gemm_ws);
        if (a->zp_x != 0) {
            bp.wtap = wtap;
            bp.table = border;
            bp.oc = static_cast<int32_t>(g.oc);
            bp.kh = static_cast<int32_t>(g.kh);
            bp.kw = static_cast<int32_t>(g.kw);
            bp.nh = conv_border_masks(static_cast<int>(g.oh), static_cast<int>(g.ih), bp.kh, static_cast<int>(g.sh),
                                      static_cast<int>(g.dh), static_cast<int>(g.ph), bp.mask_h);
            bp.nw = conv_border_masks(static_cast<int>(g.ow), static_cast<int>(g.iw), bp.kw, static_cast<int>(g.sw),
                                      static_cast<int>(g.dw), static_cast<int>(g.pw), bp.mask_w);
            if (bp.nh < 0 || bp.nw < 0) {
                return NNB200_INTERNAL;   // implicit_form() admits only geometries with at most eight classes
            }
            const int64_t items = static_cast<int64_t>(bp.nh + 1) * (bp.nw + 1) * g.oc;
            conv_border_table_kernel<<<static_cast<unsigned>((items + 255) / 256), 256, 0, stream>>>(bp);
            note_launch();
            if (cudaGetLastError() != cudaSuccess) {
                return NNB200_INTERNAL;
            }
        }
        for (int64_t grp = 0; grp < g.groups; ++grp) {
            const int64_t c0 = grp * g.ocg;
            I8Epilogue ep;
            std::memset(&ep, 0, sizeof(ep));
            ep.out = static_cast<uint8_t*>(a->out) + c0 * out_esz;
            ep.ldc = a->out_stride_w;
            ep.out_kind = a->out_kind;
            ep.bias = a->bias != nullptr ? static_cast<const uint8_t*>(a->bias) + c0 * bias_esz : nullptr;
            ep.relu = int_out ? (a->relu != 0) : 0;
            ep.activation = int_out ? NNB200_ACT_NONE : a->activation;
            ep.act_alpha = a->act_alpha;
            ep.act_beta = a->act_beta;
            ep.min_clip = a->min_clip;
            ep.max_clip = a->max_clip;
            ep.scale_w = a->scale_w != nullptr ? a->scale_w + c0 : nullptr;
            ep.zp_w = nullptr;                       // every weight zero point is 0 in this form
            ep.scale_a_scalar = a->scale_x;
            ep.scale_w_scalar = a->scale_w_scalar;
            ep.zp_a_scalar = a->zp_x;
            ep.zp_w_scalar = 0;
            ep.compensate = a->zp_x != 0 ? 1 : 0;
            ep.r_a = nullptr;
            ep.r_w = a->zp_x != 0 ? r_w + c0 : nullptr;
            ep.k = static_cast<int32_t>(g.k);
            ep.out_scale = a->out_scale;
            ep.out_zp = a->out_zp;
            ConvUmmaArgs c;
            c.x = a->input;
            c.in_n = a->in_stride_n; c.in_h = a->in_stride_h; c.in_w = a->in_stride_w;
            c.batch = static_cast<int32_t>(g.batch); c.ih = static_cast<int32_t>(g.ih); c.iw = static_cast<int32_t>(g.iw);
            c.ic_total = static_cast<int32_t>(g.ic); c.oh = static_cast<int32_t>(g.oh); c.ow = static_cast<int32_t>(g.ow);
            c.kh = static_cast<int32_t>(g.kh); c.kw = static_cast<int32_t>(g.kw);
            c.dh = static_cast<int32_t>(g.dh); c.dw = static_cast<int32_t>(g.dw);
            c.ph = static_cast<int32_t>(g.ph); c.pw = static_cast<int32_t>(g.pw);
            c.sh = static_cast<int32_t>(g.sh); c.sw = static_cast<int32_t>(g.sw);
            c.c_base = static_cast<int32_t>(grp * g.icg); c.icg = static_cast<int32_t>(g.icg);
            c.wt = wt + c0 * g.kp;
            c.ldw = g.kp;
            c.ocg = static_cast<int32_t>(g.ocg); c.k = static_cast<int32_t>(g.k);
            c.zp_x = a->zp_x;
            c.wtap_ld = static_cast<int32_t>(g.oc);
            c.nh = bp.nh;
            c.nw = bp.nw;
            for (int q = 0; q < 8; ++q) {
                c.mask_h[q] = bp.mask_h[q];
                c.mask_w[q] = bp.mask_w[q];
            }
            c.border = a->zp_x != 0 ? border + c0 : nullptr;
            c.a_unsigned = a->a_unsigned;
            const int st = launch_conv_i8_umma(c, ep, *dev, stream);
            if (st != NNB200_OK) {
                return st;
            }
        }
        return NNB200_OK;
    }
    if (!in_place) {
        GatherParams p;
        p.in = static_cast<const uint8_t*>(a->input);
        p.col = col;
        p.in_n = a->in_stride_n; p.in_h = a->in_stride_h; p.in_w = a->in_stride_w; p.in_c = a->in_stride_c;
        p.batch = static_cast<int32_t>(g.batch); p.ih = static_cast<int32_t>(g.ih); p.iw = static_cast<int32_t>(g.iw);
        p.oh = static_cast<int32_t>(g.oh); p.ow = static_cast<int32_t>(g.ow);
        p.kh = static_cast<int32_t>(g.kh); p.kw = static_cast<int32_t>(g.kw);
        p.sh = static_cast<int32_t>(g.sh); p.sw = static_cast<int32_t>(g.sw);
        p.dh = static_cast<int32_t>(g.dh); p.dw = static_cast<int32_t>(g.dw);
        p.ph = static_cast<int32_t>(g.ph); p.pw = static_cast<int32_t>(g.pw);
        p.groups = static_cast<int32_t>(g.groups); p.icg = static_cast<int32_t>(g.icg);
        p.k = static_cast<int32_t>(g.k); p.kp = static_cast<int32_t>(g.kp);
        p.pixels = g.pixels;
        p.pad_byte = static_cast<uint32_t>(a->zp_x) & 0xFFu;
        const bool vec = g.icg % 16 == 0 && a->in_stride_c == 1 && a->in_stride_w % 16 == 0 && a->in_stride_h % 16 == 0 &&
                         a->in_stride_n % 16 == 0 && reinterpret_cast<uintptr_t>(a->input) % 16 == 0;
        const DeviceInfo* dev = current_device_info();
        if (dev == nullptr) {
            return NNB200_INTERNAL;
        }
        // About 2048 pieces (eight per thread) per batch of rows, at most 64 rows.
        const int64_t cpr = g.kp / 16;
        int rows_per_block = static_cast<int>(2048 / cpr);
        rows_per_block = rows_per_block < 1 ? 1 : (rows_per_block > 64 ? 64 : rows_per_block);
        const int64_t rows_total = g.groups * g.pixels;
        int64_t blocks = (rows_total + rows_per_block - 1) / rows_per_block;
        const int64_t cap = static_cast<int64_t>(dev->sm_count) * 8;
        blocks = blocks > cap ? cap : blocks;
        const size_t smem = static_cast<size_t>(rows_per_block) * 16 + static_cast<size_t>(cpr) * 16;
        if (vec) {
            conv_gather_i8_kernel<true><<<static_cast<unsigned>(blocks), 256, smem, stream>>>(p, rows_per_block);
        } else {
            conv_gather_i8_kernel<false><<<static_cast<unsigned>(blocks), 256, smem, stream>>>(p, rows_per_block);
        }
        note_launch();
        const int st = cuda_status(cudaGetLastError());
        if (st != NNB200_OK) {
            return st;
        }
    }
    nnb200_gemm_i8_args q;
    group_gemm_args(a, g, in_place, &q);
    q.workspace = plan.gemm_bytes > 0 ? gemm_ws : nullptr;
    q.workspace_bytes = plan.gemm_bytes;
    const int64_t out_esz = out_elem_bytes(a->out_kind);
    const int64_t bias_esz = a->out_kind == NNB200_OUT_F16 ? 2 : 4;
    for (int64_t grp = 0; grp < g.groups; ++grp) {
        const int64_t c0 = grp * g.ocg;
        q.a = in_place ? static_cast<const uint8_t*>(a->input) + grp * g.icg : col + grp * g.pixels * g.kp;
        q.w = wt + c0 * g.kp;
        q.out = static_cast<uint8_t*>(a->out) + c0 * out_esz;
        q.bias = a->bias != nullptr ? static_cast<const uint8_t*>(a->bias) + c0 * bias_esz : nullptr;
        q.scale_w = a->scale_w != nullptr ? a->scale_w + c0 : nullptr;
        q.zp_w = a->zp_w != nullptr ? a->zp_w + c0 : nullptr;
        q.r_w = comp ? r_w + c0 : nullptr;
        const int st = nnb200_gemm_i8(&q, stream_v);
        if (st != NNB200_OK) {
            return st;
        }
    }
    return NNB200_OK;
}

}  // extern "C"
