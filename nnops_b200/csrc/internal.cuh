// Declarations shared between the translation units of libnnb200: engine launchers, the
// per-device state cache and the TMA descriptor helper.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../../include/nnb200.h"
#include "epilogue.cuh"

namespace nnb200 {

constexpr int kMaxDevices = 64;

// Per-device facts, looked up once per device (never keyed on "the device current at first
// call").
struct DeviceInfo {
    int device = -1;
    int sm_count = 0;
    int cc_major = 0;
    int cc_minor = 0;
    int32_t* error_word = nullptr;  // device address of this device's error word
};

// State of the calling thread's current device; nullptr on a CUDA error.
const DeviceInfo* current_device_info();

// Value of a measurement switch (NNB200_KNOB_*); negative = default.
int knob(int id);

// Sticky "a rank-barrier wait ran out" word of the current device: one int32 in pinned host
// memory that the barrier kernel sets through its device alias and the host reads without
// synchronising.  Created on first use (a set-up step: it allocates pinned memory once per
// device).  Both null on failure.
struct PeerPoison {
    volatile int32_t* host = nullptr;
    int32_t* device = nullptr;
};
PeerPoison peer_poison_for_current_device(bool create);

// Count a kernel launch (nnb200_launch_count).
void note_launch(int n = 1);

// Encode a 2-D row-major byte/half tensor [rows][cols] with row pitch `pitch_bytes` as a TMA
// descriptor with a 128-byte-swizzled box of box_cols x box_rows elements.  elem_bytes is 1
// 2 or 4 (4 = opaque 32-bit words).  swizzle128 = false leaves the box rows dense in shared
// memory.  Returns false if the driver rejects it.
bool make_tma_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t cols, uint64_t rows,
                 uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows, bool swizzle128 = true);

// box_w / box_h count the pixels a box DELIVERS; step_w / step_h (1 or 2) the distance between
// them in the tensor (the map's element strides), so the box spans box * step pixels.
bool make_tma_nhwc_u8(CUtensorMap* map, const void* base, uint64_t c, uint64_t w, uint64_t h, uint64_t n,
                      uint64_t stride_w, uint64_t stride_h, uint64_t stride_n, uint32_t box_c, uint32_t box_w,
                      uint32_t box_h, uint32_t step_w = 1, uint32_t step_h = 1);

// One 2-D int8 problem (a single batch element), Linear pose: A [m,k] and W [n,k] both
// k-contiguous.  lda / ldw are row pitches in bytes.
struct I8Problem {
    const void* a;
    const void* w;
    int64_t m, n, k;
    int64_t a_stride_m, a_stride_k, w_stride_n, w_stride_k;
    int32_t a_unsigned;
};

// True when the tensor-core engine can take the problem: k-contiguous operands whose base
// and row pitch are 16-byte aligned (the TMA rule).
bool umma_i8_supported(const I8Problem& p);

int launch_gemm_i8_umma(const I8Problem& p, const I8Epilogue& ep, const DeviceInfo& dev, cudaStream_t stream);
// One group of an int8 convolution on the tensor-core engine without a gathered copy of the
// activation (stride 1, a multiple of 128 channels per group, symmetric weights): see
// gemm_i8_umma.cu.  Strides in bytes (8-bit elements).
struct ConvUmmaArgs {
    const void* x;              // NHWC activation, all channels
    int64_t in_n, in_h, in_w;
    int32_t batch, ih, iw, ic_total, oh, ow;
    int32_t kh, kw, dh, dw, ph, pw;
    int32_t sh, sw;             // window strides (1 or 2)
    int32_t c_base, icg;        // this group's channels
    const void* wt;             // k-major filter rows of this group [ocg][ldw], k = (tap, channel)
    int64_t ldw;
    int32_t ocg, k;
    int32_t zp_x;
    int32_t wtap_ld;            // output channels of the whole filter: row length of `border`
    // Border classes (zp_x != 0): the distinct masks of out-of-image taps per axis and, per pair
    // of classes, the sum of the filter's per-tap channel sums over the taps the pair loses.
    int32_t nh, nw;
    uint32_t mask_h[8], mask_w[8];
    const int32_t* border;      // [(nh + 1) * (nw + 1)][wtap_ld], at this group's first column
    int32_t a_unsigned;
};
int launch_conv_i8_umma(const ConvUmmaArgs& c, const I8Epilogue& ep, const DeviceInfo& dev, cudaStream_t stream);
// Which taps of one filter axis fall outside the image, as a bit mask, for the output coordinate
// `o`: bit t set when o * stride - pad + t * dil is not in [0, extent_in).
inline uint32_t conv_bad_taps(int o, int stride, int pad, int dil, int taps, int extent_in)
{
    uint32_t bad = 0;
    for (int t = 0; t < taps; ++t) {
        const int i = o * stride - pad + t * dil;
        bad |= (i < 0 || i >= extent_in) ? (1u << t) : 0u;
    }
    return bad;
}
// The distinct non-zero masks over all output coordinates of an axis, into masks[0..7]; returns
// their number, or -1 when there are more than eight.
inline int conv_border_masks(int extent_out, int extent_in, int taps, int stride, int dil, int pad, uint32_t* masks)
{
    int count = 0;
    for (int o = 0; o < extent_out; ++o) {
        const uint32_t bad = conv_bad_taps(o, stride, pad, dil, taps, extent_in);
        if (bad == 0) {
            continue;
        }
        bool seen = false;
        for (int q = 0; q < count; ++q) {
            seen = seen || masks[q] == bad;
        }
        if (!seen) {
            if (count == 8) {
                return -1;
            }
            masks[count++] = bad;
        }
    }
    return count;
}

// The patch of 128 output pixels an M tile of that form covers: (128 >> lg) rows x (1 << lg)
// columns, lg in 3..7, chosen for the fewest padded pixels per image (ties: the wider patch).
// *padded = pixels per image the tiles cover.
inline int conv_patch_log2(int oh, int ow, int64_t* padded)
{
    int best = 3;
    int64_t best_cost = -1;
    for (int lg = 3; lg <= 7; ++lg) {
        const int bw = 1 << lg, bh = 128 >> lg;
        const int64_t cost = static_cast<int64_t>((ow + bw - 1) / bw) * bw * ((oh + bh - 1) / bh) * bh;
        if (best_cost < 0 || cost <= best_cost) {
            best_cost = cost;
            best = lg;
        }
    }
    if (padded != nullptr) {
        *padded = best_cost;
    }
    return best;
}
int launch_gemm_i8_generic(const I8Problem& p, const I8Epilogue& ep, const DeviceInfo& dev, cudaStream_t stream);
int launch_gemm_i8_narrow(const I8Problem& p, const I8Epilogue& ep, const DeviceInfo& dev, cudaStream_t stream);
bool narrow_i8_supported(const I8Problem& p);
int launch_gemm_i8_decode(const I8Problem& p, const I8Epilogue& ep, const DeviceInfo& dev, cudaStream_t stream);
bool decode_i8_supported(const I8Problem& p);
// split_scratch: skinny_i8_split_bytes() bytes for the equal-share split of K over all SMs, or null.
int launch_gemm_i8_skinny(const I8Problem& p, const I8Epilogue& ep, const DeviceInfo& dev, void* split_scratch,
                          cudaStream_t stream);
size_t skinny_i8_split_bytes(const I8Problem& p, const DeviceInfo& dev);
bool skinny_i8_supported(const I8Problem& p);

// R_a[m] = sum_k A[m][k] and R_w[n] = sum_k W[n][k] into int32 scratch; r_w == nullptr skips the
// sweep over W (the caller has the sums already).
int launch_i8_sums(const I8Problem& p, int32_t* r_a, int32_t* r_w, cudaStream_t stream);

int launch_q4_1_gemv(const nnb200_q4_1_args& a, const DeviceInfo& dev, cudaStream_t stream);
int launch_q4_1_gemv_mma(const nnb200_q4_1_args& a, const DeviceInfo& dev, cudaStream_t stream);
bool q4_1_gemv_mma_supported(const nnb200_q4_1_args& a);
int launch_q4_1_gemv_dsq(const nnb200_q4_1_args& a, const DeviceInfo& dev, cudaStream_t stream);
bool q4_1_gemv_dsq_supported(const nnb200_q4_1_args& a);
int launch_q4_1_gemm_umma(const nnb200_q4_1_args& a, const DeviceInfo& dev, cudaStream_t stream);
bool q4_1_gemm_umma_supported(const nnb200_q4_1_args& a);
int launch_q4_1_two_pass(const nnb200_q4_1_args& a, const DeviceInfo& dev, cudaStream_t stream);
bool q4_1_two_pass_supported(const nnb200_q4_1_args& a);
size_t q4_1_two_pass_scratch_bytes(const nnb200_q4_1_args& a);
int launch_q4_1_decode(const void* w_blocks, int64_t ldw_blocks, int64_t rows, int64_t k, void* out, int out_f16,
                       int64_t ld_out, cudaStream_t stream);

int launch_quantize_linear(const nnb200_quant_linear_args& q, const DeviceInfo& dev, cudaStream_t stream);
int launch_dequantize_linear(const nnb200_quant_linear_args& q, const DeviceInfo& dev, cudaStream_t stream);

int launch_mma_i8_peak(int iters, int pattern, double* ops_out, const DeviceInfo& dev, cudaStream_t stream);

int64_t i8_pack_pitch(int64_t k);
int64_t q4_1_pack_qs_pitch(int64_t k);
int64_t q4_1_pack_dm_pitch(int64_t k);
int launch_q4_1_pack(const void* w_blocks, int64_t ldw_blocks, int64_t n, int64_t k, void* blob, cudaStream_t stream);
int launch_i8_pack(const void* w, int64_t n, int64_t k, int64_t stride_n, int64_t stride_k, const float* scale_w,
                   float scale_scalar, const int32_t* zp_w, int32_t zp_scalar, void* blob, cudaStream_t stream);

// Device-side barrier among up to 8 GPUs: flags_by_rank[r] is rank r's flag array (int32[16],
// zeroed once), mapped into this process; limit_cycles <= 0 means the default wait limit.
int launch_rank_barrier(int32_t* const* flags_by_rank, int world, int rank, long long limit_cycles,
                        int32_t* poison, const DeviceInfo& dev, cudaStream_t stream);
int launch_interleave_shards(const void* src, void* dst, int64_t m, int64_t row_bytes_per_shard, int g,
                             int64_t dst_pitch_bytes, const DeviceInfo& dev, cudaStream_t stream);

inline int cuda_status(cudaError_t e)
{
    return e == cudaSuccess ? NNB200_OK : NNB200_INTERNAL;
}

}  // namespace nnb200
