// int8 GEMM for prefill-sized problems on sm_100a: out = epilogue(A[M,K] * W[N,K]^T).
//
// Replaces the reference's mma.sync tile engine (i8_gemm_kernel,
// src/backend/cuda/matmul/matmul_i8_ptx.cu:22-385) with a design native to Blackwell:
//
//   * persistent CTAs (one per SM), each walking 128 x BN output tiles in an L2-friendly
//     grouped order;
//   * warp 0 streams A and W tiles (128 bytes of K per stage) into a shared-memory ring with
//     TMA, 128-byte swizzle, out-of-range rows/columns zero-filled by the hardware;
//   * warp 1 issues tcgen05.mma kind::i8 (M128 x N=BN x K32) into one of two TMEM
//     accumulators and frees ring slots with tcgen05.commit;
//   * warps 2-5 drain the other accumulator with tcgen05.ld and apply the fused epilogue
//     (zero-point compensation, int32 bias, Relu, requantisation / dequantisation) in
//     registers, so the epilogue of tile i overlaps the main loop of tile i+1.
//
// Sharded form (template flag PEERS): the epilogue of an 8-bit destination stages 32 rows x 128
// columns per warp in shared memory (128-byte swizzle) and hands each such tile to TMA, once per
// destination: this GPU's output and the same window of every peer GPU's output (peer memory
// over NVLink).  The all-gather is thereby fused into the GEMM's write-back, tile by tile, as
// asynchronous bulk stores; the epilogue warps only wait for a staging buffer to be read out.
// Loads never touch peer memory.
//
// Both operands are already K-major in memory ([M,K] and [N,K]), which is the layout the
// UMMA shared-memory descriptors want, so no transposes or repacking happen anywhere.
// Every barrier wait is bounded; a wait that runs out records an error code and the CTA
// tears down cleanly.

#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>
#include <type_traits>
#include <mutex>

#include "internal.cuh"
#include "ptx.cuh"
#include "ptx_pair.cuh"

namespace nnb200 {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockKBytes = 128;  // one 128-byte swizzle row of K per stage
constexpr int kUmmaK = 32;         // K per tcgen05.mma for 8-bit operands
// TMA warp, MMA warp, then the epilogue warps: eight (two per TMEM lane quarter, each draining
// half of the tile's columns) in the plain kernels, four in the sharded form, whose staging
// tiles are per warp.  One warp per scheduler issues an instruction every ~4 cycles on the
// epilogue's dependent chains; with four warps a 128 x 256 tile took ~17k cycles to drain, which
// hid behind the main loop only from K = 4096 up.
constexpr int kMaxThreads = 320;
__host__ __device__ constexpr int epilogue_warps(int peers) { return peers ? 4 : 8; }
__host__ __device__ constexpr int num_threads(int peers) { return (2 + epilogue_warps(peers)) * 32; }
// Columns drained by the first of the two warps of a lane quarter (whole 32-column chunks).
__host__ __device__ constexpr int first_half_cols(int bn, int peers) { return peers ? bn : ((bn / 32 + 1) / 2) * 32; }

// TMA descriptors of the output windows the sharded form writes: [0] this GPU's, then the peers'.
struct alignas(64) PeerMaps {
    CUtensorMap m[8];
};

// Geometry of the implicit-GEMM convolution (CONV kernels): an M tile is a patch of bh x bw
// output pixels of one image, its A operand for the k-block (tap, 128 channels) one 4-D TMA
// box of the NHWC activation shifted by the tap -- what lies outside the image is filled with
// zeros, and rows whose window overhangs get the zero point's share added back in the epilogue.
struct ConvTile {
    int32_t oh, ow, ih, iw;
    int32_t kh, kw, dh, dw, ph, pw;
    int32_t sh, sw;                // window strides (1 or 2): the tensor map's element strides along h and w
    int32_t bw_log2, bh;           // patch: bh rows x (1 << bw_log2) columns, 128 pixels
    int32_t tiles_w, tiles_h;      // patches per image
    int32_t c_base;                // first channel of this group in the activation
    int32_t kb_per_tap;            // 128-channel k-blocks per tap
    int32_t zp_x;                  // activation zero point (0: no correction)
    int32_t wtap_ld;               // output channels of the whole filter (row length of the tables)
    // Border classes: the distinct masks of out-of-image taps along each axis (at most eight
    // each); class (i, j) -- i, j = 1 + index of the row's masks, 0 = none -- has a table row
    // holding the sum of the per-tap channel sums of the filter over the taps it loses.
    int32_t nh, nw;
    uint32_t mask_h[8], mask_w[8];
    const int32_t* border;         // [(nh + 1) * (nw + 1)][wtap_ld], at this group's first column
    int32_t m_tiles;               // patches in all (batch * tiles_h * tiles_w)
};

// Patch m_blk = (image, th, tw); a patch index past m_tiles (the second half of an odd pair)
// decodes to an image past the batch: its loads are all fill, its rows are not stored.
struct ConvPatch {
    int img, th, tw;
};

__device__ __forceinline__ ConvPatch conv_patch(const ConvTile& conv, int m_blk)
{
    ConvPatch p;
    p.tw = m_blk % conv.tiles_w;
    const int t2 = m_blk / conv.tiles_w;
    p.th = t2 % conv.tiles_h;
    p.img = t2 / conv.tiles_h;
    return p;
}

// Row r of a patch: its output pixel's flat index, whether it exists, and -- with a non-zero
// activation zero point -- the row's border class along each axis (0: every tap inside).
struct ConvRow {
    int64_t m;
    bool ok;
    uint32_t bad_h, bad_w;
};

__device__ __forceinline__ ConvRow conv_row(const ConvTile& conv, int m_blk, int r)
{
    const ConvPatch p = conv_patch(conv, m_blk);
    const int y = p.th * conv.bh + (r >> conv.bw_log2);
    const int x = (p.tw << conv.bw_log2) + (r & ((1 << conv.bw_log2) - 1));
    ConvRow o;
    o.ok = m_blk < conv.m_tiles && y < conv.oh && x < conv.ow;
    o.m = (static_cast<int64_t>(p.img) * conv.oh + y) * conv.ow + x;
    o.bad_h = 0;
    o.bad_w = 0;
    if (conv.zp_x != 0 && o.ok) {
        uint32_t lost_h = 0, lost_w = 0;
        for (int a = 0; a < conv.kh; ++a) {
            const int iy = y * conv.sh - conv.ph + a * conv.dh;
            lost_h |= (iy < 0 || iy >= conv.ih) ? (1u << a) : 0u;
        }
        for (int b = 0; b < conv.kw; ++b) {
            const int ix = x * conv.sw - conv.pw + b * conv.dw;
            lost_w |= (ix < 0 || ix >= conv.iw) ? (1u << b) : 0u;
        }
        // 1 + index of the mask among the axis's classes (0 = no tap lost).
        for (int q = 0; q < conv.nh; ++q) {
            o.bad_h = (lost_h != 0 && conv.mask_h[q] == lost_h) ? static_cast<uint32_t>(q + 1) : o.bad_h;
        }
        for (int q = 0; q < conv.nw; ++q) {
            o.bad_w = (lost_w != 0 && conv.mask_w[q] == lost_w) ? static_cast<uint32_t>(q + 1) : o.bad_w;
        }
    }
    return o;
}

// A tap outside the image was loaded as 0 where the reference's gather holds the zero point:
// add zp_x * (that tap's channel sum of the filter) back, from the row's class in the table.
__device__ __forceinline__ void conv_border_fix(const ConvTile& conv, uint32_t (&v)[32], uint32_t bad_h, uint32_t bad_w,
                                                int n0, int n_total)
{
    if ((bad_h | bad_w) == 0) {
        return;
    }
    const int32_t* tb = conv.border + static_cast<int64_t>(bad_h * (conv.nw + 1) + bad_w) * conv.wtap_ld + n0;
    if (n0 + 32 <= n_total && (reinterpret_cast<uintptr_t>(tb) & 15u) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const int4 t4 = __ldg(reinterpret_cast<const int4*>(tb + j));
            v[j] += static_cast<uint32_t>(conv.zp_x) * static_cast<uint32_t>(t4.x);
            v[j + 1] += static_cast<uint32_t>(conv.zp_x) * static_cast<uint32_t>(t4.y);
            v[j + 2] += static_cast<uint32_t>(conv.zp_x) * static_cast<uint32_t>(t4.z);
            v[j + 3] += static_cast<uint32_t>(conv.zp_x) * static_cast<uint32_t>(t4.w);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (n0 + j < n_total) {
                v[j] += static_cast<uint32_t>(conv.zp_x) * static_cast<uint32_t>(tb[j]);
            }
        }
    }
}

template <int BN, int PEERS = 0>
struct TileConfig {
    // Tiles wider than 256 columns (single-wave form, see launch_gemm_i8_umma) are issued as two
    // MMAs of BN / 2 columns over one A tile and keep ONE accumulator: a CTA owns exactly one tile.
    static constexpr int kNSplit = BN > 256 ? 2 : 1;
    static constexpr int kMmaN = BN / kNSplit;
    static constexpr int kATileBytes = kBlockM * kBlockKBytes;
    static constexpr int kBTileBytes = BN * kBlockKBytes;
    static constexpr int kStageBytes = kATileBytes + kBTileBytes;
    // Ring depth: as many stages as fit beside the epilogue staging in ~200 KB.
    static constexpr int kStages = PEERS ? ((BN == 256) ? (PEERS == 1 ? 4 : 3) : (BN == 224 ? 4 : 5))
                                   : (BN > 256) ? (BN > 384 ? 2 : 3)
                                                : ((BN > 128) ? 4 : (BN == 128 ? 6 : 8));
    // Two accumulators BN columns apart (one when BN > 256); a power of two of at least that.
    static constexpr int kTmemCols = BN > 128 ? 512 : 2 * BN;
    // Per epilogue warp {scale, bias, r_w, zp_w} of the columns it drains, 4 B each.
    static constexpr int kHalf0 = first_half_cols(BN, PEERS);
    static constexpr int kColParamBytes = epilogue_warps(PEERS) * 4 * kHalf0 * 4;
    static constexpr int kBarrierBytes = (2 * kStages + 4) * 8 + 16;
    // Sharded form (PEERS = 2): two staging tiles of 32 rows x 128 B per epilogue warp, one being
    // filled while the other is being stored.  With few peers (PEERS = 1, used up to three) the
    // stores are not what saturates first and the main loop decides: one staging tile per warp,
    // and the shared memory that frees keeps the ring at four stages.
    // (Rows of 256 bytes per bulk store from a plain 32 x 256 tile were tried: no change on four
    // GPUs at the same ring depth.)
    static constexpr int kStageTiles = PEERS == 2 ? 2 : 1;
    static constexpr int kStageGroupCols = 128;   // columns per staging tile
    static constexpr int kPeerStageBytes = PEERS ? 4 * kStageTiles * 32 * kStageGroupCols : 0;
    static constexpr int kSmemBytes =
        1024 /*alignment slack*/ + kStages * kStageBytes + kPeerStageBytes + kColParamBytes + kBarrierBytes;
};

struct TileCoord {
    int m_blk;
    int n_blk;
};

// Where a tile's walk over the K blocks starts.  Integer accumulation does not depend on the order
// of the K blocks, so each tile may start somewhere else: CTAs that share an operand tile (every
// CTA of a wave when N is one tile wide, as in a convolution's GEMM) then ask the L2 for
// different lines at any one time instead of all for the same ones.  k_rot == 0 keeps 0.
__device__ __forceinline__ int k_rotation(int tile, int k_rot, int num_kb)
{
    return k_rot == 0 ? 0 : static_cast<int>((static_cast<unsigned>(tile) * static_cast<unsigned>(k_rot)) % static_cast<unsigned>(num_kb));
}

// Division of a number below 2^31 by a fixed divisor as a multiply and a shift (the GPU has no
// integer divider: a plain `/` is a chain of some thirty dependent instructions, and the tile
// walk below needs three of them per tile in every role's loop).
struct FastDiv {
    uint32_t mul, shift;
    __device__ __forceinline__ void init(uint32_t d)
    {
        shift = d > 1 ? 32u - static_cast<uint32_t>(__clz(static_cast<int>(d - 1))) : 0u;
        mul = static_cast<uint32_t>(((static_cast<uint64_t>(1) << 32) * ((static_cast<uint64_t>(1) << shift) - d)) / d + 1);
    }
    __device__ __forceinline__ uint32_t div(uint32_t n) const { return (__umulhi(n, mul) + n) >> shift; }
};

// Tiles are walked m-fastest inside groups of `group_m` m-blocks, groups n-fastest: the CTAs of
// one wave then share a band of A (kept in L2 for the whole pass over N) while W streams by once
// per group.  The last group may hold fewer m-blocks.
struct TileWalk {
    int num_m, group_m, group_size, last_gm;
    FastDiv by_group, by_gm, by_last_gm;
    __device__ __forceinline__ TileWalk(int num_m_, int num_n, int group_m_)
    {
        num_m = num_m_;
        group_m = group_m_ < num_m_ ? group_m_ : (num_m_ > 0 ? num_m_ : 1);
        group_size = group_m * num_n;
        const int groups = (num_m + group_m - 1) / group_m;
        last_gm = num_m - (groups - 1) * group_m;
        last_gm = last_gm > 0 ? last_gm : 1;
        by_group.init(static_cast<uint32_t>(group_size > 0 ? group_size : 1));
        by_gm.init(static_cast<uint32_t>(group_m));
        by_last_gm.init(static_cast<uint32_t>(last_gm));
    }
    __device__ __forceinline__ TileCoord operator()(int tile) const
    {
        const int group = static_cast<int>(by_group.div(static_cast<uint32_t>(tile)));
        const int first_m = group * group_m;
        const int in_group = tile - group * group_size;
        const bool last = num_m - first_m < group_m;
        const int gm = last ? last_gm : group_m;
        TileCoord c;
        c.n_blk = static_cast<int>(last ? by_last_gm.div(static_cast<uint32_t>(in_group))
                                        : by_gm.div(static_cast<uint32_t>(in_group)));
        c.m_blk = first_m + in_group - c.n_blk * gm;
        return c;
    }
};

// The per-column terms of the epilogue as one epilogue warp stages them in shared memory.
struct ColTerms {
    float scale;     // s_w[n], or (s_a / s_out) * s_w[n] when the row factor is folded in
    int32_t bias;    // int32 bias (integer destinations) or the fp bias as bits; with fold_comp also -zp_a * R_w[n]
    int32_t rw;      // R_w[n] when compensation is live
    int32_t zpw;     // zp_w[n]
};

// The loads only, so that they can be issued a tile ahead: nothing here depends on a loaded
// value (an f16 bias stays as its 16 bits).  finish_col_terms() does the arithmetic when the
// terms are staged.
template <int KIND>
__device__ __forceinline__ ColTerms load_col_terms(const I8Epilogue& ep, int n, int n_total)
{
    ColTerms c;
    const bool in = n < n_total;
    c.scale = ep.scale_w_scalar;
    if (in && ep.scale_w != nullptr) {
        c.scale = ep.scale_w[n];
    }
    c.bias = 0;
    if (in && ep.bias != nullptr) {
        if constexpr (KIND <= NNB200_OUT_U8) {
            c.bias = static_cast<const int32_t*>(ep.bias)[n];
        } else if constexpr (KIND == NNB200_OUT_F32) {
            c.bias = __float_as_int(static_cast<const float*>(ep.bias)[n]);
        } else {
            c.bias = static_cast<int32_t>(static_cast<const uint16_t*>(ep.bias)[n]);
        }
    }
    c.rw = 0;
    if (in && ep.compensate && ep.r_w != nullptr) {
        c.rw = ep.r_w[n];
    }
    c.zpw = ep.zp_w_scalar;
    if (in && ep.zp_w != nullptr) {
        c.zpw = ep.zp_w[n];
    }
    return c;
}

// fold_scale: the per-tensor row factor s_a / s_out goes into the column scale.
// fold_comp: a per-tensor activation zero point against weights whose zero points are all 0 -- the
// only live compensation term is -zp_a * R_w[n], a column constant, and goes into the bias.
template <int KIND>
__device__ __forceinline__ ColTerms finish_col_terms(const I8Epilogue& ep, ColTerms c, bool fold_scale, float folded_row_k,
                                                     bool fold_comp)
{
    if (fold_scale) {
        c.scale = __fmul_rn(folded_row_k, c.scale);
    }
    if constexpr (KIND == NNB200_OUT_F16) {
        c.bias = __float_as_int(__half2float(__ushort_as_half(static_cast<unsigned short>(c.bias))));
    }
    if (fold_comp) {
        c.bias = static_cast<int32_t>(static_cast<uint32_t>(c.bias) -
                                      static_cast<uint32_t>(ep.zp_a_scalar) * static_cast<uint32_t>(c.rw));
    }
    return c;
}

// Four requantised 8-bit values in one word, first value in the low byte.  Same bytes as four
// i8_requant() calls, with fewer instructions: that routine clamps x = float(v) * req to
// [lo - zp, hi - zp], rounds half away from zero as trunc(x + copysign(0.5, x)) and adds zp;
// the bounds are integers, so clamping before the rounding or saturating after it (and after
// the zero-point add) gives the same value.  Here the 8-bit saturation rides the packing
// instruction; with a non-zero zero point x is first kept inside +-32000 so that the add cannot
// overflow, with ZP0 (out_zp == 0, the usual s8 destination) not even that is needed.
template <bool U8, bool ZP0>
__device__ __forceinline__ uint32_t requant_pack4(const int32_t (&v)[4], const float (&req)[4], int32_t zp)
{
    int32_t r[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        float x = __fmul_rn(__int2float_rn(v[b]), req[b]);
        if constexpr (ZP0) {
            // The conversion itself saturates at the int32 range; nothing is added afterwards.
            r[b] = __float2int_rz(__fadd_rn(x, copysignf(0.5f, x)));
        } else {
            x = fminf(fmaxf(x, -32000.0f), 32000.0f);
            r[b] = __float2int_rz(__fadd_rn(x, copysignf(0.5f, x))) + zp;
        }
    }
    uint32_t hi, out;
    if constexpr (U8) {
        asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(r[3]), "r"(r[2]), "r"(0));
        asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(r[1]), "r"(r[0]), "r"(hi));
    } else {
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(r[3]), "r"(r[2]), "r"(0));
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(r[1]), "r"(r[0]), "r"(hi));
    }
    return out;
}

// Epilogue of one 32-column chunk of one row.  `acc` holds the raw int32 sums of columns
// n0..n0+31; col_* point at the chunk's staged per-column terms in shared memory.
template <int KIND>
__device__ __forceinline__ void epilogue_chunk(const I8Epilogue& e, const I8RowTerms& t, const uint32_t (&acc)[32],
                                               int64_t m, bool row_ok, int n0, int n_total,
                                               const float* col_scale, const int32_t* col_bias,
                                               const int32_t* col_rw, const int32_t* col_zpw, int vec,
                                               bool scale_folded = false, bool plain = false)
{
    // plain: no per-element compensation terms are needed -- either every zero point is 0, or
    // the only live term (-zp_a * R_w[n], a per-tensor activation zero point against symmetric
    // weights) was folded into the staged column bias.
    // vec: bit 0 = the destination takes 16-byte stores, bit 1 = 32-byte stores as well.
    const bool vec_ok = (vec & 1) != 0;
    const bool vec32 = (vec & 2) != 0;
    const bool full = n0 + 32 <= n_total;
    const float zpf = static_cast<float>(e.out_zp);

    if constexpr (KIND == NNB200_OUT_S32) {
        int32_t o[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            o[j] = i8_int_value(e, t, static_cast<int32_t>(acc[j]), col_zpw[j], col_rw[j], col_bias[j]);
        }
        if (!row_ok) {
            return;
        }
        int32_t* dst = static_cast<int32_t*>(e.out) + m * e.ldc + n0;
        if (full && vec32) {
            // The lane's 128 bytes as four 256-bit stores (whole 32-byte sectors).
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                st_global_32(dst + j, static_cast<uint32_t>(o[j]), static_cast<uint32_t>(o[j + 1]), static_cast<uint32_t>(o[j + 2]),
                             static_cast<uint32_t>(o[j + 3]), static_cast<uint32_t>(o[j + 4]), static_cast<uint32_t>(o[j + 5]),
                             static_cast<uint32_t>(o[j + 6]), static_cast<uint32_t>(o[j + 7]));
            }
        } else if (full && vec_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                *reinterpret_cast<int4*>(dst + j) = make_int4(o[j], o[j + 1], o[j + 2], o[j + 3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (n0 + j < n_total) {
                    dst[j] = o[j];
                }
            }
        }
    } else if constexpr (KIND == NNB200_OUT_S8 || KIND == NNB200_OUT_U8) {
        const float lo = (KIND == NNB200_OUT_S8 ? -128.0f : 0.0f) - zpf;
        const float hi = (KIND == NNB200_OUT_S8 ? 127.0f : 255.0f) - zpf;
        uint32_t packed[8];
        if (!e.compensate || plain) {
            // Common case: with a per-tensor activation scale the staged column scales already
            // carry (s_a / s_out) * s_w[n].  The column terms are read four at a time.
            (void)lo;
            (void)hi;
            // Branch-free per element: the run-time switches become operands (a lower bound for
            // the ReLU, a row factor of exactly 1 when the scale is already folded -- x * 1.0f is
            // x), and the zero-point variant is chosen once per chunk.
            const int32_t relu_lo = e.relu ? 0 : INT32_MIN;
            const float row_k = scale_folded ? 1.0f : t.row_k;
            const auto body = [&](auto zp0_tag) {
                constexpr bool kZp0 = decltype(zp0_tag)::value;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const int4 b4 = *reinterpret_cast<const int4*>(col_bias + j);
                    const float4 s4 = *reinterpret_cast<const float4*>(col_scale + j);
                    const int32_t bias4[4] = {b4.x, b4.y, b4.z, b4.w};
                    const float scale4[4] = {s4.x, s4.y, s4.z, s4.w};
                    int32_t v[4];
                    float req[4];
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        v[b] = max(static_cast<int32_t>(static_cast<uint32_t>(acc[j + b]) + static_cast<uint32_t>(bias4[b])),
                                   relu_lo);
                        req[b] = __fmul_rn(row_k, scale4[b]);
                    }
                    packed[j / 4] = requant_pack4<KIND == NNB200_OUT_U8, kZp0>(v, req, e.out_zp);
                }
            };
            if (e.out_zp == 0) {
                body(std::true_type{});
            } else {
                body(std::false_type{});
            }
        } else {
            // Compensation live (zero points on both sides, or per-row ones): the integer terms, then
            // the same packed requantisation, one loop for every zero point (more code here slows
            // the common path above measurably).
            (void)lo;
            (void)hi;
            const int32_t relu_lo = e.relu ? 0 : INT32_MIN;
            const float row_k = scale_folded ? 1.0f : t.row_k;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                int32_t v[4];
                float req[4];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const int32_t c = i8_compensate(static_cast<int32_t>(acc[j + b]), t.zpa, col_zpw[j + b], t.ra,
                                                    col_rw[j + b], e.k);
                    v[b] = max(static_cast<int32_t>(static_cast<uint32_t>(c) + static_cast<uint32_t>(col_bias[j + b])),
                               relu_lo);
                    req[b] = __fmul_rn(row_k, col_scale[j + b]);
                }
                packed[j / 4] = requant_pack4<KIND == NNB200_OUT_U8, false>(v, req, e.out_zp);
            }
        }
        if (!row_ok) {
            return;
        }
        uint8_t* dst = static_cast<uint8_t*>(e.out) + m * e.ldc + n0;
        if (full && vec32) {
            // The lane's 32 values are exactly one 32-byte sector of its row.
            st_global_32(dst, packed[0], packed[1], packed[2], packed[3], packed[4], packed[5], packed[6], packed[7]);
            // Two-rank shards: the same sector into the other rank's copy, over the link (the
            // launcher has checked that every chunk is full and every pointer 32-byte aligned).
            for (int d = 0; d < e.direct_peers; ++d) {
                st_global_32(static_cast<uint8_t*>(e.peer_out[d]) + m * e.ldc + n0, packed[0], packed[1], packed[2],
                             packed[3], packed[4], packed[5], packed[6], packed[7]);
            }
        } else if (full && vec_ok) {
            *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            *reinterpret_cast<uint4*>(dst + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (n0 + j < n_total) {
                    dst[j] = static_cast<uint8_t>(packed[j / 4] >> (8 * (j % 4)));
                }
            }
        }
    } else {  // F32 / F16
        // One loop per (compensation live?, activation class): the run-time switches are taken
        // once per chunk, not once per element.  With a per-tensor activation scale the staged
        // column scale already carries s_a * s_w[n] (row factor exactly 1: x * 1.0f is x).
        const float row_s = scale_folded ? 1.0f : t.s_a;
        float o[32];
        const auto body = [&](auto comp_tag, auto act_tag) {
            constexpr bool kComp = decltype(comp_tag)::value;
            constexpr int kAct = decltype(act_tag)::value;   // 0 none, 1 Relu, 2 any other, 3 Gelu
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                const int4 b4 = *reinterpret_cast<const int4*>(col_bias + j);
                const float4 s4 = *reinterpret_cast<const float4*>(col_scale + j);
                const float bias4[4] = {__int_as_float(b4.x), __int_as_float(b4.y), __int_as_float(b4.z), __int_as_float(b4.w)};
                const float scale4[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    int32_t v = static_cast<int32_t>(acc[j + b]);
                    if constexpr (kComp) {
                        v = i8_compensate(v, t.zpa, col_zpw[j + b], t.ra, col_rw[j + b], e.k);
                    }
                    float f = __fmul_rn(__int2float_rn(v), __fmul_rn(row_s, scale4[b]));
                    const float fb = __fadd_rn(f, bias4[b]);
                    f = bias4[b] != 0.0f ? fb : f;   // a zero bias is not added (-0 stays -0)
                    f = fminf(fmaxf(f, e.min_clip), e.max_clip);
                    if constexpr (kAct == 1) {
                        f = fmaxf(f, 0.0f);
                    } else if constexpr (kAct == 2) {
                        f = act_apply(e.activation, e.act_alpha, e.act_beta, f);
                    } else if constexpr (kAct == 3) {
                        f = act_apply(NNB200_ACT_GELU, e.act_alpha, e.act_beta, f);   // the switch folds away
                    }
                    o[j + b] = f;
                }
            }
        };
        // Gelu (the usual partner of a Linear) gets a loop of its own; the remaining activations
        // share one with the switch inside.
        const int act_class = e.activation == NNB200_ACT_NONE ? 0
                              : e.activation == NNB200_ACT_RELU ? 1
                              : e.activation == NNB200_ACT_GELU ? 3 : 2;
        if (e.compensate) {
            if (act_class == 0) {
                body(std::true_type{}, std::integral_constant<int, 0>{});
            } else if (act_class == 1) {
                body(std::true_type{}, std::integral_constant<int, 1>{});
            } else {
                body(std::true_type{}, std::integral_constant<int, 2>{});
            }
        } else {
            if (act_class == 0) {
                body(std::false_type{}, std::integral_constant<int, 0>{});
            } else if (act_class == 1) {
                body(std::false_type{}, std::integral_constant<int, 1>{});
            } else if (act_class == 3) {
                body(std::false_type{}, std::integral_constant<int, 3>{});
            } else {
                body(std::false_type{}, std::integral_constant<int, 2>{});
            }
        }
        if (!row_ok) {
            return;
        }
        if constexpr (KIND == NNB200_OUT_F32) {
            float* dst = static_cast<float*>(e.out) + m * e.ldc + n0;
            if (full && vec32) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    st_global_32(dst + j, __float_as_uint(o[j]), __float_as_uint(o[j + 1]), __float_as_uint(o[j + 2]),
                                 __float_as_uint(o[j + 3]), __float_as_uint(o[j + 4]), __float_as_uint(o[j + 5]),
                                 __float_as_uint(o[j + 6]), __float_as_uint(o[j + 7]));
                }
            } else if (full && vec_ok) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    *reinterpret_cast<float4*>(dst + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if (n0 + j < n_total) {
                        dst[j] = o[j];
                    }
                }
            }
        } else {
            uint32_t packed[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                packed[j / 2] = static_cast<uint32_t>(__half_as_ushort(__float2half_rn(o[j]))) |
                                (static_cast<uint32_t>(__half_as_ushort(__float2half_rn(o[j + 1]))) << 16);
            }
            uint16_t* dst = static_cast<uint16_t*>(e.out) + m * e.ldc + n0;
            if (full && vec32) {
                st_global_32(dst, packed[0], packed[1], packed[2], packed[3], packed[4], packed[5], packed[6], packed[7]);
                st_global_32(dst + 16, packed[8], packed[9], packed[10], packed[11], packed[12], packed[13], packed[14],
                             packed[15]);
            } else if (full && vec_ok) {
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                    *reinterpret_cast<uint4*>(dst + 2 * j) =
                        make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if (n0 + j < n_total) {
                        dst[j] = static_cast<uint16_t>(packed[j / 2] >> (16 * (j % 2)));
                    }
                }
            }
        }
    }
}

template <int BN, int KIND, int PEERS, bool CONV = false>
__global__ void __launch_bounds__(kMaxThreads, 1)
gemm_i8_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ PeerMaps peer_maps, const I8Epilogue ep, const int m_total,
                    const int n_total, const int k_total, const uint32_t idesc, const int vec_ok, const int group_m, const int k_rot,
                    int32_t* error_word, const ConvTile conv)
{
    static_assert(!CONV || PEERS == 0, "the convolution form has no sharded epilogue");
    using Cfg = TileConfig<BN, PEERS>;
    constexpr int kStages = Cfg::kStages;

    extern __shared__ uint8_t smem_raw[];
    // The swizzled tiles must start on a 1024-byte boundary.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stage_base = smem;
    // Per-column epilogue terms, one private copy per epilogue warp (no cross-warp barrier).
    uint8_t* peer_stage = smem + kStages * Cfg::kStageBytes;  // 1024-byte aligned (PEERS only)
    int32_t* col_params = reinterpret_cast<int32_t*>(peer_stage + Cfg::kPeerStageBytes);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(col_params + Cfg::kColParamBytes / 4);
    uint64_t* empty_bar = full_bar + kStages;
    uint64_t* acc_full_bar = empty_bar + kStages;
    uint64_t* acc_empty_bar = acc_full_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // Operand poses ride in bits 4-5 of vec_ok: bit 4 = A stored [K][M], bit 5 = W stored [K][N]
    // (MN-major operands: the tensor maps, the descriptors and the K step change, nothing else).
    const int pose = (vec_ok >> 4) & 3;

    const int num_m = (m_total + kBlockM - 1) / kBlockM;
    const int num_n = (n_total + BN - 1) / BN;
    const int num_tiles = num_m * num_n;
    const int num_kb = (k_total + kBlockKBytes - 1) / kBlockKBytes;
    const TileWalk walk(num_m, num_n, group_m);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full_bar[a], 1);
            mbar_init(&acc_empty_bar[a], epilogue_warps(PEERS));
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_w);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t armed = 0;        // bit s: slot s has been armed at least once
            uint32_t armed_phase = 0;  // bit s: parity of the phase slot s was last armed in
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                const TileCoord tc = walk(tile);
                const int rot = k_rotation(tile, k_rot, num_kb);
                for (int step = 0; step < num_kb; ++step) {
                    const int kb = step + rot < num_kb ? step + rot : step + rot - num_kb;
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
                        atomicCAS(error_word, 0, kErrProducerWait);
                        ok = false;
                        break;
                    }
                    uint8_t* a_dst = stage_base + stage * Cfg::kStageBytes;
                    uint8_t* b_dst = a_dst + Cfg::kATileBytes;
                    mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
                    if constexpr (CONV) {
                        // Patch (image, th, tw) shifted by the k-block's tap; 128 channels of it.
                        const ConvPatch pt = conv_patch(conv, tc.m_blk);
                        const int tap = kb / conv.kb_per_tap;
                        const int c0 = (kb - tap * conv.kb_per_tap) * kBlockKBytes;
                        const int ta = tap / conv.kw;
                        const int tb = tap - ta * conv.kw;
                        tma_load_4d(a_dst, &map_a, &full_bar[stage], conv.c_base + c0,
                                    (pt.tw << conv.bw_log2) * conv.sw - conv.pw + tb * conv.dw,
                                    pt.th * conv.bh * conv.sh - conv.ph + ta * conv.dh, pt.img);
                    } else if (pose & 1) {
                        // A stored [K][M]: the box is 128 k-rows of 128 m-bytes.
                        tma_load_2d(a_dst, &map_a, &full_bar[stage], tc.m_blk * kBlockM, kb * kBlockKBytes);
                    } else {
                        tma_load_2d(a_dst, &map_a, &full_bar[stage], kb * kBlockKBytes, tc.m_blk * kBlockM);
                    }
                    if (pose & 2) {
                        // W stored [K][N]: one box of 128 k-rows x 128 n-bytes per 128 columns of the tile.
#pragma unroll
                        for (int blk = 0; blk < BN / 128; ++blk) {
                            tma_load_2d(b_dst + blk * (128 * kBlockKBytes), &map_w, &full_bar[stage],
                                        tc.n_blk * BN + blk * 128, kb * kBlockKBytes);
                        }
                    } else {
#pragma unroll
                        for (int h = 0; h < Cfg::kNSplit; ++h) {  // TMA boxes hold at most 256 rows
                            tma_load_2d(b_dst + h * Cfg::kMmaN * kBlockKBytes, &map_w, &full_bar[stage], kb * kBlockKBytes,
                                        tc.n_blk * BN + h * Cfg::kMmaN);
                        }
                    }
                    armed |= 1u << stage;
                    armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                // Copies already issued still land in shared memory: wait (bounded) for the
                // armed slots so the CTA does not exit underneath them.
                const long long t0 = clock64();
                for (int s = 0; s < kStages; ++s) {
                    if ((armed >> s) & 1u) {
                        // The full barrier of the phase this slot was last armed in completes
                        // when its bytes have landed.
                        while (!mbar_try_wait(&full_bar[s], (armed_phase >> s) & 1u)) {
                            if (clock64() - t0 > kWaitLimitCycles) {
                                atomicCAS(error_word, 0, kErrDrainWait);
                                break;
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int local_tile = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local_tile) {
                const int acc = Cfg::kNSplit > 1 ? 0 : (local_tile & 1);
                const uint32_t acc_phase = Cfg::kNSplit > 1 ? (local_tile & 1u) : ((local_tile >> 1) & 1u);
                if (!mbar_wait(&acc_empty_bar[acc], acc_phase ^ 1u, abort_flag)) {
                    atomicCAS(error_word, 0, kErrAccumWait);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
                        atomicCAS(error_word, 0, kErrMmaWait);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(stage_base + stage * Cfg::kStageBytes);
                    const uint32_t b_addr = a_addr + Cfg::kATileBytes;
                    // K-major tiles step 32 bytes along their 128-byte rows per MMA (+2 in the
                    // descriptor's 16-byte units); MN-major tiles step 32 k-rows of 128 bytes (+256).
                    const uint64_t a_desc = (pose & 1) ? umma_desc_sw128_mnmajor(a_addr, 128 * kBlockKBytes)
                                                       : umma_desc_sw128_kmajor(a_addr);
                    const uint64_t b_desc = (pose & 2) ? umma_desc_sw128_mnmajor(b_addr, 128 * kBlockKBytes)
                                                       : umma_desc_sw128_kmajor(b_addr);
                    const uint64_t a_step = (pose & 1) ? 256u : 2u;
                    const uint64_t b_step = (pose & 2) ? 256u : 2u;
#pragma unroll
                    for (int ks = 0; ks < kBlockKBytes / kUmmaK; ++ks) {
#pragma unroll
                        for (int h = 0; h < Cfg::kNSplit; ++h) {
                            // Second half of a wide tile: kMmaN rows further down the W tile (16-byte
                            // descriptor units), kMmaN columns further along the accumulator.
                            umma_i8(d_tmem + static_cast<uint32_t>(h * Cfg::kMmaN),
                                    a_desc + static_cast<uint64_t>(ks) * a_step,
                                    b_desc + static_cast<uint64_t>(ks) * b_step +
                                        static_cast<uint64_t>(h * (Cfg::kMmaN * kBlockKBytes / 16)),
                                    idesc, (kb > 0 || ks > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(&empty_bar[stage]);  // slot is free once these MMAs have read it
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) {
                    umma_commit(&acc_full_bar[acc]);  // accumulator complete
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue warps ----------------
        const int quarter = warp & 3;  // the TMEM lane quarter this warp may read
        // 8-bit destinations with a per-tensor activation scale: the row factor s_a / s_out is the
        // same for every row, so it is folded into the staged column scales (same two roundings,
        // once per column instead of once per element).  The sharded form keeps the plain scales.
        // fp destinations: the row factor is s_a itself.
        const bool fold_scale = !PEERS && KIND != NNB200_OUT_S32 && ep.scale_a == nullptr;
        const float folded_row_k = (KIND == NNB200_OUT_S8 || KIND == NNB200_OUT_U8)
                                       ? __fdiv_rn(ep.scale_a_scalar, ep.out_scale) : ep.scale_a_scalar;
        const bool fold_comp = !PEERS && (KIND == NNB200_OUT_S8 || KIND == NNB200_OUT_U8) && ep.compensate != 0 &&
                               ep.zp_a == nullptr && ep.r_a == nullptr;
        // The next tile's column terms are loaded into registers before this tile is drained,
        // so their latency is not paid between tiles (up to four per lane and term).
        constexpr int kTermIters = (Cfg::kHalf0 + 31) / 32;
        constexpr bool kPrefetch = !PEERS && kTermIters <= 4;
        ColTerms next_terms[kPrefetch ? kTermIters : 1];
        // Two warps per lane quarter: the first drains columns [0, kHalf0), the second the rest.
        constexpr int kHalf0 = Cfg::kHalf0;
        const int half = PEERS ? 0 : ((warp - 2) >> 2);
        const int col0 = half * kHalf0;
        const int ncols = half ? BN - kHalf0 : kHalf0;
        float* cs = reinterpret_cast<float*>(col_params + (warp - 2) * 4 * kHalf0);
        int32_t* cb = reinterpret_cast<int32_t*>(cs) + kHalf0;
        int32_t* cr = cb + kHalf0;
        int32_t* cz = cr + kHalf0;
        int stage_turn = 0;  // sharded form: which of the warp's two staging tiles is next
        (void)stage_turn;
        int local_tile = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local_tile) {
            const TileCoord tc = walk(tile);
            const int acc = Cfg::kNSplit > 1 ? 0 : (local_tile & 1);
            const uint32_t acc_phase = Cfg::kNSplit > 1 ? (local_tile & 1u) : ((local_tile >> 1) & 1u);
            const int n_base = tc.n_blk * BN + col0;   // first column this warp drains

            // This tile's per-column terms: fetched while the previous tile was being drained
            // (kPrefetch), or now, hidden behind the tile's main loop.
            __syncwarp();  // previous tile's reads of the staging are done
#pragma unroll
            for (int i = 0; i < kTermIters; ++i) {
                const int j = lane + i * 32;
                if (j < ncols) {
                    const ColTerms ct = finish_col_terms<KIND>(
                        ep, (kPrefetch && local_tile > 0) ? next_terms[kPrefetch ? i : 0] : load_col_terms<KIND>(ep, n_base + j, n_total),
                        fold_scale, folded_row_k, fold_comp);
                    cs[j] = ct.scale;
                    cb[j] = ct.bias;
                    cr[j] = ct.rw;
                    cz[j] = ct.zpw;
                }
            }
            __syncwarp();

            int64_t m = static_cast<int64_t>(tc.m_blk) * kBlockM + quarter * 32 + lane;
            bool row_ok = m < m_total;
            uint32_t bad_h = 0, bad_w = 0;   // CONV: the row's border class along each axis (0: every tap inside)
            if constexpr (CONV) {
                const ConvRow cr_ = conv_row(conv, tc.m_blk, quarter * 32 + lane);
                m = cr_.m;
                row_ok = cr_.ok;
                bad_h = cr_.bad_h;
                bad_w = cr_.bad_w;
            }
            I8RowTerms rt;
            rt.zpa = 0;
            rt.ra = 0;
            rt.s_a = 1.0f;
            rt.row_k = 1.0f;
            if (row_ok) {
                rt = i8_row_terms(ep, m);
            }

            // Warp-uniform outcome, so no lane is left behind at a later warp sync.
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(&acc_full_bar[acc], acc_phase, abort_flag))) {
                atomicCAS(error_word, 0, kErrEpilogueWait);
                break;
            }
            tc_fence_after_sync();

            if constexpr (kPrefetch) {
                const int next = tile + static_cast<int>(gridDim.x);
                if (next < num_tiles) {
                    const int next_base = walk(next).n_blk * BN + col0;
#pragma unroll
                    for (int i = 0; i < kTermIters; ++i) {
                        next_terms[i] = load_col_terms<KIND>(ep, next_base + lane + i * 32, n_total);
                    }
                }
            }

            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(acc * BN + col0);
            if constexpr (PEERS && (KIND == NNB200_OUT_S8 || KIND == NNB200_OUT_U8)) {
                // Sharded write-back: 128 columns at a time through a per-warp staging tile.
                const float zpf = static_cast<float>(ep.out_zp);
                const float lo = (KIND == NNB200_OUT_S8 ? -128.0f : 0.0f) - zpf;
                const float hi = (KIND == NNB200_OUT_S8 ? 127.0f : 255.0f) - zpf;
                (void)lo;
                (void)hi;
                const int row0 = tc.m_blk * kBlockM + quarter * 32;
                const int num_dst = 1 + ep.num_peers;
                const bool multicast = ep.mc_out != nullptr;
                constexpr int kGroupCols = Cfg::kStageGroupCols;       // 128 (swizzled tile) or 256 (plain tile)
                constexpr int kGroupChunks = kGroupCols / 32;
#pragma unroll 1
                for (int c4 = 0; c4 < (BN + kGroupCols - 1) / kGroupCols; ++c4) {
                    const int n128 = n_base + c4 * kGroupCols;
                    if (n128 >= n_total) {
                        break;  // uniform across the warp
                    }
                    // Two staging tiles per warp, used alternately: before refilling one, its
                    // previous bulk stores must have finished READING it (they may still be in flight
                    // on the wire).  Only lane 0 issues bulk stores, so only lane 0 has groups to wait on.
                    uint8_t* stage = peer_stage + ((warp - 2) * Cfg::kStageTiles + (stage_turn % Cfg::kStageTiles)) *
                                                      (32 * kGroupCols);
                    ++stage_turn;
                    if (lane == 0) {
                        bulk_wait_group_read<Cfg::kStageTiles - 1>();
                    }
                    __syncwarp();
#pragma unroll 1
                    for (int cc = 0; cc < kGroupChunks; ++cc) {
                        const int c = c4 * kGroupChunks + cc;
                        if (c >= BN / 32) {
                            break;  // a 224-wide tile ends inside its second 128-column group
                        }
                        uint32_t v[32];
                        tmem_ld_32x32(t_row + static_cast<uint32_t>(c * 32), v);
                        tmem_ld_wait();
                        // No branch per element: the ReLU is a lower bound, compensation is chosen
                        // once per chunk, saturation rides the packing instruction.
                        uint32_t packed[8];
                        const int32_t relu_lo = ep.relu ? 0 : INT32_MIN;
                        if (ep.compensate) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                int32_t vv[4];
                                float rq[4];
#pragma unroll
                                for (int b = 0; b < 4; ++b) {
                                    const int col = c * 32 + j + b;
                                    const int32_t x = i8_compensate(static_cast<int32_t>(v[j + b]), rt.zpa, cz[col], rt.ra,
                                                                    cr[col], ep.k);
                                    vv[b] = max(static_cast<int32_t>(static_cast<uint32_t>(x) + static_cast<uint32_t>(cb[col])),
                                                relu_lo);
                                    rq[b] = __fmul_rn(rt.row_k, cs[col]);
                                }
                                packed[j / 4] = requant_pack4<KIND == NNB200_OUT_U8, false>(vv, rq, ep.out_zp);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                int32_t vv[4];
                                float rq[4];
#pragma unroll
                                for (int b = 0; b < 4; ++b) {
                                    const int col = c * 32 + j + b;
                                    vv[b] = max(static_cast<int32_t>(v[j + b] + static_cast<uint32_t>(cb[col])), relu_lo);
                                    rq[b] = __fmul_rn(rt.row_k, cs[col]);
                                }
                                packed[j / 4] = requant_pack4<KIND == NNB200_OUT_U8, false>(vv, rq, ep.out_zp);
                            }
                        }
                        // This lane's row of the tile: 16-byte pieces 2cc and 2cc+1 (swizzled in the 128-byte form).
                        uint4* srow = reinterpret_cast<uint4*>(stage + lane * kGroupCols);
                        const int sw = lane & 7;
                        srow[(2 * cc) ^ sw] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        srow[(2 * cc + 1) ^ sw] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    }
                    if (multicast) {
                        // One store per tile for all ranks: the staged rows go out as 16-byte
                        // multimem stores, eight lanes covering one 128-byte row, four rows per
                        // pass, and the switch replicates them into every rank's copy.
                        __syncwarp();
                        const int piece = lane & 7;
                        const int cols_here = min(min(128, BN - c4 * 128), n_total - n128);
#pragma unroll 1
                        for (int pass = 0; pass < 8; ++pass) {
                            const int r = pass * 4 + (lane >> 3);
                            const int64_t grow = static_cast<int64_t>(row0) + r;
                            if (grow < m_total && piece * 16 < cols_here) {
                                const uint4 q = *reinterpret_cast<const uint4*>(stage + r * 128 + ((piece ^ (r & 7)) * 16));
                                multimem_st_16(static_cast<uint8_t*>(ep.mc_out) + grow * ep.ldc + n128 + piece * 16, q);
                            }
                        }
                        __syncwarp();  // the staging tile may be refilled
                        continue;
                    }
                    fence_proxy_async_smem();  // generic-proxy writes -> visible to the TMA engine
                    __syncwarp();
                    if (lane == 0) {
                        // One bulk store per destination; rows past M and columns past N are clipped
                        // by the descriptor.
                        for (int d = 0; d < num_dst; ++d) {
                            tma_store_2d(&peer_maps.m[d], stage, n128, row0);
                        }
                        bulk_commit_group();
                    }
                }
            } else {
                // Chunks of 32 columns, two register sets: the load of the next chunk is in flight
                // while this one is requantised and stored.
                const int left = n_total - n_base;   // columns of the matrix from this warp's first one
                const int nch = left <= 0 ? 0 : min(ncols / 32, (left + 31) / 32);   // uniform across the warp
                const auto finish = [&](int c, uint32_t (&v)[32]) {
                    const int n0 = n_base + c * 32;
                    if constexpr (CONV) {
                        conv_border_fix(conv, v, bad_h, bad_w, n0, n_total);
                    }
                    epilogue_chunk<KIND>(ep, rt, v, m, row_ok, n0, n_total, cs + c * 32, cb + c * 32, cr + c * 32,
                                         cz + c * 32, vec_ok, fold_scale, fold_comp);
                };
                uint32_t va[32], vb[32];
                if (nch > 0) {
                    tmem_ld_32x32(t_row, va);
                }
#pragma unroll 1
                for (int c = 0; c < nch; c += 2) {
                    tmem_ld_wait();
                    if (c + 1 < nch) {
                        tmem_ld_32x32(t_row + static_cast<uint32_t>((c + 1) * 32), vb);
                    }
                    finish(c, va);
                    if (c + 1 < nch) {
                        tmem_ld_wait();
                        if (c + 2 < nch) {
                            tmem_ld_32x32(t_row + static_cast<uint32_t>((c + 2) * 32), va);
                        }
                        finish(c + 1, vb);
                    }
                }
            }
            // Accumulator drained: hand it back to the MMA warp.
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&acc_empty_bar[acc]);
            }
        }
        if (!PEERS && ep.direct_peers > 0) {
            __threadfence_system();  // this warp's stores into the peer's copy are performed before the kernel completes
        }
        if constexpr (PEERS) {
            if (ep.mc_out != nullptr) {
                __threadfence_system();  // this warp's multicast stores are performed before the kernel completes
            }
            if (lane == 0) {
                bulk_wait_group<0>();  // every bulk store of this warp has completed before the CTA exits
            }
            __syncwarp();
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}


// ---- CTA-pair form ---------------------------------------------------------------------------
// Two CTAs (a cluster of two, on neighbouring SMs) share one 256 x BN output tile: each loads its
// own 128 rows of A and HALF of the tile's W rows, the pair leader issues tcgen05.mma with
// cta_group::2 (M = 256 over both SMs' tensor cores and TMEM), and each CTA drains its own 128
// accumulator rows through the same epilogue.  Per multiply-add the pair moves two thirds of the
// operand bytes through L2 and shared memory, which under the power cap is worth clock.
//
// What the form lives or dies by is how often the tensor pipe is interrupted: every commit is a
// point the pipe drains to, and every barrier wait a round trip for the issuing thread.  With one
// 128-byte k-block per barrier slot (4 MMAs between commits, one commit per destination CTA) the
// pipe was busy 75 % of the cycles and the form LOST to the single-CTA kernel; with two k-blocks
// per slot (SUB = 2: 8 MMAs between commits) and one commit instruction that arrives on both
// CTAs' barriers (MC) it is busy about 89 % and wins by 8-9 %.  Three k-blocks per slot leave a
// ring of two slots, too coarse to hide the loads, and lose again.
//
// Signalling: TMA loads of both CTAs report their bytes to the LEADER's full barrier; the
// leader's commits arrive on BOTH CTAs' empty / accumulator-full barriers; the epilogue warps of
// both CTAs arrive on the leader's accumulator-empty barrier.  A cluster barrier brackets the
// kernel so neither CTA initialises late or exits early.
template <int BN>
struct PairTileConfig {
    static constexpr int kATileBytes = kBlockM * kBlockKBytes;   // this CTA's 128 rows of A
    static constexpr int kBTileBytes = (BN / 2) * kBlockKBytes;  // this CTA's half of the W rows
    static constexpr int kStageBytes = kATileBytes + kBTileBytes;
    static constexpr int kHalf0 = first_half_cols(BN, 0);
    static constexpr int kColParamBytes = epilogue_warps(0) * 4 * kHalf0 * 4;
    static constexpr int kStages = (208 * 1024 - kColParamBytes) / kStageBytes;  // 256: 6, 224: 6, 192: 7
    static constexpr int kTmemCols = 512;
    static constexpr int kBarrierBytes = (2 * kStages + 4) * 8 + 16;
    static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kColParamBytes + kBarrierBytes;
};

template <int BN, int KIND, int SUB, bool MC, bool CONV = false, int POSE = 0>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMaxThreads, 1)
gemm_i8_umma_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                         const I8Epilogue ep, const int m_total, const int n_total, const int k_total,
                         const uint32_t idesc, const int vec_ok, const int group_m, const int k_rot,
                         int32_t* error_word, const ConvTile conv)
{
    using Cfg = PairTileConfig<BN>;
    // SUB consecutive 128-byte k-blocks share one pair of barriers (a "slot"): one wait, one
    // expect-tx and one pair of commits per SUB x 4 MMAs.
    constexpr int kStages = Cfg::kStages / SUB;           // slots in the ring
    constexpr int kSlotBytes = SUB * Cfg::kStageBytes;
    constexpr int kPairM = 2 * kBlockM;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stage_base = smem;
    int32_t* col_params = reinterpret_cast<int32_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(col_params + Cfg::kColParamBytes / 4);
    uint64_t* empty_bar = full_bar + Cfg::kStages;
    uint64_t* acc_full_bar = empty_bar + Cfg::kStages;
    uint64_t* acc_empty_bar = acc_full_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();  // 0 = pair leader
    const int pair = static_cast<int>(blockIdx.x >> 1);
    const int num_pairs = static_cast<int>(gridDim.x >> 1);
    const int num_m = (m_total + kPairM - 1) / kPairM;
    const int num_n = (n_total + BN - 1) / BN;
    const int num_tiles = num_m * num_n;
    const int num_kb = (k_total + kBlockKBytes - 1) / kBlockKBytes;
    const TileWalk walk(num_m, num_n, group_m);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);   // the leader's: its own expect-tx arrival; bytes come from both CTAs
            mbar_init(&empty_bar[s], 1);  // one commit from the leader
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full_bar[a], 1);
            mbar_init(&acc_empty_bar[a], 2 * epilogue_warps(0));  // the leader's: the epilogue warps of both CTAs
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_w);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    cluster_sync_all();  // both CTAs' barriers and TMEM exist before anything is signalled across
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer (each CTA loads its own halves) ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
                const TileCoord tc = walk(tile);
                const int m0 = tc.m_blk * kPairM + static_cast<int>(rank) * kBlockM;
                const int n0 = tc.n_blk * BN + static_cast<int>(rank) * (BN / 2);
                const int rot = k_rotation(tile, k_rot, num_kb);
                for (int kb = 0; kb < num_kb; kb += SUB) {
                    if (!mbar_wait_cluster(&empty_bar[stage], phase ^ 1u, abort_flag)) {
                        atomicCAS(error_word, 0, kErrProducerWait);
                        ok = false;
                        break;
                    }
                    const int nsub = (num_kb - kb) < SUB ? (num_kb - kb) : SUB;
                    if (rank == 0) {
                        mbar_expect_tx(&full_bar[stage], 2 * nsub * Cfg::kStageBytes);
                    }
                    const uint32_t leader_full = map_to_cta(smem_u32(&full_bar[stage]), 0);
#pragma unroll
                    for (int j = 0; j < SUB; ++j) {
                        if (j < nsub) {
                            uint8_t* a_dst = stage_base + stage * kSlotBytes + j * Cfg::kStageBytes;
                            uint8_t* b_dst = a_dst + Cfg::kATileBytes;
                            const int kx = kb + j + rot < num_kb ? kb + j + rot : kb + j + rot - num_kb;
                            if constexpr (CONV) {
                                // This CTA's patch of the pair (2 * m_blk + rank), shifted by the k-block's tap.
                                const ConvPatch pt = conv_patch(conv, 2 * tc.m_blk + static_cast<int>(rank));
                                const int tap = kx / conv.kb_per_tap;
                                const int c0 = (kx - tap * conv.kb_per_tap) * kBlockKBytes;
                                const int ta = tap / conv.kw;
                                const int tb = tap - ta * conv.kw;
                                tma_load_4d_pair(a_dst, &map_a, leader_full, conv.c_base + c0,
                                                 (pt.tw << conv.bw_log2) * conv.sw - conv.pw + tb * conv.dw,
                                                 pt.th * conv.bh * conv.sh - conv.ph + ta * conv.dh, pt.img);
                            } else if constexpr ((POSE & 1) != 0) {
                                // A stored [K][M]: 128 k-rows of this CTA's 128 m-bytes.
                                tma_load_2d_pair(a_dst, &map_a, leader_full, m0, kx * kBlockKBytes);
                            } else {
                                tma_load_2d_pair(a_dst, &map_a, leader_full, kx * kBlockKBytes, m0);
                            }
                            if constexpr ((POSE & 2) != 0) {
                                // W stored [K][N]: 128 k-rows of this CTA's 128 n-bytes (BN = 256).
                                tma_load_2d_pair(b_dst, &map_w, leader_full, n0, kx * kBlockKBytes);
                            } else {
                                tma_load_2d_pair(b_dst, &map_w, leader_full, kx * kBlockKBytes, n0);
                            }
                        }
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer (pair leader only) ----------------
        if (lane == 0 && rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int local_tile = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += num_pairs, ++local_tile) {
                const int acc = local_tile & 1;
                const uint32_t acc_phase = (local_tile >> 1) & 1u;
                if (!mbar_wait_cluster(&acc_empty_bar[acc], acc_phase ^ 1u, abort_flag)) {
                    atomicCAS(error_word, 0, kErrAccumWait);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * 256);
                for (int kb = 0; kb < num_kb; kb += SUB) {
                    if (!mbar_wait_cluster(&full_bar[stage], phase, abort_flag)) {
                        atomicCAS(error_word, 0, kErrMmaWait);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const int nsub = (num_kb - kb) < SUB ? (num_kb - kb) : SUB;
#pragma unroll
                    for (int j = 0; j < SUB; ++j) {
                        if (j < nsub) {
                            const uint32_t a_addr = smem_u32(stage_base + stage * kSlotBytes + j * Cfg::kStageBytes);
                            const uint32_t b_addr = a_addr + Cfg::kATileBytes;
                            // MN-major tiles (POSE bits): 32 k-rows of 128 bytes per K step instead of 32 bytes
                            // along the row, as in the single-CTA kernel.
                            const uint64_t a_desc = (POSE & 1) ? umma_desc_sw128_mnmajor(a_addr, 128 * kBlockKBytes)
                                                               : umma_desc_sw128_kmajor(a_addr);
                            const uint64_t b_desc = (POSE & 2) ? umma_desc_sw128_mnmajor(b_addr, 128 * kBlockKBytes)
                                                               : umma_desc_sw128_kmajor(b_addr);
                            constexpr uint64_t a_step = (POSE & 1) ? 256u : 2u;
                            constexpr uint64_t b_step = (POSE & 2) ? 256u : 2u;
#pragma unroll
                            for (int ks = 0; ks < kBlockKBytes / kUmmaK; ++ks) {
                                umma_i8_pair(d_tmem, a_desc + static_cast<uint64_t>(ks) * a_step,
                                             b_desc + static_cast<uint64_t>(ks) * b_step, idesc,
                                             (kb > 0 || j > 0 || ks > 0) ? 1u : 0u);
                            }
                        }
                    }
                    // The slot is free in BOTH CTAs once these MMAs have read it.
                    if constexpr (MC) {
                        umma_commit_pair_mask(&empty_bar[stage], 3);
                    } else {
                        const uint32_t e = smem_u32(&empty_bar[stage]);
                        umma_commit_pair(map_to_cta(e, 0));
                        umma_commit_pair(map_to_cta(e, 1));
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) {
                    if constexpr (MC) {
                        umma_commit_pair_mask(&acc_full_bar[acc], 3);
                    } else {
                        const uint32_t f = smem_u32(&acc_full_bar[acc]);
                        umma_commit_pair(map_to_cta(f, 0));
                        umma_commit_pair(map_to_cta(f, 1));
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue warps (each CTA drains its own 128 rows) ----------------
        const int quarter = warp & 3;
        const bool fold_scale = KIND != NNB200_OUT_S32 && ep.scale_a == nullptr;
        const float folded_row_k = (KIND == NNB200_OUT_S8 || KIND == NNB200_OUT_U8)
                                       ? __fdiv_rn(ep.scale_a_scalar, ep.out_scale) : ep.scale_a_scalar;
        const bool fold_comp = (KIND == NNB200_OUT_S8 || KIND == NNB200_OUT_U8) && ep.compensate != 0 &&
                               ep.zp_a == nullptr && ep.r_a == nullptr;
        constexpr int kTermIters = (Cfg::kHalf0 + 31) / 32;   // 4 for 256-wide tiles
        ColTerms next_terms[kTermIters];
        constexpr int kHalf0 = Cfg::kHalf0;
        const int half = (warp - 2) >> 2;   // two warps per lane quarter, half of the columns each
        const int col0 = half * kHalf0;
        const int ncols = half ? BN - kHalf0 : kHalf0;
        float* cs = reinterpret_cast<float*>(col_params + (warp - 2) * 4 * kHalf0);
        int32_t* cb = reinterpret_cast<int32_t*>(cs) + kHalf0;
        int32_t* cr = cb + kHalf0;
        int32_t* cz = cr + kHalf0;
        int local_tile = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local_tile) {
            const TileCoord tc = walk(tile);
            const int acc = local_tile & 1;
            const uint32_t acc_phase = (local_tile >> 1) & 1u;
            const int n_base = tc.n_blk * BN + col0;   // first column this warp drains

            // This tile's per-column terms: fetched while the previous tile was being drained, or
            // (first tile) now, hidden behind the tile's main loop.
            __syncwarp();
#pragma unroll
            for (int i = 0; i < kTermIters; ++i) {
                const int j = lane + i * 32;
                if (j < ncols) {
                    const ColTerms ct = finish_col_terms<KIND>(
                        ep, local_tile > 0 ? next_terms[i] : load_col_terms<KIND>(ep, n_base + j, n_total), fold_scale,
                        folded_row_k, fold_comp);
                    cs[j] = ct.scale;
                    cb[j] = ct.bias;
                    cr[j] = ct.rw;
                    cz[j] = ct.zpw;
                }
            }
            __syncwarp();

            int64_t m = static_cast<int64_t>(tc.m_blk) * kPairM + static_cast<int64_t>(rank) * kBlockM +
                        quarter * 32 + lane;
            bool row_ok = m < m_total;
            uint32_t bad_h = 0, bad_w = 0;   // CONV: the row's border class along each axis
            if constexpr (CONV) {
                const ConvRow cr_ = conv_row(conv, 2 * tc.m_blk + static_cast<int>(rank), quarter * 32 + lane);
                m = cr_.m;
                row_ok = cr_.ok;
                bad_h = cr_.bad_h;
                bad_w = cr_.bad_w;
            }
            I8RowTerms rt;
            rt.zpa = 0;
            rt.ra = 0;
            rt.s_a = 1.0f;
            rt.row_k = 1.0f;
            if (row_ok) {
                rt = i8_row_terms(ep, m);
            }

            int ok = 1;
            if (lane == 0) {
                ok = mbar_wait_cluster(&acc_full_bar[acc], acc_phase, abort_flag) ? 1 : 0;
            }
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) {
                atomicCAS(error_word, 0, kErrEpilogueWait);
                break;
            }
            tc_fence_after_sync();

            {
                // The next tile's column terms, in flight while this tile is drained.
                const int next = tile + num_pairs;
                if (next < num_tiles) {
                    const int next_base = walk(next).n_blk * BN + col0;
#pragma unroll
                    for (int i = 0; i < kTermIters; ++i) {
                        next_terms[i] = load_col_terms<KIND>(ep, next_base + lane + i * 32, n_total);
                    }
                }
            }

            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(acc * 256 + col0);
            // Chunks of 32 columns, two register sets: the load of the next chunk is in flight while
            // this one is requantised and stored.
            const int left = n_total - n_base;
            const int nch = left <= 0 ? 0 : min(ncols / 32, (left + 31) / 32);   // uniform across the warp
            const auto finish = [&](int c, uint32_t (&v)[32]) {
                const int n0 = n_base + c * 32;
                if constexpr (CONV) {
                    conv_border_fix(conv, v, bad_h, bad_w, n0, n_total);
                }
                epilogue_chunk<KIND>(ep, rt, v, m, row_ok, n0, n_total, cs + c * 32, cb + c * 32, cr + c * 32,
                                     cz + c * 32, vec_ok, fold_scale, fold_comp);
            };
            uint32_t va[32], vb[32];
            if (nch > 0) {
                tmem_ld_32x32(t_row, va);
            }
#pragma unroll 1
            for (int c = 0; c < nch; c += 2) {
                tmem_ld_wait();
                if (c + 1 < nch) {
                    tmem_ld_32x32(t_row + static_cast<uint32_t>((c + 1) * 32), vb);
                }
                finish(c, va);
                if (c + 1 < nch) {
                    tmem_ld_wait();
                    if (c + 2 < nch) {
                        tmem_ld_32x32(t_row + static_cast<uint32_t>((c + 2) * 32), va);
                    }
                    finish(c + 1, vb);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty_bar[acc]), 0));
            }
        }
        if (ep.direct_peers > 0) {
            __threadfence_system();  // stores into the other rank's copy are performed before the kernel completes
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before_sync();
    cluster_sync_all();  // the peer has stopped signalling into / reading from this CTA
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    }
}

// CTA-pair launch: 256 x BN tiles, two CTAs per tile.  NNB200_UNSUPPORTED when the device cannot
// co-schedule a single pair (the caller then uses the single-CTA form).
// Step of the per-tile K rotation (see k_rotation).  Default: 5 blocks per tile index where the
// weight has at most 4096 rows -- few column tiles, so many CTAs of a wave share each W tile
// (measured +3..10 % there, -2 % at 8192 rows); knob I8_K_ROTATE sets it, 0 = every tile starts
// at block 0.
inline int k_rotation_step(int n)
{
    const int kn = knob(NNB200_KNOB_I8_K_ROTATE);
    return kn >= 0 ? kn : (n <= 4096 ? 5 : 0);
}

template <int BN, int KIND, int SUB = 1, bool MC = false, int POSE = 0>
int launch_pair_variant(const I8Problem& p, const I8Epilogue& ep, int m, int n, int k, uint32_t a_fmt, int vec_ok,
                        const DeviceInfo& dev, cudaStream_t stream)
{
    static_assert(POSE == 0 || BN == 256, "an MN-major W half is one 128-column block");
    using Cfg = PairTileConfig<BN>;
    auto kernel = gemm_i8_umma_pair_kernel<BN, KIND, SUB, MC, false, POSE>;
    static std::once_flag once[kMaxDevices];
    static cudaError_t attr_err[kMaxDevices];
    static int max_pairs[kMaxDevices];
    std::call_once(once[dev.device], [&] {
        attr_err[dev.device] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        max_pairs[dev.device] = 0;
        if (attr_err[dev.device] == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(static_cast<unsigned>(dev.sm_count & ~1));
            cfg.blockDim = dim3(num_threads(0));
            cfg.dynamicSmemBytes = Cfg::kSmemBytes;
            int count = 0;
            if (cudaOccupancyMaxActiveClusters(&count, kernel, &cfg) == cudaSuccess) {
                max_pairs[dev.device] = count;
            }
        }
    });
    if (attr_err[dev.device] != cudaSuccess) {
        return NNB200_INTERNAL;
    }
    if (max_pairs[dev.device] < 1) {
        return NNB200_UNSUPPORTED;
    }
    CUtensorMap map_a, map_w;
    const bool map_a_ok =
        (POSE & 1) ? make_tma_2d(&map_a, p.a, 1, static_cast<uint64_t>(m), static_cast<uint64_t>(k),
                                 static_cast<uint64_t>(p.a_stride_k), kBlockM, kBlockKBytes)
                   : make_tma_2d(&map_a, p.a, 1, static_cast<uint64_t>(k), static_cast<uint64_t>(m),
                                 static_cast<uint64_t>(p.a_stride_m), kBlockKBytes, kBlockM);
    const bool map_w_ok =
        (POSE & 2) ? make_tma_2d(&map_w, p.w, 1, static_cast<uint64_t>(n), static_cast<uint64_t>(k),
                                 static_cast<uint64_t>(p.w_stride_k), 128, kBlockKBytes)
                   : make_tma_2d(&map_w, p.w, 1, static_cast<uint64_t>(k), static_cast<uint64_t>(n),
                                 static_cast<uint64_t>(p.w_stride_n), kBlockKBytes, BN / 2);
    if (!map_a_ok || !map_w_ok) {
        return NNB200_INTERNAL;
    }
    const int num_tiles = ((m + 2 * kBlockM - 1) / (2 * kBlockM)) * ((n + BN - 1) / BN);
    const int pairs = num_tiles < max_pairs[dev.device] ? num_tiles : max_pairs[dev.device];
    int group_m = static_cast<int>((40ll << 20) / (static_cast<int64_t>(2 * kBlockM) * (k > 0 ? k : 1)));
    group_m = group_m < 2 ? 2 : group_m;
    constexpr uint32_t major_bits = ((POSE & 1) ? kUmmaAMajorMN : 0u) | ((POSE & 2) ? kUmmaBMajorMN : 0u);
    kernel<<<2 * pairs, num_threads(0), Cfg::kSmemBytes, stream>>>(map_a, map_w, ep, m, n, k,
                                                               umma_idesc(2, a_fmt, 1, 2 * kBlockM, BN) | major_bits, vec_ok, group_m,
                                                               k_rotation_step(n), dev.error_word, ConvTile{});
    note_launch();
    return cuda_status(cudaGetLastError());
}

template <int BN, int SUB = 1, bool MC = false, int POSE = 0>
int launch_pair_bn(const I8Problem& p, const I8Epilogue& ep, int m, int n, int k, uint32_t a_fmt, int vec_ok,
                   const DeviceInfo& dev, cudaStream_t stream)
{
    switch (ep.out_kind) {
    case NNB200_OUT_S32: return launch_pair_variant<BN, NNB200_OUT_S32, SUB, MC, POSE>(p, ep, m, n, k, a_fmt, vec_ok, dev, stream);
    case NNB200_OUT_S8: return launch_pair_variant<BN, NNB200_OUT_S8, SUB, MC, POSE>(p, ep, m, n, k, a_fmt, vec_ok, dev, stream);
    case NNB200_OUT_U8: return launch_pair_variant<BN, NNB200_OUT_U8, SUB, MC, POSE>(p, ep, m, n, k, a_fmt, vec_ok, dev, stream);
    case NNB200_OUT_F32: return launch_pair_variant<BN, NNB200_OUT_F32, SUB, MC, POSE>(p, ep, m, n, k, a_fmt, vec_ok, dev, stream);
    case NNB200_OUT_F16: return launch_pair_variant<BN, NNB200_OUT_F16, SUB, MC, POSE>(p, ep, m, n, k, a_fmt, vec_ok, dev, stream);
    default: return NNB200_UNSUPPORTED;
    }
}

template <int BN, int KIND, int PEERS>
int launch_variant(const CUtensorMap& map_a, const CUtensorMap& map_w, const I8Epilogue& ep, int m, int n, int k,
                   uint32_t idesc, int vec_ok, const DeviceInfo& dev, cudaStream_t stream)
{
    using Cfg = TileConfig<BN, PEERS>;
    auto kernel = gemm_i8_umma_kernel<BN, KIND, PEERS>;
    constexpr int kSmem = Cfg::kSmemBytes;
    PeerMaps maps;
    std::memset(&maps, 0, sizeof(maps));
    if constexpr (PEERS) {
        // Output windows as 2-D byte tensors [m][n] with the caller's pitch; 128 x 32 boxes.
        for (int d = 0; d <= ep.num_peers; ++d) {
            const void* base = d == 0 ? ep.out : ep.peer_out[d - 1];
            if (!make_tma_2d(&maps.m[d], base, 1, static_cast<uint64_t>(n), static_cast<uint64_t>(m),
                             static_cast<uint64_t>(ep.ldc), Cfg::kStageGroupCols, 32)) {
                return NNB200_INTERNAL;
            }
        }
    }
    static std::once_flag once[kMaxDevices];
    static cudaError_t attr_err[kMaxDevices];
    std::call_once(once[dev.device], [&] {
        attr_err[dev.device] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    });
    if (attr_err[dev.device] != cudaSuccess) {
        return NNB200_INTERNAL;
    }
    const int num_tiles = ((m + kBlockM - 1) / kBlockM) * ((n + BN - 1) / BN);
    const int grid = num_tiles < dev.sm_count ? num_tiles : dev.sm_count;
    // Raster group: as many m-blocks as keep the group's band of A within about a third of L2
    // (126 MB on B200), so that W is read from DRAM once per group.
    int group_m = static_cast<int>((40ll << 20) / (static_cast<int64_t>(kBlockM) * (k > 0 ? k : 1)));
    group_m = group_m < 4 ? 4 : group_m;
    if (knob(NNB200_KNOB_GROUP_M) > 0) {
        group_m = knob(NNB200_KNOB_GROUP_M);
    }
    kernel<<<grid, num_threads(PEERS), kSmem, stream>>>(map_a, map_w, maps, ep, m, n, k, idesc, vec_ok, group_m,
                                                 k_rotation_step(n), dev.error_word, ConvTile{});
    note_launch();
    return cuda_status(cudaGetLastError());
}

template <int BN>
int launch_bn(int kind, const CUtensorMap& map_a, const CUtensorMap& map_w, const I8Epilogue& ep, int m, int n, int k,
              uint32_t idesc, int vec_ok, const DeviceInfo& dev, cudaStream_t stream)
{
    if (ep.num_peers > 0 || ep.mc_out != nullptr) {
        // Sharded write-back exists for the 8-bit destinations: 256- and 128-wide tiles, and --
        // multicast stores only, whose pieces need not be whole 128-byte boxes -- 224-wide ones.
        // knob I8_PEER_STAGING = 1 / 2 forces the staging depth (measurement aid).
        // One staging tile per warp and the fourth ring stage it leaves room for: measured faster than
        // two tiles and three stages at every size (per step, one / three / seven peers:
        // 0.380 -> 0.346, 0.262 -> 0.237 and 0.255 -> 0.238 ms).  Multicast stores leave the SM as
        // ordinary stores: one staging tile per warp is all they need.
        bool single = true;
        if (const int staging = knob(NNB200_KNOB_I8_PEER_STAGING); staging == 1 || staging == 2) {
            single = staging == 1;
        }
        if constexpr (BN == 256 || BN == 128) {
            if (kind == NNB200_OUT_S8) {
                return single
                           ? launch_variant<BN, NNB200_OUT_S8, 1>(map_a, map_w, ep, m, n, k, idesc, vec_ok, dev, stream)
                           : launch_variant<BN, NNB200_OUT_S8, 2>(map_a, map_w, ep, m, n, k, idesc, vec_ok, dev, stream);
            }
            if (kind == NNB200_OUT_U8) {
                return single
                           ? launch_variant<BN, NNB200_OUT_U8, 1>(map_a, map_w, ep, m, n, k, idesc, vec_ok, dev, stream)
                           : launch_variant<BN, NNB200_OUT_U8, 2>(map_a, map_w, ep, m, n, k, idesc, vec_ok, dev, stream);
            }
        }
        if constexpr (BN == 224) {
            if (ep.mc_out != nullptr && kind == NNB200_OUT_S8) {
                return launch_variant<BN, NNB200_OUT_S8, 1>(map_a, map_w, ep, m, n, k, idesc, vec_ok, dev, stream);
            }
            if (ep.mc_out != nullptr && kind == NNB200_OUT_U8) {
                return launch_variant<BN, NNB200_OUT_U8, 1>(map_a, map_w, ep, m, n, k, idesc, vec_ok, dev, stream);
            }
        }
        return NNB200_UNSUPPORTED;
    }
    switch (kind) {
    case NNB200_OUT_S32: return launch_variant<BN, NNB200_OUT_S32, 0>(map_a, map_w, ep, m, n, k, idesc, vec_ok, dev, stream);
    case NNB200_OUT_S8: return launch_variant<BN, NNB200_OUT_S8, 0>(map_a, map_w, ep, m, n, k, idesc, vec_ok, dev, stream);
    case NNB200_OUT_U8: return launch_variant<BN, NNB200_OUT_U8, 0>(map_a, map_w, ep, m, n, k, idesc, vec_ok, dev, stream);
    case NNB200_OUT_F32: return launch_variant<BN, NNB200_OUT_F32, 0>(map_a, map_w, ep, m, n, k, idesc, vec_ok, dev, stream);
    case NNB200_OUT_F16: return launch_variant<BN, NNB200_OUT_F16, 0>(map_a, map_w, ep, m, n, k, idesc, vec_ok, dev, stream);
    default: return NNB200_UNSUPPORTED;
    }
}

}  // namespace

namespace {

template <int BN, int KIND>
int launch_conv_variant(const CUtensorMap& map_a, const CUtensorMap& map_w, const I8Epilogue& ep, int m_tiles, int n,
                        int k, uint32_t idesc, int vec_ok, const ConvTile& conv, const DeviceInfo& dev,
                        cudaStream_t stream)
{
    using Cfg = TileConfig<BN, 0>;
    auto kernel = gemm_i8_umma_kernel<BN, KIND, 0, true>;
    static std::once_flag once[kMaxDevices];
    static cudaError_t attr_err[kMaxDevices];
    std::call_once(once[dev.device], [&] {
        attr_err[dev.device] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    });
    if (attr_err[dev.device] != cudaSuccess) {
        return NNB200_INTERNAL;
    }
    PeerMaps maps;
    std::memset(&maps, 0, sizeof(maps));
    const int num_tiles = m_tiles * ((n + BN - 1) / BN);
    const int grid = num_tiles < dev.sm_count ? num_tiles : dev.sm_count;
    int group_m = static_cast<int>((40ll << 20) / (static_cast<int64_t>(kBlockM) * (k > 0 ? k : 1)));
    group_m = group_m < 4 ? 4 : group_m;
    kernel<<<grid, num_threads(0), Cfg::kSmemBytes, stream>>>(map_a, map_w, maps, ep, m_tiles * kBlockM, n, k, idesc, vec_ok,
                                                            group_m, k_rotation_step(n), dev.error_word, conv);
    note_launch();
    return cuda_status(cudaGetLastError());
}

// The CTA-pair form of the same: two patches per 256 x 256 tile, each CTA loading its own patch
// and half of the filter rows.  NNB200_UNSUPPORTED when the device cannot co-schedule a pair.
template <int KIND>
int launch_conv_pair_variant(const CUtensorMap& map_a, const CUtensorMap& map_w, const I8Epilogue& ep, int m_tiles, int n,
                             int k, uint32_t a_fmt, int vec_ok, const ConvTile& conv, const DeviceInfo& dev,
                             cudaStream_t stream)
{
    constexpr int BN = 256;
    using Cfg = PairTileConfig<BN>;
    auto kernel = gemm_i8_umma_pair_kernel<BN, KIND, 2, true, true>;
    static std::once_flag once[kMaxDevices];
    static cudaError_t attr_err[kMaxDevices];
    static int max_pairs[kMaxDevices];
    std::call_once(once[dev.device], [&] {
        attr_err[dev.device] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        max_pairs[dev.device] = 0;
        if (attr_err[dev.device] == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(static_cast<unsigned>(dev.sm_count & ~1));
            cfg.blockDim = dim3(num_threads(0));
            cfg.dynamicSmemBytes = Cfg::kSmemBytes;
            int count = 0;
            if (cudaOccupancyMaxActiveClusters(&count, kernel, &cfg) == cudaSuccess) {
                max_pairs[dev.device] = count;
            }
        }
    });
    if (attr_err[dev.device] != cudaSuccess) {
        return NNB200_INTERNAL;
    }
    if (max_pairs[dev.device] < 1) {
        return NNB200_UNSUPPORTED;
    }
    const int num_tiles = ((m_tiles + 1) / 2) * ((n + BN - 1) / BN);
    const int pairs = num_tiles < max_pairs[dev.device] ? num_tiles : max_pairs[dev.device];
    int group_m = static_cast<int>((40ll << 20) / (static_cast<int64_t>(2 * kBlockM) * (k > 0 ? k : 1)));
    group_m = group_m < 2 ? 2 : group_m;
    kernel<<<2 * pairs, num_threads(0), Cfg::kSmemBytes, stream>>>(map_a, map_w, ep, m_tiles * kBlockM, n, k,
                                                               umma_idesc(2, a_fmt, 1, 2 * kBlockM, BN), vec_ok, group_m,
                                                               k_rotation_step(n), dev.error_word, conv);
    note_launch();
    return cuda_status(cudaGetLastError());
}

int launch_conv_pair(const CUtensorMap& map_a, const CUtensorMap& map_w, const I8Epilogue& ep, int m_tiles, int n, int k,
                     uint32_t a_fmt, int vec_ok, const ConvTile& conv, const DeviceInfo& dev, cudaStream_t stream)
{
    switch (ep.out_kind) {
    case NNB200_OUT_S8: return launch_conv_pair_variant<NNB200_OUT_S8>(map_a, map_w, ep, m_tiles, n, k, a_fmt, vec_ok, conv, dev, stream);
    case NNB200_OUT_U8: return launch_conv_pair_variant<NNB200_OUT_U8>(map_a, map_w, ep, m_tiles, n, k, a_fmt, vec_ok, conv, dev, stream);
    case NNB200_OUT_F32: return launch_conv_pair_variant<NNB200_OUT_F32>(map_a, map_w, ep, m_tiles, n, k, a_fmt, vec_ok, conv, dev, stream);
    case NNB200_OUT_F16: return launch_conv_pair_variant<NNB200_OUT_F16>(map_a, map_w, ep, m_tiles, n, k, a_fmt, vec_ok, conv, dev, stream);
    default: return NNB200_UNSUPPORTED;
    }
}

template <int BN>
int launch_conv_bn(const CUtensorMap& map_a, const CUtensorMap& map_w, const I8Epilogue& ep, int m_tiles, int n, int k,
                   uint32_t idesc, int vec_ok, const ConvTile& conv, const DeviceInfo& dev, cudaStream_t stream)
{
    switch (ep.out_kind) {
    case NNB200_OUT_S8: return launch_conv_variant<BN, NNB200_OUT_S8>(map_a, map_w, ep, m_tiles, n, k, idesc, vec_ok, conv, dev, stream);
    case NNB200_OUT_U8: return launch_conv_variant<BN, NNB200_OUT_U8>(map_a, map_w, ep, m_tiles, n, k, idesc, vec_ok, conv, dev, stream);
    case NNB200_OUT_F32: return launch_conv_variant<BN, NNB200_OUT_F32>(map_a, map_w, ep, m_tiles, n, k, idesc, vec_ok, conv, dev, stream);
    case NNB200_OUT_F16: return launch_conv_variant<BN, NNB200_OUT_F16>(map_a, map_w, ep, m_tiles, n, k, idesc, vec_ok, conv, dev, stream);
    default: return NNB200_UNSUPPORTED;
    }
}

}  // namespace

// Implicit-GEMM convolution of one group: output pixels are tiled in patches of 128 (bh rows x
// bw columns of one image, bw a power of two chosen for the least padding), the activation is
// read through a 4-D tensor map {c, w, h, n} whose boxes are those patches shifted by the tap.
int launch_conv_i8_umma(const ConvUmmaArgs& c, const I8Epilogue& ep, const DeviceInfo& dev, cudaStream_t stream)
{
    ConvTile t;
    std::memset(&t, 0, sizeof(t));
    const int best = conv_patch_log2(c.oh, c.ow, nullptr);
    t.oh = c.oh; t.ow = c.ow; t.ih = c.ih; t.iw = c.iw;
    t.kh = c.kh; t.kw = c.kw; t.dh = c.dh; t.dw = c.dw; t.ph = c.ph; t.pw = c.pw;
    t.sh = c.sh; t.sw = c.sw;
    t.bw_log2 = best;
    t.bh = 128 >> best;
    t.tiles_w = (c.ow + (1 << best) - 1) >> best;
    t.tiles_h = (c.oh + t.bh - 1) / t.bh;
    t.c_base = c.c_base;
    t.kb_per_tap = c.icg / kBlockKBytes;
    t.zp_x = c.zp_x;
    t.wtap_ld = c.wtap_ld;
    t.nh = c.nh;
    t.nw = c.nw;
    for (int q = 0; q < 8; ++q) {
        t.mask_h[q] = c.mask_h[q];
        t.mask_w[q] = c.mask_w[q];
    }
    t.border = c.border;
    const int64_t m_tiles64 = static_cast<int64_t>(c.batch) * t.tiles_h * t.tiles_w;
    if (m_tiles64 > (INT32_MAX / kBlockM)) {
        return NNB200_UNSUPPORTED;
    }
    const int m_tiles = static_cast<int>(m_tiles64);
    t.m_tiles = m_tiles;
    const int n = c.ocg, k = c.k;
    int bn = 256;
    if (static_cast<int64_t>(m_tiles) * ((n + 255) / 256) < dev.sm_count || n <= 128) {
        bn = 128;
        if (static_cast<int64_t>(m_tiles) * ((n + 127) / 128) < dev.sm_count || n <= 64) {
            bn = 64;
        }
    }
    CUtensorMap map_a, map_w;
    if (!make_tma_nhwc_u8(&map_a, c.x, static_cast<uint64_t>(c.ic_total), static_cast<uint64_t>(c.iw),
                          static_cast<uint64_t>(c.ih), static_cast<uint64_t>(c.batch), static_cast<uint64_t>(c.in_w),
                          static_cast<uint64_t>(c.in_h), static_cast<uint64_t>(c.in_n), kBlockKBytes, 1u << best,
                          static_cast<uint32_t>(t.bh), static_cast<uint32_t>(c.sw), static_cast<uint32_t>(c.sh)) ||
        !make_tma_2d(&map_w, c.wt, 1, static_cast<uint64_t>(k), static_cast<uint64_t>(n), static_cast<uint64_t>(c.ldw),
                     kBlockKBytes, static_cast<uint32_t>(bn))) {
        return NNB200_INTERNAL;
    }
    const int elem = ep.out_kind == NNB200_OUT_S32 || ep.out_kind == NNB200_OUT_F32 ? 4 : (ep.out_kind == NNB200_OUT_F16 ? 2 : 1);
    const uint64_t pitch_bytes = static_cast<uint64_t>(ep.ldc) * elem;
    const int vec_ok = (((reinterpret_cast<uintptr_t>(ep.out) & 15u) == 0 && (pitch_bytes & 15u) == 0) ? 1 : 0) |
                       (((reinterpret_cast<uintptr_t>(ep.out) & 31u) == 0 && (pitch_bytes & 31u) == 0) ? 2 : 0);
    // CTA pairs (two patches per tile, half of the filter rows per CTA) where there are enough
    // pair tiles to fill the device: a single CTA's 128 x 256 tile asks its SM for more operand
    // bytes per clock than the L2 delivers to one SM, the pair's halves do not.  Knob I8_PAIR = 0
    // keeps the single-CTA form.
    if (bn == 256 && knob(NNB200_KNOB_I8_PAIR) != 0 &&
        static_cast<int64_t>((m_tiles + 1) / 2) * ((n + 255) / 256) >= dev.sm_count / 2) {
        CUtensorMap map_wh;
        if (!make_tma_2d(&map_wh, c.wt, 1, static_cast<uint64_t>(k), static_cast<uint64_t>(n), static_cast<uint64_t>(c.ldw),
                         kBlockKBytes, 128u)) {
            return NNB200_INTERNAL;
        }
        const int st = launch_conv_pair(map_a, map_wh, ep, m_tiles, n, k, c.a_unsigned ? 0u : 1u, vec_ok, t, dev, stream);
        if (st != NNB200_UNSUPPORTED) {
            return st;
        }
    }
    const uint32_t idesc = umma_idesc(2, c.a_unsigned ? 0u : 1u, 1, kBlockM, bn);
    switch (bn) {
    case 256: return launch_conv_bn<256>(map_a, map_w, ep, m_tiles, n, k, idesc, vec_ok, t, dev, stream);
    case 128: return launch_conv_bn<128>(map_a, map_w, ep, m_tiles, n, k, idesc, vec_ok, t, dev, stream);
    default: return launch_conv_bn<64>(map_a, map_w, ep, m_tiles, n, k, idesc, vec_ok, t, dev, stream);
    }
}

bool umma_i8_supported(const I8Problem& p)
{
    if (p.m < 1 || p.n < 1 || p.k < 1 || p.m > INT32_MAX || p.n > INT32_MAX || p.k > INT32_MAX) {
        return false;
    }
    // Each operand in either pose, as long as TMA can address it: the contiguous index has
    // stride 1, the other a pitch that is a multiple of 16 bytes and covers a row; 16-byte base.
    const auto aligned16 = [](uint64_t v) { return (v & 15u) == 0; };
    const auto operand_ok = [&](const void* base, int64_t stride_mn, int64_t stride_k, int64_t mn, int64_t k) {
        if (!aligned16(reinterpret_cast<uintptr_t>(base))) {
            return false;
        }
        if (stride_k == 1) {   // K-major: rows of k bytes
            return aligned16(static_cast<uint64_t>(stride_mn)) && stride_mn >= k;
        }
        return stride_mn == 1 && aligned16(static_cast<uint64_t>(stride_k)) && stride_k >= mn;   // MN-major
    };
    return operand_ok(p.a, p.a_stride_m, p.a_stride_k, p.m, p.k) && operand_ok(p.w, p.w_stride_n, p.w_stride_k, p.n, p.k);
}

int launch_gemm_i8_umma(const I8Problem& p, const I8Epilogue& ep_in, const DeviceInfo& dev, cudaStream_t stream)
{
    const int m = static_cast<int>(p.m);
    const int n = static_cast<int>(p.n);
    const int k = static_cast<int>(p.k);

    // A shard with ONE peer (two ranks) is bound by its GEMM, not by the link: it runs the
    // ordinary kernels -- the CTA-pair form where that applies -- whose epilogue stores each
    // 32-byte sector a second time, into the peer's copy, instead of the staged bulk stores of
    // the sharded form.  Needs whole 32-column chunks and 32-byte aligned destinations.
    I8Epilogue ep = ep_in;
    {
        const auto mis32 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 31u) != 0; };
        const uint64_t pitch = static_cast<uint64_t>(ep.ldc);   // 8-bit destinations: bytes
        if (ep.num_peers == 1 && ep.mc_out == nullptr && knob(NNB200_KNOB_I8_PEER_STAGING) <= 0 &&
            (ep.out_kind == NNB200_OUT_S8 || ep.out_kind == NNB200_OUT_U8) && p.a_stride_k == 1 && p.w_stride_k == 1 &&
            m >= 4 * kBlockM && k >= 2048 && n % 32 == 0 && pitch % 32 == 0 && !mis32(ep.out) && !mis32(ep.peer_out[0])) {
            ep.direct_peers = 1;
            ep.num_peers = 0;
        }
    }

    // Tile width.  When even the widest tile gives every SM work, take the width with the least
    // padded work over whole waves (waves x width; ties to the wider tile); narrow problems
    // trade arithmetic intensity for parallelism.
    const int num_m = (m + kBlockM - 1) / kBlockM;
    const bool sharded = ep.num_peers > 0 || ep.mc_out != nullptr;
    int bn = 256;
    if (static_cast<int64_t>(num_m) * ((n + 255) / 256) < dev.sm_count) {
        bn = 128;
        if (static_cast<int64_t>(num_m) * ((n + 127) / 128) < dev.sm_count && !sharded) {
            bn = 64;
        }
    } else if (sharded) {
        // A shard of a wide layer often ends a little past a whole number of waves (N / 8 = 3584:
        // 448 tiles of 256 columns on 148 SMs = 3.03 waves).  With multicast stores the 224-wide
        // tile is available: 512 tiles = 3.46 waves, an eighth less padded work.
        const auto padded_work = [&](int width) {
            const int64_t tiles = static_cast<int64_t>(num_m) * ((n + width - 1) / width);
            return (tiles + dev.sm_count - 1) / dev.sm_count * width;
        };
        if (ep.mc_out != nullptr && padded_work(224) * 100 < padded_work(256) * 92) {
            bn = 224;
        }
    } else {
        const auto padded_work = [&](int width) {
            const int64_t tiles = static_cast<int64_t>(num_m) * ((n + width - 1) / width);
            return (tiles + dev.sm_count - 1) / dev.sm_count * width;
        };
        int64_t best_cost = padded_work(256);
        for (const int cand : {224, 192}) {
            // A narrower tile moves more operand bytes per multiply-add (measured: about 8 % slower
            // per unit of work at 224): it has to save more than that.
            if (padded_work(cand) * 100 < best_cost * 92) {
                best_cost = padded_work(cand);
                bn = cand;
            }
        }
        // Single-wave form: when the problem needs a second, mostly empty wave, a tile wide enough
        // to give every CTA exactly one tile (two MMAs of BN / 2 columns per k-step) ends sooner.
        for (const int wide : {320, 384, 448, 512}) {
            const int64_t tiles = static_cast<int64_t>(num_m) * ((n + wide - 1) / wide);
            if (tiles <= dev.sm_count) {
                if (static_cast<int64_t>(wide) * 100 < best_cost * 92) {
                    best_cost = wide;
                    bn = wide;
                }
                break;  // wider ones only add padding
            }
        }
    }
    if (const int v = knob(NNB200_KNOB_I8_BN); v > 0) {  // measurement aid
        if (v == 512 || v == 448 || v == 384 || v == 320 || v == 256 || v == 224 || v == 192 || v == 128 || v == 64) {
            bn = v;
        }
    }
    // Operand poses: MN-major means the operand's M / N index is the contiguous one in memory
    // (MatMul's transpose_a, and its default [K, N] weights).  An MN-major W tile is brought in as
    // whole 128-column blocks, so its width is 256 or 128.
    const bool a_mn = p.a_stride_k != 1;
    const bool w_mn = p.w_stride_k != 1;
    if (w_mn && bn != 256 && bn != 128) {
        bn = (bn > 256 || static_cast<int64_t>(num_m) * ((n + 255) / 256) >= dev.sm_count) ? 256 : 128;
    }
    const uint32_t major_bits = (a_mn ? kUmmaAMajorMN : 0u) | (w_mn ? kUmmaBMajorMN : 0u);
    const auto idesc_of = [&](int mma_n) { return umma_idesc(2, p.a_unsigned ? 0u : 1u, 1, kBlockM, mma_n) | major_bits; };

    CUtensorMap map_a, map_w;
    const bool map_a_ok =
        a_mn ? make_tma_2d(&map_a, p.a, 1, static_cast<uint64_t>(m), static_cast<uint64_t>(k),
                           static_cast<uint64_t>(p.a_stride_k), kBlockM, kBlockKBytes)
             : make_tma_2d(&map_a, p.a, 1, static_cast<uint64_t>(k), static_cast<uint64_t>(m),
                           static_cast<uint64_t>(p.a_stride_m), kBlockKBytes, kBlockM);
    const bool map_w_ok =
        w_mn ? make_tma_2d(&map_w, p.w, 1, static_cast<uint64_t>(n), static_cast<uint64_t>(k),
                           static_cast<uint64_t>(p.w_stride_k), 128, kBlockKBytes)
             : make_tma_2d(&map_w, p.w, 1, static_cast<uint64_t>(k), static_cast<uint64_t>(n),
                           static_cast<uint64_t>(p.w_stride_n), kBlockKBytes, static_cast<uint32_t>(bn > 256 ? bn / 2 : bn));
    if (!map_a_ok || !map_w_ok) {
        return NNB200_INTERNAL;
    }

    // Destination vector stores need a 16-byte aligned base and row pitch.
    const int elem = (ep.out_kind == NNB200_OUT_S32 || ep.out_kind == NNB200_OUT_F32) ? 4
                     : (ep.out_kind == NNB200_OUT_F16)                                ? 2
                                                                                      : 1;
    // Destination vector stores: bit 0 = 16-byte aligned base and row pitch, bit 1 = 32-byte.
    const uint64_t pitch_bytes = static_cast<uint64_t>(ep.ldc) * static_cast<uint64_t>(elem);
    const int vec_ok = (((reinterpret_cast<uintptr_t>(ep.out) & 15u) == 0 && (pitch_bytes & 15u) == 0) ? 1 : 0) |
                       (((reinterpret_cast<uintptr_t>(ep.out) & 31u) == 0 && (pitch_bytes & 31u) == 0) ? 2 : 0) |
                       (a_mn ? 16 : 0) | (w_mn ? 32 : 0);   // bits 4-5: operand poses, read by the kernel

    const uint32_t a_fmt = p.a_unsigned ? 0u : 1u;

    // CTA-pair form from 256 rows up, with a K of 2048 or more (below that single CTAs are level or
    // ahead: 22.3 against 23.7 us at 4096 x 4096 x 1024, 35.6 against 37.4 at 8192 x 4096 x 1024) and at
    // least 24 tiles of 256 x 256.  CUDA-graph timings, single / pair: 512 x 4096 x 4096 (32 tiles)
    // 24.9 / 16.6 us, 256 x 8192 x 8192 (32) 45.3 / 26.1, 384 x 8192 x 4096 (64) 26.9 / 17.0, 512 x 4096 x 11008
    // (32) 58.3 / 31.9; with 16 tiles or fewer they are level or single CTAs ahead (256 x 4096 x 4096:
    // 14.9 / 16.3).  With more tiles than SM pairs, where the single-CTA form would pick a narrower
    // tile to fill its waves, the pairs' own waves must be at least three quarters full
    // (2048 x 8192 x 2048, 256 tiles on 74 pairs: 30.9 / 28.5; not 640 x 8192 x 4096, 96 tiles: 22.5 / 27.2;
    // not M = 512, N = 11008, 86 tiles: 22.3 / 27.3).
    // Knob I8_PAIR: 0 = never; 2 = the pair form whatever the shape, or an error; 1 / 3 = older
    // forms kept for comparison (one k-block per barrier slot; two k-blocks but one commit per
    // destination CTA), forced likewise.
    {
        const int pair_knob = knob(NNB200_KNOB_I8_PAIR);
        const int64_t pair_tiles = static_cast<int64_t>((m + 2 * kBlockM - 1) / (2 * kBlockM)) * ((n + 255) / 256);
        const bool forced = pair_knob >= 1 && pair_knob <= 3;   // 1, 2, 3: a pair form or an error
        const int64_t pairs = dev.sm_count / 2 > 0 ? dev.sm_count / 2 : 1;
        const bool pair_waves_full = pair_tiles * 4 >= ((pair_tiles + pairs - 1) / pairs) * pairs * 3;
        const bool mn = a_mn || w_mn;   // MN-major operands: the default pair form only (knob 1 / 3: K-major)
        if (forced && (sharded || (mn && pair_knob != 2))) {
            return NNB200_UNSUPPORTED;
        }
        if (pair_knob != 0 && !sharded &&
            (forced || (m >= 2 * kBlockM && k >= 2048 && pair_tiles >= 24 &&
                        (pair_tiles <= pairs || bn == 256 || pair_waves_full)))) {
            const int pose = (a_mn ? 1 : 0) | (w_mn ? 2 : 0);
            const int st = pair_knob == 1   ? launch_pair_bn<256, 1, false>(p, ep, m, n, k, a_fmt, vec_ok, dev, stream)
                           : pair_knob == 3 ? launch_pair_bn<256, 2, false>(p, ep, m, n, k, a_fmt, vec_ok, dev, stream)
                           : pose == 1      ? launch_pair_bn<256, 2, true, 1>(p, ep, m, n, k, a_fmt, vec_ok, dev, stream)
                           : pose == 2      ? launch_pair_bn<256, 2, true, 2>(p, ep, m, n, k, a_fmt, vec_ok, dev, stream)
                           : pose == 3      ? launch_pair_bn<256, 2, true, 3>(p, ep, m, n, k, a_fmt, vec_ok, dev, stream)
                                            : launch_pair_bn<256, 2, true>(p, ep, m, n, k, a_fmt, vec_ok, dev, stream);
            if (st != NNB200_UNSUPPORTED || forced) {
                return st;
            }
        }
    }
    switch (bn) {
    case 512:
        return launch_bn<512>(ep.out_kind, map_a, map_w, ep, m, n, k, idesc_of(256), vec_ok,
                              dev, stream);
    case 448:
        return launch_bn<448>(ep.out_kind, map_a, map_w, ep, m, n, k, idesc_of(224), vec_ok,
                              dev, stream);
    case 384:
        return launch_bn<384>(ep.out_kind, map_a, map_w, ep, m, n, k, idesc_of(192), vec_ok,
                              dev, stream);
    case 320:
        return launch_bn<320>(ep.out_kind, map_a, map_w, ep, m, n, k, idesc_of(160), vec_ok,
                              dev, stream);
    case 256:
        return launch_bn<256>(ep.out_kind, map_a, map_w, ep, m, n, k, idesc_of(256), vec_ok,
                              dev, stream);
    case 224:
        return launch_bn<224>(ep.out_kind, map_a, map_w, ep, m, n, k, idesc_of(224), vec_ok,
                              dev, stream);
    case 192:
        return launch_bn<192>(ep.out_kind, map_a, map_w, ep, m, n, k, idesc_of(192), vec_ok,
                              dev, stream);
    case 128:
        return launch_bn<128>(ep.out_kind, map_a, map_w, ep, m, n, k, idesc_of(128), vec_ok,
                              dev, stream);
    default:
        return launch_bn<64>(ep.out_kind, map_a, map_w, ep, m, n, k, idesc_of(64), vec_ok,
                             dev, stream);
    }
}

}  // namespace nnb200
