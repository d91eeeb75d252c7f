/*
 * nnb200 -- C ABI of the B200 (sm_100a) quantized-matmul backend for nnops.
 *
 * Every entry point takes plain pointers and sizes; all data pointers are DEVICE pointers
 * of the current CUDA device unless a comment says otherwise.  Calls enqueue work on the
 * given stream (a cudaStream_t passed as void*, NULL = default stream) and return without
 * synchronising.  Return values use the numbering of nnops::Status
 * (reference include/nnops/core/status.hpp:19-33).  A call refused for its arguments
 * (INVALID_ARGUMENT, UNSUPPORTED, OUT_OF_MEMORY) has launched nothing and written nothing to its
 * outputs.  INTERNAL reports a CUDA launch failure; with batch > 1 earlier batch elements may
 * have been enqueued by then.  Pointers must be naturally aligned for what they point at
 * (4 bytes for int32 / float arrays, 2 for f16, 16 for a workspace); a misaligned one is
 * INVALID_ARGUMENT.
 */
#ifndef NNB200_H
#define NNB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define NNB200_API __attribute__((visibility("default")))
#else
#define NNB200_API
#endif

#define NNB200_OK 0
#define NNB200_INVALID_ARGUMENT 1
#define NNB200_UNSUPPORTED 2
#define NNB200_NOT_INITIALIZED 3
#define NNB200_OUT_OF_MEMORY 4
#define NNB200_INTERNAL 5

/* Destination kinds of the int8 route (reference I8OutKind,
 * src/backend/cuda/matmul/matmul_i8_common.cuh:38-58). */
#define NNB200_OUT_S32 0
#define NNB200_OUT_S8 1
#define NNB200_OUT_U8 2
#define NNB200_OUT_F32 3
#define NNB200_OUT_F16 4

/* Activation codes = nnops::EpilogueActivateType (include/nnops/core/epilogue.hpp:23-34). */
#define NNB200_ACT_NONE 0
#define NNB200_ACT_RELU 1
#define NNB200_ACT_GELU 2
#define NNB200_ACT_SIGMOID 3
#define NNB200_ACT_TANH 4
#define NNB200_ACT_LEAKY_RELU 5
#define NNB200_ACT_SILU 6
#define NNB200_ACT_HARD_SWISH 7
#define NNB200_ACT_ELU 8
#define NNB200_ACT_RELU6 9

/* Engines, for nnb200_gemm_i8_args.force_engine and the *_engine_name queries. */
#define NNB200_ENGINE_AUTO 0
#define NNB200_ENGINE_UMMA 1    /* TMA + tcgen05.mma kind::i8, TMEM accumulators           */
#define NNB200_ENGINE_NARROW 2  /* M <= 16 decode, any K: one warp per channel, dp4a        */
#define NNB200_ENGINE_GENERIC 3 /* any pose / alignment: SIMT tile, correctness tier        */
#define NNB200_ENGINE_DECODE 4  /* M <= 16, K % 64 == 0: streaming loads + warp MMA        */
#define NNB200_ENGINE_SKINNY 5  /* M <= 128: tcgen05 with the weights as the 128-row operand */

/*
 * One int8 matmul call: out[b][m][n] = epilogue( sum_k A[b][m][k] * W[b][n][k] ).
 * Replaces the parameter block the reference launcher takes
 * (GemmI8Params, src/backend/cuda/matmul/matmul_i8_common.cuh:69-112, filled by
 * linear_i8_cuda src/backend/cuda/matmul/linear.cu:27-90 and matmul_i8_cuda
 * src/backend/cuda/matmul/matmul.cu:35-95).
 *
 * Strides are in ELEMENTS.  The Linear pose is a_stride_k == 1 and w_stride_k == 1
 * (A [M,K] and W [N,K], both k-contiguous); MatMul's transposes are expressed by
 * swapping which stride is 1.  batch_stride 0 broadcasts that operand over the batch.
 *
 * Integer destinations (S32/S8/U8): v = raw - zp_a*R_w[n] - zp_w*R_a[m] + K*zp_a*zp_w
 * (+ int32 bias[n]) (Relu if relu != 0); S8/U8 then requantise with
 * req = (scale_a[m] / out_scale) * scale_w[n], x = float(v) * req, clamp to the type's
 * range minus out_zp, round half away from zero as trunc(x + copysign(0.5, x)), add out_zp.
 * fp destinations (F32/F16): f = float(v) * (scale_a[m]*scale_w[n]) (+ fp bias[n] if
 * non-zero), clamp to [min_clip, max_clip], activation.
 *
 * scale_a / zp_a are per row m (NULL -> the *_scalar value), scale_w / zp_w per output
 * channel n.  For a batched call the same arrays serve every batch element.
 *
 * workspace: nnb200_gemm_i8_workspace_bytes() bytes of 16-byte aligned device scratch (may be
 * NULL when that is 0).  It holds the row/column sums R_a, R_w when any zero point is non-zero
 * and, for calls of up to 128 activation rows that the weights-as-rows tensor-core engine
 * serves, the partial sums and arrival counters with which that engine shares K evenly among
 * all SMs.  Only the first part is required: a workspace of at least
 * nnb200_gemm_i8_min_workspace_bytes() is accepted, and the call then runs with whole tiles
 * per SM (same results, slower when N / 128 does not fill the SMs evenly).
 */
typedef struct nnb200_gemm_i8_args {
    const void* a;
    const void* w;
    void* out;
    int64_t m, n, k;
    int64_t a_stride_m, a_stride_k;
    int64_t w_stride_n, w_stride_k;
    int64_t ldc;
    int64_t batch;
    int64_t a_batch_stride, w_batch_stride, out_batch_stride;
    int32_t a_unsigned; /* A holds u8 instead of s8 */
    int32_t out_kind;   /* NNB200_OUT_* */
    const void* bias;   /* [n]: int32 for integer destinations, out type for fp ones; may be NULL */
    int32_t relu;       /* integer destinations honour only Relu */
    int32_t activation; /* NNB200_ACT_*, fp destinations */
    float act_alpha, act_beta;
    float min_clip, max_clip;
    const float* scale_a;
    const float* scale_w;
    const int32_t* zp_a;
    const int32_t* zp_w;
    float scale_a_scalar, scale_w_scalar;
    int32_t zp_a_scalar, zp_w_scalar;
    int32_t zp_a_nonzero; /* caller's promise about the ARRAYS: 0 = every zp_a[] entry is 0 */
    int32_t zp_w_nonzero; /* (lets the backend skip the R_a / R_w sweeps); scalars are checked here */
    float out_scale;
    int32_t out_zp;
    void* workspace;
    size_t workspace_bytes;
    int32_t force_engine; /* NNB200_ENGINE_*; AUTO picks */
    /* Column-sharded layers: besides `out`, write the same [m, n] window (same ldc) into up to
     * seven more buffers -- the other GPUs' copies of the full output, mapped into this process
     * (CUDA IPC / peer access).  The GEMM's write-back then IS the all-gather.  S8/U8
     * destinations on the tensor-core engine only, batch 1, every pointer and ldc a multiple of
     * 16, n a multiple of 16; otherwise NNB200_UNSUPPORTED.  The caller orders the ranks (all
     * ranks' kernels must finish before any rank reads its buffer).  The reference has no
     * multi-GPU path; this has no counterpart there. */
    int32_t num_peer_outs;
    void* peer_out[7];
    /* Optional: sum_k W[n][k] per channel, already on the device (the r_w section of a packed
     * weight, see nnb200_i8_pack).  A call that needs zero-point compensation then skips its
     * sweep over W.  Single-batch weights only (w_batch_stride == 0 or batch == 1). */
    const int32_t* r_w;
    /* Optional, column-sharded layers on GPUs behind an NVSwitch: the address of this call's
     * [m, n] output window (same ldc) inside a MULTICAST mapping that is bound to every rank's
     * copy of the full output, this rank's included.  Each finished tile is then stored once
     * with multimem.st and the switch replicates it to all copies, instead of one store per
     * destination: `out` and peer_out[] are not written (num_peer_outs must be 0; `out` must
     * still name this rank's own window, it decides alignment and pitch).  Same conditions as
     * peer_out.  The address must come from a multicast object (cuMulticastCreate /
     * cuMulticastBindMem, or a library that wraps them): anything else is not a valid operand
     * of the instruction.  No counterpart in the reference. */
    void* multicast_out;
} nnb200_gemm_i8_args;

/* Scratch the call runs fastest with (0 for the common zero-point-free tensor-core call), and
 * the least it accepts. */
NNB200_API size_t nnb200_gemm_i8_workspace_bytes(const nnb200_gemm_i8_args* args);
NNB200_API size_t nnb200_gemm_i8_min_workspace_bytes(const nnb200_gemm_i8_args* args);

/* Enqueue the matmul.  Replaces dense_gemm_i8_status
 * (src/backend/cuda/matmul/matmul_i8.cuh:284-446). */
NNB200_API int nnb200_gemm_i8(const nnb200_gemm_i8_args* args, void* stream);

/*
 * Same computation as nnb200_gemm_i8 for callers that may not allocate device memory and so
 * have no workspace to pass: a plugin inside an inference runtime, or any code on a
 * latency-critical path, where cudaMalloc is off limits because it serialises the device and
 * can fail at run time.  The scratch the zero-point-compensated call needs (the int32 row sums
 * of A and W) is kept in a fixed array of NNB200_STATIC_SCRATCH_BYTES inside the library, in
 * the memory of every GPU that loads it, for the life of the process.  args->workspace is
 * ignored.  This entry point has no counterpart in the reference, whose launcher always
 * allocates from its own pool (src/backend/cuda/matmul/gemm_common.cuh:296-340).
 *
 *  - Needs more than NNB200_STATIC_SCRATCH_BYTES (batch * (4*m + 4*n), each term rounded up
 *    to 256): returns NNB200_OUT_OF_MEMORY and launches nothing.
 *  - Never calls cudaMalloc, cudaFree or any allocating routine.
 *  - The first call on each device looks up that device's copy of the array; make that first
 *    call with the device current and outside any stream capture.
 *  - All calls on a device share the one array.  Nothing in it has to be zeroed between
 *    calls (every entry read is written first), but two calls whose kernels may overlap on
 *    the GPU -- different streams, no ordering between them -- race on it: serialise them.
 */
#define NNB200_STATIC_SCRATCH_BYTES (1 << 20)
NNB200_API int nnb200_gemm_i8_static_scratch(const nnb200_gemm_i8_args* args, void* stream);

/*
 * int8 Conv2D: a pre-quantised u8/s8 NHWC activation against an s8 HWIO filter, output NHWC.
 * Replaces conv2d_i8_cuda (src/backend/cuda/conv/conv2d_i8.cu:910-1100; kernel :358-785) and
 * the packed-filter pair conv_i8_packed_weight_desc / conv_i8_packed_weight_pack
 * (src/backend/cuda/conv/conv2d_pack.h:30-37).
 *
 * out[n][oh][ow][oc] = epilogue( sum_{kh,kw,c} x[n][oh*sh - ph + kh*dh][ow*sw - pw + kw*dw][g*IC/G + c]
 *                                              * w[kh][kw][c][oc] ),  g = oc / (OC/G),
 * where a tap outside the image holds the activation's zero point (the real value 0) and the
 * epilogue is nnb200_gemm_i8's with K = kh*kw*IC/G, a per-tensor activation (scale_x, zp_x) and
 * per-channel or per-tensor filter parameters: integer destinations S8/U8 (compensation, int32
 * bias, Relu, requantisation), fp destinations F32/F16 (dequantisation, fp bias, clip,
 * activation).  An S32 destination answers NNB200_UNSUPPORTED, as in the reference.
 *
 * pad_h / pad_w are the leading paddings and oh / ow are given by the caller (an auto-padded
 * convolution pads the trailing edge differently); an extent whose last window would start more
 * than the leading padding plus one filter span past the image answers NNB200_INVALID_ARGUMENT.
 *
 * Strides are in ELEMENTS.  The output's channel stride is 1 and its pixels lie at one pitch:
 * out_stride_h == ow * out_stride_w and, for batch > 1, out_stride_n == oh * out_stride_h
 * (otherwise NNB200_UNSUPPORTED).  weight_packed != 0: `weight` is a blob written by
 * nnb200_conv2d_i8_pack for the same kh, kw, IC/G, oc and groups (16-byte aligned); the filter
 * strides are then ignored and the per-call filter pass is skipped.
 *
 * workspace: nnb200_conv2d_i8_workspace_bytes() bytes of 16-byte aligned device scratch: the
 * gathered activation [groups][pixels][K rounded up to 16] (none for a 1x1, stride-1, unpadded
 * convolution over a dense activation, which the GEMM reads in place), the k-major filter and
 * its channel sums (none with a packed filter), and the GEMM's own scratch.
 */
typedef struct nnb200_conv2d_i8_args {
    const void* input;
    const void* weight;
    void* out;
    int64_t batch, ih, iw, ic;
    int64_t oh, ow, oc;
    int64_t kh, kw, stride_h, stride_w, dil_h, dil_w, pad_h, pad_w, groups;
    int64_t in_stride_n, in_stride_h, in_stride_w, in_stride_c;
    int64_t w_stride_kh, w_stride_kw, w_stride_ic, w_stride_oc;
    int64_t out_stride_n, out_stride_h, out_stride_w;
    int32_t weight_packed;
    int32_t a_unsigned;   /* the activation holds u8 instead of s8 */
    int32_t out_kind;     /* NNB200_OUT_S8 / U8 / F32 / F16 */
    const void* bias;     /* [oc]: int32 for integer destinations, out type for fp ones; may be NULL */
    int32_t relu;
    int32_t activation;   /* NNB200_ACT_*, fp destinations */
    float act_alpha, act_beta;
    float min_clip, max_clip;
    const float* scale_w;   /* [oc] on the device, or NULL -> scale_w_scalar */
    const int32_t* zp_w;    /* [oc] on the device, or NULL -> zp_w_scalar */
    float scale_x, scale_w_scalar;
    int32_t zp_x, zp_w_scalar;
    int32_t zp_w_nonzero;   /* 0 = every zp_w[] entry is 0 (skips the activation row sums) */
    float out_scale;
    int32_t out_zp;
    void* workspace;
    size_t workspace_bytes;
} nnb200_conv2d_i8_args;

NNB200_API size_t nnb200_conv2d_i8_workspace_bytes(const nnb200_conv2d_i8_args* args);
NNB200_API int nnb200_conv2d_i8(const nnb200_conv2d_i8_args* args, void* stream);

/* Packed filter: rows [oc][K rounded up to 16] with k contiguous (k = (kh*KW + kw)*IC/G + c),
 * then, 256-byte aligned, the int32 sum of each row.  pack_bytes is the allocation. */
NNB200_API size_t nnb200_conv2d_i8_pack_bytes(int64_t kh, int64_t kw, int64_t ic_per_group, int64_t oc);
NNB200_API int nnb200_conv2d_i8_pack(const void* weight, int64_t w_stride_kh, int64_t w_stride_kw,
                                     int64_t w_stride_ic, int64_t w_stride_oc, int64_t kh, int64_t kw,
                                     int64_t ic_per_group, int64_t oc, int64_t groups, void* blob, void* stream);

/*
 * Measurement aid: the int8 tensor rate of this GPU.  Enqueues one launch in which every SM
 * issues iters groups of four tcgen05.mma kind::i8 M128 x N256 x K32 (the int8 GEMM's own
 * instruction) on operand tiles resident in shared memory, with no loads, stores or epilogue;
 * pattern 0 fills the tiles with zeros (the pipe's issue rate), 1 with pseudo-random bytes (the
 * rate the power cap allows once the operands toggle); adding 2 runs the CTA-pair form of the
 * instruction (cta_group::2, M256 over two SMs, each holding half of the W tile).  *ops receives the integer operations
 * the launch performs (2 per multiply-add).  The caller times the launch with events on the
 * stream: ops / time is the denominator the GEMM's roofline fraction is quoted against.
 * 1 <= iters <= 2^21.  No counterpart in the reference.
 */
NNB200_API int nnb200_measure_i8_mma_peak(int32_t iters, int32_t pattern, double* ops, void* stream);

/*
 * Measurement and test switches: process-wide integers, in the manner of the reference's bench
 * knobs (src/detail/bench_knobs.hpp:15-38).  They only select among code paths that give
 * identical results; production code leaves them alone.  A negative value means "default".
 * The environment is never read.  nnb200_set_knob returns the previous value (or
 * INT32_MIN for an unknown knob).
 *   GROUP_M          raster group (m-blocks) of the int8 tensor-core GEMM
 *   I8_BN            force its tile width: 64, 128, 192, 224, 256, 320, 384, 448 or 512
 *   I8_PAIR          0 single-CTA form only, 2 CTA-pair form whatever the shape, or an error (default: pair form
 *                    where it pays);
 *                    1 / 3 earlier pair forms kept for comparison (one k-block per barrier slot / two commits);
 *                    0 also keeps the implicit-GEMM convolution on single CTAs
 *   I8_PEER_STAGING  1 / 2 staging tiles per epilogue warp in the sharded write-back
 *   F16_PAIR         as I8_PAIR for the dense f16 GEMM of the Q4_1 two-pass form
 *   I8_SHARE_K       0 never share K among SMs in the few-row engine, 2 offer it from 8 K blocks per SM
 *   Q4_GEMV          Q4_1 GEMV engine of the automatic choice: 1 never the deferred-scaling kernel, 2 that
 *                    kernel whenever it can run (default: for a single activation row)
 *   CONV_FORM        1 = nnb200_conv2d_i8 never takes its implicit-GEMM form (gather pass + GEMM always),
 *                    2 = that form wherever it can run, small and heavily padded planes included
 *   I8_K_ROTATE      tile t of the int8 tensor-core GEMM starts its walk over the 128-byte K blocks at block
 *                    (t * value) mod blocks; 0 = every tile at block 0 (default: 5 up to 4096 weight rows, else 0)
 */
#define NNB200_KNOB_GROUP_M 0
#define NNB200_KNOB_I8_BN 1
#define NNB200_KNOB_I8_PAIR 2
#define NNB200_KNOB_I8_PEER_STAGING 3
#define NNB200_KNOB_F16_PAIR 4
#define NNB200_KNOB_I8_SHARE_K 5
#define NNB200_KNOB_Q4_GEMV 6
#define NNB200_KNOB_CONV_FORM 7
#define NNB200_KNOB_I8_K_ROTATE 8
#define NNB200_KNOB_COUNT 9
NNB200_API int nnb200_set_knob(int knob, int value);
NNB200_API int nnb200_get_knob(int knob);

/* Which engine nnb200_gemm_i8 would run for these arguments (NNB200_ENGINE_*), the workspace the
 * block carries included: with enough of it some few-row calls move to the weights-as-rows engine. */
NNB200_API int nnb200_gemm_i8_engine(const nnb200_gemm_i8_args* args);

/*
 * Q4_1 weight-decode product: out[m][n] = act( alpha * sum_k A[m][k] * dequant(W)[n][k]
 * + bias[n] ), W stored as llama.cpp Q4_1 rows: ceil(k/32) blocks of 20 bytes
 * {f16 d, f16 m, 16 nibble bytes; low nibble = value j, high nibble = value j+16; w = d*q+m}
 * (reference include/nnops/detail/q4_1.hpp:53-79).  Replaces the CPU-only routes
 * matmul_qblock_fused (src/backend/cpu/matmul/matmul_qblock_fused.cpp:151-197) and the packed
 * route (src/backend/cpu/matmul/matmul.cpp:137-156); the reference has no CUDA kernel for it
 * (src/backend/cuda/matmul/linear.cu:116-119 returns unsupported).
 *
 * a_f16 / out_f16: 1 = IEEE half, 0 = float.  Reference poses are f16->f16 and f32->f32;
 * f16 activations with f32 output is accepted as an extension.  lda / ldc in elements,
 * ldw_blocks in 20-byte blocks.
 */
typedef struct nnb200_q4_1_args {
    const void* a;
    const void* w_blocks;
    void* out;
    int64_t m, n, k;
    int64_t lda, ldw_blocks, ldc;
    int32_t a_f16, out_f16;
    const void* bias; /* [n] in the output type; may be NULL */
    int32_t activation;
    float act_alpha, act_beta;
    float min_clip, max_clip;
    float alpha;
    void* workspace;
    size_t workspace_bytes;
    int32_t force_engine; /* 0 auto, 1 fused tensor-core GEMM, 2 GEMV (best), 3 GEMV on CUDA cores, 4 GEMV with
                             warp MMA after per-weight dequantisation, 5 two-pass GEMM (needs the workspace),
                             6 GEMV with warp MMA on raw nibbles, scale and minimum applied per block afterwards */
    int32_t flags;        /* NNB200_Q4_FLAG_* */
    /* Prepacked weights (nnb200_q4_1_pack): when w_dm is not NULL, w_blocks points at the nibble
     * plane -- 16 bytes per block, ldw_blocks still counted in blocks -- and w_dm at the plane of
     * (f16 d, f16 m) pairs, 4 bytes per block, rows ld_dm blocks apart.  Served by the GEMV
     * engine with deferred scaling and by the two-pass GEMM; other shapes of call answer
     * NNB200_UNSUPPORTED. */
    const void* w_dm;
    int64_t ld_dm;
} nnb200_q4_1_args;

/* The launch may begin while the preceding kernel of the stream is still finishing
 * (programmatic dependent launch): its weight fetch overlaps that kernel's tail; activations
 * are read and outputs written only after that kernel has completed.  Only set this when
 * the preceding kernel does not write w_blocks.  Honoured by the GEMV engine. */
#define NNB200_Q4_FLAG_OVERLAP_PREVIOUS 1

/* Optional device scratch (16-byte aligned).  Non-zero for tall problems (f16 activations: m >= 256;
 * f32 activations: m >= 17): given that many bytes, the call expands the weights to f16 once into
 * the scratch (and splits f32 activations into [hi | lo] f16 halves there) and runs a dense
 * tensor-core GEMM over them; without it (NULL or too small) the same call runs the fused kernel
 * (f16) or the GEMV engine tile by tile (f32).  The scratch is dead when the call's work has
 * completed on the stream. */
NNB200_API size_t nnb200_q4_1_workspace_bytes(const nnb200_q4_1_args* args);
NNB200_API int nnb200_linear_q4_1(const nnb200_q4_1_args* args, void* stream);
NNB200_API int nnb200_q4_1_engine(const nnb200_q4_1_args* args);

/* Decode `rows` Q4_1 rows of `k` values into f32 (out_f16 == 0) or f16, ld in elements.
 * Device twin of pack_q4 (include/nnops/detail/q4_1.hpp:152-184). */
NNB200_API int nnb200_q4_1_decode(const void* w_blocks, int64_t ldw_blocks, int64_t rows, int64_t k, void* out,
                       int32_t out_f16, int64_t ld_out, void* stream);

/*
 * Prepacked int8 weights -- the device blob behind the operators' two-step prepackWeights
 * contract (reference include/nnops/core/op_base.hpp:72-80).  The reference's CUDA operators
 * answer "no packed form" (src/ops/linear.cpp:125-128); with a blob a call stages no per-channel
 * array and, when activation zero points are in play, does not sweep W a second time.
 *
 * Blob = nnb200_i8_pack_bytes(n, k) = n * (pitch + 12) bytes, pitch = k rounded up to 16:
 * W as [n][pitch] s8 k-contiguous and zero padded (whatever pose the source had), then scale_w[n]
 * f32, zp_w[n] s32, r_w[n] s32 (sum_k W[n][k]).  nnb200_i8_packed_view only does the pointer
 * arithmetic.  w is device memory; scale_w / zp_w may be host or device arrays or NULL (then the
 * scalar fills the section).  blob must be 16-byte aligned device memory.
 */
typedef struct nnb200_i8_packed {
    const void* w;        /* [n][pitch] s8; use with w_stride_n = pitch, w_stride_k = 1 */
    int64_t pitch;
    const float* scale_w; /* [n] */
    const int32_t* zp_w;  /* [n] */
    const int32_t* r_w;   /* [n] */
} nnb200_i8_packed;

NNB200_API size_t nnb200_i8_pack_bytes(int64_t n, int64_t k);
NNB200_API int nnb200_i8_pack(const void* w, int64_t n, int64_t k, int64_t w_stride_n, int64_t w_stride_k,
                              const float* scale_w, float scale_w_scalar, const int32_t* zp_w, int32_t zp_w_scalar,
                              void* blob, size_t blob_bytes, void* stream);
NNB200_API int nnb200_i8_packed_view(const void* blob, int64_t n, int64_t k, nnb200_i8_packed* view);

/*
 * Prepacked Q4_1 weights: the raw llama.cpp stream interleaves a 4-byte (d, m) header with 16
 * nibble bytes, so a block is only 4-byte aligned and no load wider than 32 bits can be aimed
 * at it.  The packed form separates the two: a nibble plane [n][row of ceil(k/32) 16-byte
 * entries] whose every block is 16-byte aligned, then a (d, m) plane [n][ceil(k/32) 4-byte
 * entries]; both row pitches are rounded up to 16 bytes.  Same 20 bytes per block in total, so
 * the bytes a product moves are unchanged.  This is the "Q4_1 repacked into separated scale
 * and nibble planes" form of the operators' two-step prepackWeights contract (reference
 * include/nnops/core/op_base.hpp:72-80; its CUDA front end answers "no packed form",
 * src/ops/linear.cpp:125-128).  One-time cost, a pure re-layout: decoding the planes gives the
 * same values bit for bit.
 */
typedef struct nnb200_q4_1_packed {
    const void* qs;     /* nibble plane */
    int64_t qs_pitch;   /* its row pitch in 16-byte blocks */
    const void* dm;     /* (d, m) plane */
    int64_t dm_pitch;   /* its row pitch in 4-byte entries */
} nnb200_q4_1_packed;

NNB200_API size_t nnb200_q4_1_pack_bytes(int64_t n, int64_t k);
NNB200_API int nnb200_q4_1_pack(const void* w_blocks, int64_t ldw_blocks, int64_t n, int64_t k, void* blob,
                                size_t blob_bytes, void* stream);
NNB200_API int nnb200_q4_1_packed_view(const void* blob, int64_t n, int64_t k, nnb200_q4_1_packed* view);

/*
 * QuantizeLinear / DequantizeLinear (reference operators include/nnops/ops/quant_linear.hpp:24-141;
 * these two calls stand where the reference's CUDA entry points quantize_linear_cuda /
 * dequantize_linear_cuda are Status::unsupported stubs, src/backend/cuda/not_implemented.cu:28-37;
 * the arithmetic is the one of its CPU route, src/backend/cpu/quant_linear.cpp:80-262).
 *
 * The dense tensor is viewed as [outer][rows][inner]; scale[r] / zero_point[r] serve row r of
 * every outer group: per tensor = [1][1][numel], per token = [1][numel/last][last], per channel
 * (axis a) = [prod(shape[:a])][shape[a]][prod(shape[a+1:])].  x, y, scale and zero_point are
 * device pointers; the floating side is f32 or f16, the integer side s8 or u8, the zero point
 * s8, u8 or int32 on its own flag.
 *   quantize:   y = saturate(round_half_even(fma(x, 1/scale, zero_point)))
 *   dequantize: y = (x - zero_point) * scale   (rounded as the reference's kernels round it)
 */
#define NNB200_ZP_S8 0
#define NNB200_ZP_U8 1
#define NNB200_ZP_S32 2 /* the int32 zero points of a view's QuantParams (fp-activation route) */

typedef struct nnb200_quant_linear_args {
    const void* x;
    void* y;
    int64_t outer, rows, inner;
    const float* scale;     /* [rows] */
    const void* zero_point; /* [rows], s8 or u8 */
    int32_t zp_unsigned;    /* NNB200_ZP_*: storage type of zero_point */
    int32_t float_f16;      /* floating side (x of quantize, y of dequantize) is f16, else f32 */
    int32_t int_unsigned;   /* integer side (y of quantize, x of dequantize) is u8, else s8 */
} nnb200_quant_linear_args;

NNB200_API int nnb200_quantize_linear(const nnb200_quant_linear_args* args, void* stream);
NNB200_API int nnb200_dequantize_linear(const nnb200_quant_linear_args* args, void* stream);

/*
 * Column-sharded Linear, reassembly step: `gathered` holds `shards` dense slabs
 * [shards][m][row_bytes_per_shard] (what an all-gather of per-rank [m, n/shards] outputs
 * produces); writes the row-major [m][shards*row_bytes_per_shard] matrix with row pitch
 * out_pitch_bytes.  All sizes and pointers must be 16-byte multiples.  No counterpart in the
 * reference, which has no multi-GPU code.
 */
NNB200_API int nnb200_interleave_shards(const void* gathered, void* out, int64_t m, int64_t row_bytes_per_shard,
                                        int32_t shards, int64_t out_pitch_bytes, void* stream);

/*
 * Device-side barrier among the GPUs of one node, for ordering the ranks after the sharded
 * write-back without a collective: flags_by_rank[r] is rank r's flag array -- NNB200_RANK_FLAG_BYTES
 * bytes from nnb200_peer_buffer_alloc, zeroed once, rank r's own for r == rank and the mapping
 * from nnb200_peer_buffer_open for the others.  The kernel (one warp) advances this rank's
 * epoch, which lives in its flag array so that a captured launch stays valid on replay, writes
 * it into every other rank's array and polls its own array until every other rank has done the
 * same.  Every rank must call it the same number of times.  Work enqueued on the stream after
 * it sees everything the other ranks' streams had completed before their call.  The wait is
 * bounded by limit_cycles SM clock cycles (0 = the library's default, about half a minute:
 * ranks of one job drift apart by seconds for ordinary reasons): when it runs out the kernel
 * records code 8 in the error word and sets a sticky host-visible flag for this device, and
 * returns.  From then on the outputs gathered on this device are not to be trusted, and every
 * later nnb200_rank_barrier, and every nnb200_gemm_i8 with peer outputs, on this device returns
 * NNB200_INTERNAL without launching anything, until nnb200_take_device_error has been called
 * (it reports code 8 and clears the flag).  A sharded output is valid only if the error word
 * read after it is 0.  The first call on a device allocates 64 bytes of pinned host memory
 * for that flag: make it outside any stream capture.  world <= 8.  No counterpart in the
 * reference, which has no multi-GPU code.
 */
#define NNB200_RANK_FLAG_BYTES 64
#define NNB200_DEVICE_ERROR_PEER_WAIT 8
NNB200_API int nnb200_rank_barrier(int32_t* const* flags_by_rank, int32_t world, int32_t rank, int64_t limit_cycles,
                                   void* stream);

/*
 * Kernels never spin forever: a pipeline wait that runs out records a code in a per-device
 * error word and the kernel exits.  This synchronises the device, returns that word through
 * *code (0 = no error) and clears it.
 */
NNB200_API int nnb200_take_device_error(int32_t* code);

/*
 * Exercises that mechanism without disturbing anything: launches one thread that waits, for
 * at most limit_cycles SM clock cycles (1 .. 2e8), on a barrier nothing arrives at.  The wait
 * runs out, the kernel records NNB200_DEVICE_ERROR_SELFTEST (7) in the error word and returns
 * normally; the context stays usable.  The next nnb200_take_device_error reports the code.
 */
#define NNB200_DEVICE_ERROR_SELFTEST 7
NNB200_API int nnb200_selftest_wait_limit(int64_t limit_cycles, void* stream);

/* Stage a host array into device memory on the stream (the reference launcher's per-call
 * H2D of quantization arrays, src/backend/cuda/matmul/matmul_i8.cuh:357-376). */
NNB200_API int nnb200_copy_h2d_async(void* dst_device, const void* src_host, size_t bytes, void* stream);

/* Stream-ordered scratch from the device's default memory pool, for host glue that has to
 * stage host-side quantization arrays itself (the reference launcher's private pool,
 * gemm_workspace_alloc / gemm_workspace_free, src/backend/cuda/matmul/gemm_common.cuh:296-354). */
NNB200_API int nnb200_scratch_alloc_async(void** out, size_t bytes, void* stream);
NNB200_API int nnb200_scratch_free_async(void* p, void* stream);

/*
 * Output buffers that other processes' GPUs can store into (the peer_out pointers of
 * nnb200_gemm_i8_args).  alloc: plain device memory on the current device (this is the one
 * place the library allocates on request; free it with nnb200_peer_buffer_free).  export: a
 * 64-byte CUDA IPC handle to send to the other ranks.  open: map another rank's buffer for the
 * CURRENT device -- call it with the device that will run the kernels current; returns
 * NNB200_UNSUPPORTED when the two GPUs have no peer path.  close: unmap.  No counterpart in the
 * reference.
 */
NNB200_API int nnb200_peer_buffer_alloc(void** ptr, size_t bytes);
NNB200_API int nnb200_peer_buffer_free(void* ptr);
NNB200_API int nnb200_peer_buffer_export(const void* ptr, uint8_t handle[64]);
NNB200_API int nnb200_peer_buffer_open(const uint8_t handle[64], void** ptr);
NNB200_API int nnb200_peer_buffer_close(void* ptr);

/* Let kernels of the current device store into memory of `peer_device` (needed once per pair
 * before nnb200_gemm_i8 is given peer_out pointers).  NNB200_UNSUPPORTED if the two GPUs have
 * no peer path. */
NNB200_API int nnb200_enable_peer_access(int32_t peer_device);

/* 1 if p is device (or managed) memory usable by kernels of the current device, else 0. */
NNB200_API int nnb200_is_device_pointer(const void* p);

/* Count of kernel launches this process has enqueued through this library. */
NNB200_API uint64_t nnb200_launch_count(void);

NNB200_API const char* nnb200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* NNB200_H */
