/*
 * CPU restatement of the nnops quantized-matmul path.  TEST INFRASTRUCTURE ONLY:
 * the shipped CUDA path never links, loads or calls this file; it exists so the
 * parity tests and the bench's cpu_baseline leg have a checker that runs anywhere
 * gcc does.
 *
 * Parity pin: every function below is checked (tests/test_oracle.py) against the
 * hand-computed vectors of the reference's own tests
 *   tests/test_matmul_int8.cpp:106-285   (s32, zero points, u8 A, requant = 5, clamp = 127)
 *   tests/test_q4_1.cpp:175-260          (block layout / decode)
 * and, where the reference's CPU route was compiled (oracle/_ref), against its
 * outputs on seeded random tensors stored under tests/golden/.
 *
 * Each function cites the reference file:line whose arithmetic it restates.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- IEEE half <-> float (reference: include/nnops/detail/half.hpp; RNE) ---- */

float oracle_f16_to_f32(uint16_t h)
{
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t oracle_f32_to_f16(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    x &= 0x7FFFFFFFu;
    if (x >= 0x7F800000u) {                       /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((x > 0x7F800000u) ? 0x200u : 0));
    }
    if (x >= 0x477FF000u) {                       /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (x < 0x33000001u) {                        /* < 2^-25 (ties to zero) */
        return sign;
    }
    int32_t e = (int32_t)(x >> 23) - 127;
    uint32_t m = (x & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) {                                /* subnormal half */
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        m &= 0x7FFFFFu;
    }
    uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) {
        ++q;
    }
    return (uint16_t)(sign | (base + q));        /* carry into the exponent is correct */
}

/* ---- Q4_1 codec (reference: include/nnops/detail/q4_1.hpp:53-79,81-150) ---- */

#define Q4_1_BLOCK_ELEMS 32
#define Q4_1_BLOCK_BYTES 20

/* One 20-byte block -> 32 floats: w[j] = d*(qs[j]&15)+m, w[j+16] = d*(qs[j]>>4)+m.
 * The x86 kernels fuse the multiply-add (src/backend/cpu/x86_64/pack_q4_1.hpp:74-77);
 * fmaf reproduces that single rounding. */
void oracle_q4_1_unpack_block(const uint8_t* block, float* out)
{
    uint16_t d_bits, m_bits;
    memcpy(&d_bits, block, 2);
    memcpy(&m_bits, block + 2, 2);
    const float d = oracle_f16_to_f32(d_bits);
    const float m = oracle_f16_to_f32(m_bits);
    const uint8_t* qs = block + 4;
    for (int j = 0; j < 16; ++j) {
        out[j] = fmaf((float)(qs[j] & 0x0F), d, m);
        out[j + 16] = fmaf((float)(qs[j] >> 4), d, m);
    }
}

/* `count` logical values of one row, decoded from ceil(count/32) consecutive blocks. */
void oracle_q4_1_decode_row(const uint8_t* blocks, int64_t count, float* out)
{
    float vals[Q4_1_BLOCK_ELEMS];
    for (int64_t base = 0; base < count; base += Q4_1_BLOCK_ELEMS) {
        oracle_q4_1_unpack_block(blocks + (base / Q4_1_BLOCK_ELEMS) * Q4_1_BLOCK_BYTES, vals);
        const int64_t n = (count - base < Q4_1_BLOCK_ELEMS) ? count - base : Q4_1_BLOCK_ELEMS;
        for (int64_t j = 0; j < n; ++j) {
            out[base + j] = vals[j];
        }
    }
}

/* llama.cpp Q4_1 quantizer as the reference spells it (q4_1.hpp:81-150):
 * d = (max-min)/15, q = min(15, int((x-min)/d + 0.5)); d and min stored as f16. */
void oracle_q4_1_quantize_row(const float* src, int64_t count, uint8_t* blocks)
{
    for (int64_t base = 0; base < count; base += Q4_1_BLOCK_ELEMS) {
        const int n = (int)((count - base < Q4_1_BLOCK_ELEMS) ? count - base : Q4_1_BLOCK_ELEMS);
        const float* x = src + base;
        float vmin = x[0], vmax = x[0];
        for (int j = 1; j < n; ++j) {
            vmin = x[j] < vmin ? x[j] : vmin;
            vmax = x[j] > vmax ? x[j] : vmax;
        }
        const float d = (vmax - vmin) / 15.0f;
        const float id = (d != 0.0f) ? 1.0f / d : 0.0f;
        uint8_t* blk = blocks + (base / Q4_1_BLOCK_ELEMS) * Q4_1_BLOCK_BYTES;
        const uint16_t d_bits = oracle_f32_to_f16(d);
        const uint16_t m_bits = oracle_f32_to_f16(vmin);
        memcpy(blk, &d_bits, 2);
        memcpy(blk + 2, &m_bits, 2);
        uint8_t qs[16] = {0};
        for (int j = 0; j < n; ++j) {
            const float qf = (x[j] - vmin) * id + 0.5f;
            const uint8_t q = (uint8_t)(qf < 15.0f ? (int)qf : 15);
            if (j < 16) {
                qs[j] = q;
            } else {
                qs[j - 16] |= (uint8_t)(q << 4);
            }
        }
        memcpy(blk + 4, qs, 16);
    }
}

/* ---- int8 matmul + fused epilogue --------------------------------------- */

enum { ORACLE_OUT_S32 = 0, ORACLE_OUT_S8 = 1, ORACLE_OUT_U8 = 2, ORACLE_OUT_F32 = 3, ORACLE_OUT_F16 = 4 };

typedef struct oracle_gemm_i8_args {
    const void* a;            /* s8 or u8; element (m,k) at a[m*a_stride_m + k*a_stride_k] */
    const int8_t* w;          /* s8;       element (n,k) at w[n*w_stride_n + k*w_stride_k] */
    void* out;                /* element (m,n) at out + m*ldc + n (elements of out kind)   */
    int64_t m, n, k;
    int64_t a_stride_m, a_stride_k, w_stride_n, w_stride_k, ldc;
    int32_t a_unsigned;
    int32_t out_kind;
    const void* bias;         /* [n]: int32 for integer outputs, f32/f16 for fp outputs     */
    int32_t relu;             /* integer outputs honour only Relu                           */
    const float* scale_a;     /* [m] or NULL -> scale_a_scalar                              */
    const float* scale_w;     /* [n] or NULL -> scale_w_scalar                              */
    const int32_t* zp_a;      /* [m] or NULL -> zp_a_scalar                                 */
    const int32_t* zp_w;      /* [n] or NULL -> zp_w_scalar                                 */
    float scale_a_scalar, scale_w_scalar;
    int32_t zp_a_scalar, zp_w_scalar;
    float out_scale;
    int32_t out_zp;
    float min_clip, max_clip; /* fp outputs only                                            */
} oracle_gemm_i8_args;

/* src/backend/cpu/simd_kernel/simd_epilogue.hpp:129-147 (matmul_int8_requant):
 * f32 product, f32 clamp, x + copysign(0.5, x) in f32, truncate, add zero point. */
static int32_t requant_value(int32_t acc, float req, int32_t zp_out, float lo, float hi)
{
    const float zpf = (float)zp_out;
    volatile float prod = (float)acc * req;      /* volatile: keep the f32 rounding step */
    float x = prod;
    const float lo_b = lo - zpf, hi_b = hi - zpf;
    x = x > lo_b ? x : lo_b;                     /* std::max(x, lo) */
    x = x < hi_b ? x : hi_b;                     /* std::min(.., hi) */
    volatile float biased = x + copysignf(0.5f, x);
    const float r = truncf(biased);
    return (int32_t)r + zp_out;
}

/* Reference: tests/reference/matmul_int8_ref.cpp:109-171 (naive route) and
 * simd_epilogue.hpp:341-467 (row pass).  raw wraps in int32 like the kernels do. */
void oracle_gemm_i8(const oracle_gemm_i8_args* p)
{
    const int8_t* a_s = (const int8_t*)p->a;
    const uint8_t* a_u = (const uint8_t*)p->a;
    const int need_comp = (p->zp_a != NULL) || (p->zp_w != NULL) || p->zp_a_scalar != 0 || p->zp_w_scalar != 0;

    int32_t* r_b = NULL;
    if (need_comp) {
        r_b = (int32_t*)malloc(sizeof(int32_t) * (size_t)(p->n > 0 ? p->n : 1));
        for (int64_t n = 0; n < p->n; ++n) {
            int32_t s = 0;
            for (int64_t k = 0; k < p->k; ++k) {
                s += p->w[n * p->w_stride_n + k * p->w_stride_k];
            }
            r_b[n] = s;
        }
    }
    const int k_contig = (p->a_stride_k == 1 && p->w_stride_k == 1);

#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < p->m; ++m) {
        int32_t r_a = 0;
        if (need_comp) {
            for (int64_t k = 0; k < p->k; ++k) {
                r_a += p->a_unsigned ? (int32_t)a_u[m * p->a_stride_m + k * p->a_stride_k]
                                     : (int32_t)a_s[m * p->a_stride_m + k * p->a_stride_k];
            }
        }
        const int32_t zpa = p->zp_a ? p->zp_a[m] : p->zp_a_scalar;
        const float s_a = p->scale_a ? p->scale_a[m] : p->scale_a_scalar;
        /* simd_epilogue.hpp:353 — f32 division once per row */
        volatile float row_k_v = s_a / p->out_scale;
        const float row_k = row_k_v;
        for (int64_t n = 0; n < p->n; ++n) {
            uint32_t acc = 0;                     /* unsigned: defined wrap-around */
            if (k_contig) {
                const int8_t* wr = p->w + n * p->w_stride_n;
                int32_t s = 0;
                if (p->a_unsigned) {
                    const uint8_t* ar = a_u + m * p->a_stride_m;
                    for (int64_t k = 0; k < p->k; ++k) s += (int32_t)ar[k] * (int32_t)wr[k];
                } else {
                    const int8_t* ar = a_s + m * p->a_stride_m;
                    for (int64_t k = 0; k < p->k; ++k) s += (int32_t)ar[k] * (int32_t)wr[k];
                }
                acc = (uint32_t)s;
            } else {
                for (int64_t k = 0; k < p->k; ++k) {
                    const int32_t av = p->a_unsigned ? (int32_t)a_u[m * p->a_stride_m + k * p->a_stride_k]
                                                     : (int32_t)a_s[m * p->a_stride_m + k * p->a_stride_k];
                    acc += (uint32_t)(av * (int32_t)p->w[n * p->w_stride_n + k * p->w_stride_k]);
                }
            }
            uint32_t v = acc;
            const int32_t zpw = p->zp_w ? p->zp_w[n] : p->zp_w_scalar;
            if (need_comp) {
                /* matmul_int8_compensate: raw - zp_a*R_b - zp_b*R_a + K*zp_a*zp_b (int32, wrapping) */
                v -= (uint32_t)zpa * (uint32_t)r_b[n];
                v -= (uint32_t)zpw * (uint32_t)r_a;
                v += (uint32_t)(int32_t)p->k * (uint32_t)zpa * (uint32_t)zpw;
            }
            const float s_w = p->scale_w ? p->scale_w[n] : p->scale_w_scalar;
            if (p->out_kind <= ORACLE_OUT_U8) {
                if (p->bias) v += (uint32_t)((const int32_t*)p->bias)[n];
                int32_t vi = (int32_t)v;
                if (p->relu && vi < 0) vi = 0;
                if (p->out_kind == ORACLE_OUT_S32) {
                    ((int32_t*)p->out)[m * p->ldc + n] = vi;
                } else {
                    volatile float req_v = row_k * s_w;
                    if (p->out_kind == ORACLE_OUT_S8) {
                        ((int8_t*)p->out)[m * p->ldc + n] =
                            (int8_t)requant_value(vi, req_v, p->out_zp, -128.0f, 127.0f);
                    } else {
                        ((uint8_t*)p->out)[m * p->ldc + n] =
                            (uint8_t)requant_value(vi, req_v, p->out_zp, 0.0f, 255.0f);
                    }
                }
            } else {
                /* simd_epilogue.hpp:924-948 / matmul_i8_common.cuh:184-211: dequantize with
                 * s_a*s_w, add a non-zero fp bias, clip, then (Relu only here) activate. */
                volatile float sc = s_a * s_w;
                volatile float fv = (float)(int32_t)v * sc;
                float f = fv;
                float b = 0.0f;
                if (p->bias) {
                    b = (p->out_kind == ORACLE_OUT_F32) ? ((const float*)p->bias)[n]
                                                         : oracle_f16_to_f32(((const uint16_t*)p->bias)[n]);
                }
                if (b != 0.0f) {
                    volatile float t = f + b;
                    f = t;
                }
                f = f > p->min_clip ? f : p->min_clip;
                f = f < p->max_clip ? f : p->max_clip;
                if (p->relu && f < 0.0f) f = 0.0f;
                if (p->out_kind == ORACLE_OUT_F32) {
                    ((float*)p->out)[m * p->ldc + n] = f;
                } else {
                    ((uint16_t*)p->out)[m * p->ldc + n] = oracle_f32_to_f16(f);
                }
            }
        }
    }
    free(r_b);
}

/* ---- Q4_1 weight-decode matmul ------------------------------------------- */

/* out[m][n] = sum_k a[m][k] * w[n][k], W given as Q4_1 rows of `ldw_blocks` blocks.
 * Reference: src/backend/cpu/x86_64/mma_qblock.hpp:144-291 (fused small-M route, f32
 * accumulation over the whole K) and tests/test_matmul_q4_1.cpp:190-224 (the order-free
 * expected value the reference's own test uses).  Sum order is not pinned by the
 * reference (its tests are tolerance-based), so this accumulates in f64 and rounds
 * once.  a_is_f16: activations are IEEE half; w_round_f16: each decoded weight is
 * rounded to half first (the reference's f16 route, test_matmul_q4_1.cpp:205-207).
 * out_is_f16: result rounded once to half (mma_qblock.hpp:112-115). */
void oracle_q4_1_matmul(const void* a, int a_is_f16, int64_t lda,
                        const uint8_t* w_blocks, int64_t ldw_blocks,
                        void* out, int out_is_f16, int64_t ldc,
                        int64_t m, int64_t n, int64_t k, int w_round_f16,
                        const void* bias)
{
    float* arow_all = (float*)malloc(sizeof(float) * (size_t)(m * k > 0 ? m * k : 1));
    for (int64_t i = 0; i < m; ++i) {
        for (int64_t j = 0; j < k; ++j) {
            arow_all[i * k + j] = a_is_f16 ? oracle_f16_to_f32(((const uint16_t*)a)[i * lda + j])
                                           : ((const float*)a)[i * lda + j];
        }
    }
#pragma omp parallel
    {
        float* wrow = (float*)malloc(sizeof(float) * (size_t)(k > 0 ? k : 1));
#pragma omp for schedule(static)
        for (int64_t j = 0; j < n; ++j) {
            oracle_q4_1_decode_row(w_blocks + j * ldw_blocks * Q4_1_BLOCK_BYTES, k, wrow);
            if (w_round_f16) {
                for (int64_t kk = 0; kk < k; ++kk) {
                    wrow[kk] = oracle_f16_to_f32(oracle_f32_to_f16(wrow[kk]));
                }
            }
            for (int64_t i = 0; i < m; ++i) {
                const float* ar = arow_all + i * k;
                double acc = 0.0;
                for (int64_t kk = 0; kk < k; ++kk) {
                    acc += (double)ar[kk] * (double)wrow[kk];
                }
                float r = (float)acc;
                if (bias) {
                    r += out_is_f16 ? oracle_f16_to_f32(((const uint16_t*)bias)[j]) : ((const float*)bias)[j];
                }
                if (out_is_f16) {
                    ((uint16_t*)out)[i * ldc + j] = oracle_f32_to_f16(r);
                } else {
                    ((float*)out)[i * ldc + j] = r;
                }
            }
        }
        free(wrow);
    }
    free(arow_all);
}

/* ---- QuantizeLinear / DequantizeLinear ----------------------------------------------------
 * The tensor is a flat row-major array seen as [outer][rows][inner]; parameter r (scale,
 * zero point) serves every element of row r of every outer group
 * (src/backend/cpu/quant_linear.cpp:83-118: per tensor = [1][1][numel], per token =
 * [1][numel/last][last], per channel = [outer][shape[axis]][inner]).
 *
 * Arithmetic of the x86 arch kernels (src/backend/cpu/x86_64/quant.hpp:117-165, 278-325):
 *   quantize:   inv = 1.0f / scale; v = fma(x, inv, zp) in ONE rounding; q = v rounded to
 *               nearest-even as int32, where anything outside int32 (and NaN) becomes
 *               INT32_MIN as cvtps2dq does; then saturate to the 8-bit range.
 *   dequantize: first (inner - inner % 16) elements of a row:  fma(float(q), scale, -zp*scale);
 *               the last inner % 16 elements (the scalar tail):  (float(q) - zp) * scale.
 * f16 inputs are widened exactly, f16 outputs rounded once from the f32 result (RNE).
 * tail_fused = 0 makes the quantize tail round the product before the add (the literal
 * reading of the scalar tail, quant.hpp:159-164); the reference compiled with its own flags
 * contracts it into the same fma as the vector body, which tests/test_oracle.py pins.
 */
/* zp_kind: 0 = s8, 1 = u8, 2 = int32 storage. */
static float load_zero_point(const void* zero_point, int zp_kind, int64_t r)
{
    if (zp_kind == 2) {
        return (float)((const int32_t*)zero_point)[r];
    }
    return zp_kind == 1 ? (float)((const uint8_t*)zero_point)[r] : (float)((const int8_t*)zero_point)[r];
}

static int32_t cvt_rne_x86(float v)
{
    if (!(v >= -2147483648.0f && v < 2147483648.0f)) {
        return INT32_MIN;
    }
    return (int32_t)nearbyintf(v);
}

void oracle_quantize_linear(const void* x, int x_is_f16, int64_t outer, int64_t rows, int64_t inner,
                            const float* scale, const void* zero_point, int zp_kind,
                            void* y, int y_is_u8, int tail_fused)
{
    const int32_t qmin = y_is_u8 ? 0 : -128;
    const int32_t qmax = y_is_u8 ? 255 : 127;
    const int64_t body = inner - inner % 16;
    for (int64_t o = 0; o < outer; ++o) {
        for (int64_t r = 0; r < rows; ++r) {
            const float inv = 1.0f / scale[r];
            const float zp = load_zero_point(zero_point, zp_kind, r);
            const int64_t base = (o * rows + r) * inner;
            for (int64_t i = 0; i < inner; ++i) {
                const float xv = x_is_f16 ? oracle_f16_to_f32(((const uint16_t*)x)[base + i]) : ((const float*)x)[base + i];
                float v;
                if (i < body || tail_fused) {
                    v = fmaf(xv, inv, zp);
                } else {
                    const float prod = xv * inv;
                    v = prod + zp;
                }
                int32_t q = cvt_rne_x86(v);
                q = q < qmin ? qmin : (q > qmax ? qmax : q);
                if (y_is_u8) {
                    ((uint8_t*)y)[base + i] = (uint8_t)q;
                } else {
                    ((int8_t*)y)[base + i] = (int8_t)q;
                }
            }
        }
    }
}

void oracle_dequantize_linear(const void* x, int x_is_u8, int64_t outer, int64_t rows, int64_t inner,
                              const float* scale, const void* zero_point, int zp_kind,
                              void* y, int y_is_f16)
{
    const int64_t body = inner - inner % 16;
    for (int64_t o = 0; o < outer; ++o) {
        for (int64_t r = 0; r < rows; ++r) {
            const float s = scale[r];
            const float zp = load_zero_point(zero_point, zp_kind, r);
            const float neg_zs = -zp * s;
            const int64_t base = (o * rows + r) * inner;
            for (int64_t i = 0; i < inner; ++i) {
                const float q = x_is_u8 ? (float)((const uint8_t*)x)[base + i] : (float)((const int8_t*)x)[base + i];
                float f;
                if (i < body) {
                    f = fmaf(q, s, neg_zs);
                } else {
                    const float d = q - zp;
                    f = d * s;
                }
                if (y_is_f16) {
                    ((uint16_t*)y)[base + i] = oracle_f32_to_f16(f);
                } else {
                    ((float*)y)[base + i] = f;
                }
            }
        }
    }
}
