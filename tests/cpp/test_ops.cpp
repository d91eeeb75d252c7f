// Operator-level tests of the CUDA backend through the nnops API: Linear / MatMul created with
// Backend::CUDA, pitched non-owning TensorViews over device memory, the stream in
// ComputeContext.  The cases follow the reference's own tests -- the hand-computed vectors of
// tests/test_matmul_int8.cpp:106-285, the differential cases of tests/test_cuda_matmul.cpp:681-889
// and tests/test_cuda_linear.cpp:190-351, the contract cases of tests/test_status.cpp -- and read
// like them.
//
// Built twice by nnops_b200/host/build.py:
//   * against the stand-alone API mirror (expected values from the C oracle), and
//   * with NNB200_USE_NNOPS_HEADERS against the real nnops tree, where the same operator is
//     also run on Backend::CPU (the reference's CPU route) and compared byte for byte.

#ifdef NNB200_USE_NNOPS_HEADERS
#include "nnops/ops/conv2d.hpp"
#include "nnops/ops/linear.hpp"
#include "nnops/ops/matmul.hpp"
#include "nnops/ops/quant_linear.hpp"
#else
#include "nnops_b200/nnops_api.hpp"
#endif

#include <cuda_runtime_api.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <vector>

using namespace nnops;

// ---- C oracle (oracle/nnops_oracle.c) -----------------------------------------------------
extern "C" {
struct oracle_gemm_i8_args {
    const void* a; const int8_t* w; void* out;
    int64_t m, n, k;
    int64_t a_stride_m, a_stride_k, w_stride_n, w_stride_k, ldc;
    int32_t a_unsigned; int32_t out_kind;
    const void* bias; int32_t relu;
    const float* scale_a; const float* scale_w; const int32_t* zp_a; const int32_t* zp_w;
    float scale_a_scalar, scale_w_scalar; int32_t zp_a_scalar, zp_w_scalar;
    float out_scale; int32_t out_zp; float min_clip, max_clip;
};
void oracle_gemm_i8(const oracle_gemm_i8_args* p);
void oracle_q4_1_matmul(const void* a, int a_is_f16, int64_t lda, const uint8_t* w_blocks, int64_t ldw_blocks, void* out,
                        int out_is_f16, int64_t ldc, int64_t m, int64_t n, int64_t k, int w_round_f16, const void* bias);
void oracle_quantize_linear(const void* x, int x_is_f16, int64_t outer, int64_t rows, int64_t inner, const float* scale,
                            const void* zero_point, int zp_is_u8, void* y, int y_is_u8, int tail_fused);
void oracle_dequantize_linear(const void* x, int x_is_u8, int64_t outer, int64_t rows, int64_t inner, const float* scale,
                              const void* zero_point, int zp_is_u8, void* y, int y_is_f16);
uint16_t oracle_f32_to_f16(float f);
float oracle_f16_to_f32(uint16_t h);
}

// ---- tiny harness -------------------------------------------------------------------------
static int g_checks = 0, g_failed = 0;
static const char* g_case = "";
#define EXPECT(cond)                                                                       \
    do {                                                                                   \
        ++g_checks;                                                                        \
        if (!(cond)) {                                                                     \
            ++g_failed;                                                                    \
            std::printf("FAIL [%s] %s:%d: %s\n", g_case, __FILE__, __LINE__, #cond);      \
        }                                                                                  \
    } while (0)
#define CUDA_OK(x)                                                                    \
    do {                                                                              \
        if ((x) != cudaSuccess) {                                                     \
            std::printf("CUDA error at %s:%d\n", __FILE__, __LINE__);                \
            std::exit(2);                                                             \
        }                                                                             \
    } while (0)

struct DevBuf {
    void* p = nullptr;
    size_t bytes = 0;
    explicit DevBuf(size_t n, int fill = 0) : bytes(n)
    {
        CUDA_OK(cudaMalloc(&p, n ? n : 1));
        CUDA_OK(cudaMemset(p, fill, n ? n : 1));
    }
    DevBuf(const void* host, size_t n) : bytes(n)
    {
        CUDA_OK(cudaMalloc(&p, n ? n : 1));
        CUDA_OK(cudaMemcpy(p, host, n, cudaMemcpyHostToDevice));
    }
    ~DevBuf() { cudaFree(p); }
    template <class T> std::vector<T> download() const
    {
        std::vector<T> v(bytes / sizeof(T));
        CUDA_OK(cudaDeviceSynchronize());
        CUDA_OK(cudaMemcpy(v.data(), p, bytes, cudaMemcpyDeviceToHost));
        return v;
    }
    DevBuf(const DevBuf&) = delete;
    DevBuf& operator=(const DevBuf&) = delete;
};

static QuantParams per_tensor(float s, int32_t z)
{
    QuantParams q;
    q.scale = s;
    q.zero_point = z;
    return q;
}
static QuantParams arrays(const float* s, const int32_t* z, int64_t n, QuantGranularity g)
{
    QuantParams q;
    q.granularity = g;
    q.scale_data = s;
    q.zero_point_data = z;
    q.num_scales = n;
    return q;
}
template <size_t R> static TensorView view(const int64_t (&shape)[R], DataType dt, void* data, QuantParams q = {})
{
    return TensorView(std::span<const int64_t>(shape, R), dt, data, TensorLayout::Dense, q);
}

// ---- exact-value cases (reference tests/test_matmul_int8.cpp:106-285) ----------------------

static void kat_basic_s32()
{
    g_case = "matmul_int8_basic_s32";
    const int8_t a_h[6] = {1, -2, 3, -4, 5, -6};
    const int8_t b_h[6] = {1, 2, 3, 4, 5, 6};  // [K=3, N=2]
    DevBuf a(a_h, 6), b(b_h, 6), c(16, 0x7F);
    const int64_t as[] = {2, 3}, bs[] = {3, 2}, cs[] = {2, 2};
    MatMulAttributes attrs;
    attrs.output_dtype = DataType::s32;
    auto op = MatMul::create(attrs, Backend::CUDA);
    const TensorDesc in_d[] = {view(as, DataType::s8, a.p).desc(), view(bs, DataType::s8, b.p).desc()};
    const auto od = op->getOutputTensorDesc(in_d);
    EXPECT(od[0].dtype == DataType::s32 && od[0].rank == 2 && od[0].dims[0] == 2 && od[0].dims[1] == 2);
    TensorView out = view(cs, DataType::s32, c.p);
    const TensorView ins[] = {view(as, DataType::s8, a.p), view(bs, DataType::s8, b.p)};
    EXPECT(op->compute(out, ins) == Status::ok);
    const auto r = c.download<int32_t>();
    EXPECT(r[0] == 10 && r[1] == 12 && r[2] == -19 && r[3] == -24);
}

static void kat_zero_points()
{
    g_case = "matmul_int8_zeropoint_s32";
    const int8_t a_h[6] = {1, 2, 3, 4, 5, 6}, w_h[6] = {7, 8, 9, 10, 11, 12};
    const float ones[2] = {1.0f, 1.0f};
    const int32_t a_zp[2] = {1, 2}, w_zp[2] = {3, 4};  // HOST arrays, as the reference passes them
    DevBuf a(a_h, 6), w(w_h, 6), c(16);
    const int64_t s23[] = {2, 3}, s22[] = {2, 2};
    MatMulAttributes attrs;
    attrs.transpose_b = true;
    attrs.output_dtype = DataType::s32;
    auto op = MatMul::create(attrs, Backend::CUDA);
    TensorView out = view(s22, DataType::s32, c.p);
    const TensorView ins[] = {view(s23, DataType::s8, a.p, arrays(ones, a_zp, 2, QuantGranularity::PerToken)),
                              view(s23, DataType::s8, w.p, arrays(ones, w_zp, 2, QuantGranularity::PerChannel))};
    EXPECT(op->compute(out, ins) == Status::ok);
    const auto r = c.download<int32_t>();
    EXPECT(r[0] == 17 && r[1] == 23 && r[2] == 47 && r[3] == 65);
}

static void kat_u8_zero_points()
{
    g_case = "matmul_int8_u8_zeropoint_s32";
    const uint8_t a_h[6] = {130, 128, 3, 200, 255, 0};
    const int8_t b_h[6] = {1, -4, 2, 5, 3, -6};
    const float ones[2] = {1.0f, 1.0f};
    const int32_t a_zp[2] = {128, 100};
    DevBuf a(a_h, 6), b(b_h, 6), c(16);
    const int64_t as[] = {2, 3}, bs[] = {3, 2}, cs[] = {2, 2};
    MatMulAttributes attrs;
    attrs.output_dtype = DataType::s32;
    auto op = MatMul::create(attrs, Backend::CUDA);
    TensorView out = view(cs, DataType::s32, c.p);
    const TensorView ins[] = {view(as, DataType::u8, a.p, arrays(ones, a_zp, 2, QuantGranularity::PerToken)),
                              view(bs, DataType::s8, b.p, per_tensor(1.0f, 3))};
    EXPECT(op->compute(out, ins) == Status::ok);
    const auto r = c.download<int32_t>();
    EXPECT(r[0] == -4 && r[1] == 1111 && r[2] == -355 && r[3] == 510);
}

static void kat_requant()
{
    g_case = "matmul_int8_requant_s8";
    {
        const int8_t a_h[2] = {4, 6}, w_h[4] = {1, 1, 1, 1};
        DevBuf a(a_h, 2), w(w_h, 4), c(2);
        const int64_t as[] = {1, 2}, ws[] = {2, 2}, cs[] = {1, 2};
        MatMulAttributes attrs;
        attrs.transpose_b = true;
        attrs.output_dtype = DataType::s8;
        auto op = MatMul::create(attrs, Backend::CUDA);
        TensorView out = view(cs, DataType::s8, c.p, per_tensor(2.0f, 0));
        const TensorView ins[] = {view(as, DataType::s8, a.p), view(ws, DataType::s8, w.p)};
        EXPECT(op->compute(out, ins) == Status::ok);
        const auto r = c.download<int8_t>();
        EXPECT(r[0] == 5 && r[1] == 5);
    }
    g_case = "matmul_int8_requant_clamp_s8";
    {
        const int8_t a_h[2] = {100, 100}, w_h[4] = {100, 100, 100, 100};
        DevBuf a(a_h, 2), w(w_h, 4), c(2);
        const int64_t as[] = {1, 2}, ws[] = {2, 2}, cs[] = {1, 2};
        MatMulAttributes attrs;
        attrs.transpose_b = true;
        attrs.output_dtype = DataType::s8;
        auto op = MatMul::create(attrs, Backend::CUDA);
        TensorView out = view(cs, DataType::s8, c.p, per_tensor(1.0f, 0));
        const TensorView ins[] = {view(as, DataType::s8, a.p), view(ws, DataType::s8, w.p)};
        EXPECT(op->compute(out, ins) == Status::ok);
        const auto r = c.download<int8_t>();
        EXPECT(r[0] == 127 && r[1] == 127);
    }
}

// ---- differential cases --------------------------------------------------------------------

struct LinearCase {
    int64_t batch, m, n, k;
    DataType out_dt;
    bool relu, per_token, per_channel, zero_points, device_arrays;
    int64_t a_pad, w_pad, c_pad;  // extra bytes/elements of row pitch
};

static int kind_of(DataType dt)
{
    switch (dt) {
    case DataType::s32: return 0;
    case DataType::s8: return 1;
    case DataType::u8: return 2;
    case DataType::f32: return 3;
    default: return 4;
    }
}

static void linear_i8_case(const LinearCase& c, const char* name, cudaStream_t stream)
{
    g_case = name;
    std::mt19937_64 rng(c.m * 131 + c.n * 17 + c.k);
    const int64_t rows = c.batch * c.m;
    const int64_t lda = c.k + c.a_pad, ldw = c.k + c.w_pad, ldc = c.n + c.c_pad;
    const size_t osz = data_type_size(c.out_dt);
    std::vector<int8_t> a(rows * lda), w(c.n * ldw);
    for (auto& v : a) v = static_cast<int8_t>(static_cast<int>(rng() % 255) - 127);
    for (auto& v : w) v = static_cast<int8_t>(static_cast<int>(rng() % 255) - 127);
    std::vector<int32_t> bias(c.n), zpa(c.m), zpw(c.n);
    std::vector<float> sa(c.m), sw(c.n);
    std::uniform_real_distribution<float> us(0.001f, 0.02f), ua(0.01f, 0.03f);
    for (auto& v : bias) v = static_cast<int32_t>(rng() % 2001) - 1000;
    for (auto& v : sa) v = ua(rng);
    for (auto& v : sw) v = us(rng);
    for (auto& v : zpa) v = c.zero_points ? static_cast<int32_t>(rng() % 19) - 9 : 0;
    for (auto& v : zpw) v = c.zero_points ? static_cast<int32_t>(rng() % 19) - 9 : 0;
    const bool int_out = kind_of(c.out_dt) <= 2;
    std::vector<float> bias_f(c.n);
    std::vector<uint16_t> bias_h(c.n);
    for (int64_t i = 0; i < c.n; ++i) {
        bias_f[i] = 0.01f * static_cast<float>(bias[i]);
        bias_h[i] = oracle_f32_to_f16(bias_f[i]);
    }
    const void* bias_host = int_out ? static_cast<const void*>(bias.data())
                                    : (c.out_dt == DataType::f32 ? static_cast<const void*>(bias_f.data())
                                                                 : static_cast<const void*>(bias_h.data()));
    const size_t bias_bytes = static_cast<size_t>(c.n) * (int_out ? 4 : osz);
    const float out_scale = 1.7f;
    const int32_t out_zp = c.out_dt == DataType::s32 ? 0 : 3;

    // Expected: the C oracle, one batch slice at a time (per-token arrays index the row inside the slice).
    std::vector<uint8_t> want(rows * ldc * osz, 0x5A);
    for (int64_t b = 0; b < c.batch; ++b) {
        oracle_gemm_i8_args o{};
        o.a = a.data() + b * c.m * lda;
        o.w = w.data();
        o.out = want.data() + b * c.m * ldc * osz;
        o.m = c.m; o.n = c.n; o.k = c.k;
        o.a_stride_m = lda; o.a_stride_k = 1; o.w_stride_n = ldw; o.w_stride_k = 1; o.ldc = ldc;
        o.out_kind = kind_of(c.out_dt);
        o.bias = bias_host;
        o.relu = c.relu;
        o.scale_a = c.per_token ? sa.data() : nullptr;
        o.scale_w = c.per_channel ? sw.data() : nullptr;
        o.zp_a = c.per_token && c.zero_points ? zpa.data() : nullptr;
        o.zp_w = c.per_channel && c.zero_points ? zpw.data() : nullptr;
        o.scale_a_scalar = c.per_token ? 1.0f : 0.02f;
        o.scale_w_scalar = c.per_channel ? 1.0f : 0.01f;
        o.zp_a_scalar = (!c.per_token && c.zero_points) ? 2 : 0;
        o.zp_w_scalar = (!c.per_channel && c.zero_points) ? -3 : 0;
        o.out_scale = out_scale; o.out_zp = out_zp;
        o.min_clip = -INFINITY; o.max_clip = INFINITY;
        oracle_gemm_i8(&o);
    }

    DevBuf da(a.data(), a.size()), dw(w.data(), w.size()), dbias(bias_host, bias_bytes);
    DevBuf dout(want.size(), 0x5A);
    DevBuf dsa(sa.data(), sa.size() * 4), dsw(sw.data(), sw.size() * 4), dza(zpa.data(), zpa.size() * 4),
        dzw(zpw.data(), zpw.size() * 4);
    QuantParams qa = per_tensor(0.02f, c.zero_points ? 2 : 0), qw = per_tensor(0.01f, c.zero_points ? -3 : 0);
    if (c.per_token) {
        qa = arrays(c.device_arrays ? static_cast<const float*>(dsa.p) : sa.data(),
                    c.zero_points ? (c.device_arrays ? static_cast<const int32_t*>(dza.p) : zpa.data()) : nullptr, c.m,
                    QuantGranularity::PerToken);
    }
    if (c.per_channel) {
        qw = arrays(c.device_arrays ? static_cast<const float*>(dsw.p) : sw.data(),
                    c.zero_points ? (c.device_arrays ? static_cast<const int32_t*>(dzw.p) : zpw.data()) : nullptr, c.n,
                    QuantGranularity::PerChannel);
    }
    const int64_t xs3[] = {c.batch, c.m, c.k}, xs2[] = {c.m, c.k}, ws[] = {c.n, c.k}, bs[] = {c.n};
    const int64_t os3[] = {c.batch, c.m, c.n}, os2[] = {c.m, c.n};
    const bool b3 = c.batch > 1;
    TensorView x = b3 ? TensorView(xs3, DataType::s8, da.p, lda, TensorLayout::Dense, qa)
                      : TensorView(xs2, DataType::s8, da.p, lda, TensorLayout::Dense, qa);
    TensorView wv(ws, DataType::s8, dw.p, ldw, TensorLayout::Dense, qw);
    TensorView bv(bs, int_out ? DataType::s32 : c.out_dt, dbias.p);
    TensorView out = b3 ? TensorView(os3, c.out_dt, dout.p, ldc * static_cast<int64_t>(osz), TensorLayout::Dense,
                                     per_tensor(out_scale, out_zp))
                        : TensorView(os2, c.out_dt, dout.p, ldc * static_cast<int64_t>(osz), TensorLayout::Dense,
                                     per_tensor(out_scale, out_zp));

    LinearAttributes attrs;
    attrs.output_dtype = c.out_dt;
    attrs.epilogue.type = c.relu ? EpilogueActivateType::Relu : EpilogueActivateType::None;
    auto op = Linear::create(attrs, Backend::CUDA);
    const TensorDesc in_d[] = {x.desc(), wv.desc(), bv.desc()};
    const auto od = op->getOutputTensorDesc(in_d);
    EXPECT(od[0].dtype == c.out_dt && od[0].dims[static_cast<size_t>(od[0].rank - 1)] == c.n);
    const TensorDesc out_d[] = {out.desc()};
    EXPECT(op->validate(in_d, out_d) == Status::ok);
    ComputeContext ctx;
    ctx.expected_backend = Backend::CUDA;
    ctx.cuda_stream = stream;
    const TensorView ins[] = {x, wv, bv};
    EXPECT(op->compute(out, ins, ctx) == Status::ok);
    const auto got = dout.download<uint8_t>();
    EXPECT(got == want);  // byte for byte, padding canaries included

#ifdef NNB200_USE_NNOPS_HEADERS
    // The reference's own CPU route on the same bytes (host views).
    if (!c.device_arrays) {
        std::vector<uint8_t> cpu(want.size(), 0x5A);
        QuantParams hqa = qa, hqw = qw;
        TensorView hx = b3 ? TensorView(xs3, DataType::s8, a.data(), lda, TensorLayout::Dense, hqa)
                           : TensorView(xs2, DataType::s8, a.data(), lda, TensorLayout::Dense, hqa);
        TensorView hw(ws, DataType::s8, w.data(), ldw, TensorLayout::Dense, hqw);
        TensorView hb(bs, int_out ? DataType::s32 : c.out_dt, const_cast<void*>(bias_host));
        TensorView ho = b3 ? TensorView(os3, c.out_dt, cpu.data(), ldc * static_cast<int64_t>(osz), TensorLayout::Dense,
                                        per_tensor(out_scale, out_zp))
                           : TensorView(os2, c.out_dt, cpu.data(), ldc * static_cast<int64_t>(osz), TensorLayout::Dense,
                                        per_tensor(out_scale, out_zp));
        auto cpu_op = Linear::create(attrs, Backend::CPU);
        const TensorView hins[] = {hx, hw, hb};
        EXPECT(cpu_op->compute(ho, hins) == Status::ok);
        EXPECT(cpu == got);
    }
#endif
}

static void linear_q4_1_case(int64_t m, int64_t n, int64_t k, bool out_f16, const char* name)
{
    g_case = name;
    std::mt19937_64 rng(m + n + k);
    const int64_t nblk = (k + 31) / 32;
    std::vector<uint8_t> wb(n * nblk * 20);
    std::uniform_real_distribution<float> ud(0.005f, 0.02f), uu(0.8f, 1.2f);
    std::normal_distribution<float> na(0.0f, 1.0f);
    for (int64_t i = 0; i < n * nblk; ++i) {
        const uint16_t d = oracle_f32_to_f16(ud(rng));
        const uint16_t mn = oracle_f32_to_f16(-8.0f * oracle_f16_to_f32(d) * uu(rng));
        std::memcpy(&wb[i * 20], &d, 2);
        std::memcpy(&wb[i * 20 + 2], &mn, 2);
        for (int j = 0; j < 16; ++j) wb[i * 20 + 4 + j] = static_cast<uint8_t>(rng() & 0xFF);
    }
    std::vector<uint16_t> x(m * k);
    for (auto& v : x) v = oracle_f32_to_f16(na(rng));
    const size_t osz = out_f16 ? 2 : 4;
    std::vector<uint8_t> want(m * n * osz);
    oracle_q4_1_matmul(x.data(), 1, k, wb.data(), nblk, want.data(), out_f16, n, m, n, k, 1, nullptr);

    DevBuf dx(x.data(), x.size() * 2), dw(wb.data(), wb.size()), dout(want.size());
    const int64_t xs[] = {m, k}, ws[] = {n, k}, os[] = {m, n};
    const DataType odt = out_f16 ? DataType::f16 : DataType::f32;
    LinearAttributes attrs;
    attrs.output_dtype = odt;
    auto op = Linear::create(attrs, Backend::CUDA);
    TensorView out = view(os, odt, dout.p);
    const TensorView ins[] = {view(xs, DataType::f16, dx.p), view(ws, DataType::q4_1, dw.p)};
    EXPECT(ins[1].row_stride_elems() == nblk);  // q4_1 strides count 20-byte blocks
    ComputeContext ctx;
    ctx.expected_backend = Backend::CUDA;
    EXPECT(op->compute(out, ins, ctx) == Status::ok);
    const auto got = dout.download<uint8_t>();
    // rtol 1e-2 (f16 out) / 2e-3 (f32 out) with an absolute floor of rtol * rms(reference).
    const float rtol = out_f16 ? 1e-2f : 2e-3f;
    double sq = 0;
    std::vector<float> gv(m * n), wv(m * n);
    for (int64_t i = 0; i < m * n; ++i) {
        if (out_f16) {
            uint16_t a16, b16;
            std::memcpy(&a16, &got[i * 2], 2);
            std::memcpy(&b16, &want[i * 2], 2);
            gv[i] = oracle_f16_to_f32(a16);
            wv[i] = oracle_f16_to_f32(b16);
        } else {
            std::memcpy(&gv[i], &got[i * 4], 4);
            std::memcpy(&wv[i], &want[i * 4], 4);
        }
        sq += double(wv[i]) * wv[i];
    }
    const float rms = static_cast<float>(std::sqrt(sq / double(m * n)));
    int64_t bad = 0;
    for (int64_t i = 0; i < m * n; ++i) {
        if (std::fabs(gv[i] - wv[i]) > rtol * std::fabs(wv[i]) + rtol * rms) ++bad;
    }
    EXPECT(bad == 0);
}

// ---- contract cases (reference tests/test_status.cpp, README "errors write nothing") --------

static void contract_cases()
{
    g_case = "status_contract";
    const int64_t xs[] = {4, 64}, ws[] = {8, 64}, ws_bad[] = {8, 48}, os[] = {4, 8};
    DevBuf x(4 * 64), w(8 * 64), out(4 * 8 * 4, 0x6B);
    LinearAttributes attrs;
    attrs.output_dtype = DataType::s32;
    auto op = Linear::create(attrs, Backend::CUDA);
    EXPECT(op != nullptr && op->getBackend() == Backend::CUDA);
    TensorView o = view(os, DataType::s32, out.p);

    {   // K mismatch: invalid_argument, output untouched
        const TensorView ins[] = {view(xs, DataType::s8, x.p), view(ws_bad, DataType::s8, w.p)};
        EXPECT(op->compute(o, ins) == Status::invalid_argument);
    }
    {   // wrong input count
        const TensorView ins[] = {view(xs, DataType::s8, x.p)};
        EXPECT(op->compute(o, std::span<const TensorView>(ins, 1)) == Status::invalid_argument);
    }
    {   // gated form has no CUDA route
        LinearAttributes g = attrs;
        g.gated = true;
        auto gop = Linear::create(g, Backend::CUDA);
        const TensorView ins[] = {view(xs, DataType::s8, x.p), view(ws, DataType::s8, w.p)};
        EXPECT(gop->compute(o, ins) != Status::ok);
    }
    {   // rank above six
        const int64_t x7[] = {1, 1, 1, 1, 1, 4, 64};
        const TensorView ins[] = {view(x7, DataType::s8, x.p), view(ws, DataType::s8, w.p)};
        const int64_t o7[] = {1, 1, 1, 1, 1, 4, 8};
        TensorView o7v = view(o7, DataType::s32, out.p);
        EXPECT(op->compute(o7v, ins) == Status::unsupported);
    }
    {   // dense fp Linear is not this backend's path
        const TensorView ins[] = {view(xs, DataType::f32, x.p), view(ws, DataType::f32, w.p)};
        DevBuf big(4 * 64 * 4);
        (void)big;
        EXPECT(op->compute(o, ins) == Status::unsupported);
    }
    const auto after = out.download<uint8_t>();
    bool untouched = true;
    for (uint8_t b : after) untouched = untouched && b == 0x6B;
    EXPECT(untouched);  // every rejected call wrote nothing
    {   // empty output: ok, nothing to do
        const int64_t x0[] = {0, 64}, o0[] = {0, 8};
        const TensorView ins[] = {view(x0, DataType::s8, x.p), view(ws, DataType::s8, w.p)};
        TensorView o0v = view(o0, DataType::s32, out.p);
        EXPECT(op->compute(o0v, ins) == Status::ok);
    }
    {   // the two-step prepack query
        TensorView packed;
        const TensorView ins[] = {view(ws, DataType::s8, w.p)};
        TensorView outs[] = {packed};
        op->prepackWeights(ins, outs);
#ifdef NNB200_USE_NNOPS_HEADERS
        EXPECT(outs[0].is_empty());  // the reference's CUDA front end: "no packed form"
#else
        EXPECT(outs[0].is_empty() && outs[0].rank() == 2 && outs[0].layout() == TensorLayout::PackedI8B200);
        const int64_t f32s[] = {8, 64};
        TensorView none;
        const TensorView fp[] = {view(f32s, DataType::f32, w.p)};
        TensorView fouts[] = {none};
        op->prepackWeights(fp, fouts);
        EXPECT(fouts[0].rank() == 0);  // other weights: no packed form
#endif
    }
    EXPECT(op->getWorkspaceSize({}, {}) == 0);
}

// ---- f32/f16 activations carrying QuantParams x s8 weights ---------------------------------
// (the reference's CPU-only quantize-on-the-fly route, src/backend/cpu/matmul/matmul_i8.cpp:389-464)

static void linear_fp_act_case(int64_t batch, int64_t m, int64_t n, int64_t k, bool f16, bool per_token, bool zero_points,
                               bool relu, const char* name, cudaStream_t stream)
{
    g_case = name;
    const int64_t rows = batch * m;
    std::mt19937_64 rng(m * 31 + n * 7 + k);
    std::normal_distribution<float> nd(0.0f, 2.0f);
    std::uniform_real_distribution<float> us(0.001f, 0.02f), ua(0.01f, 0.05f);
    std::vector<float> xf(rows * k), sa(rows), sw(n), bias_f(n);
    std::vector<uint16_t> xh(rows * k), bias_h(n);
    std::vector<int8_t> w(n * k);
    std::vector<int32_t> za(rows);
    for (auto& v : xf) v = nd(rng);
    for (int64_t i = 0; i < rows * k; ++i) {
        xh[i] = oracle_f32_to_f16(xf[i]);
        if (f16) xf[i] = oracle_f16_to_f32(xh[i]);
    }
    for (auto& v : w) v = static_cast<int8_t>(static_cast<int>(rng() % 255) - 127);
    for (auto& v : sa) v = ua(rng);
    for (auto& v : sw) v = us(rng);
    for (auto& v : za) v = zero_points ? static_cast<int32_t>(rng() % 19) - 9 : 0;
    for (int64_t i = 0; i < n; ++i) {
        bias_f[i] = 0.01f * static_cast<float>(static_cast<int>(rng() % 2001) - 1000);
        bias_h[i] = oracle_f32_to_f16(bias_f[i]);
    }
    const float sa0 = 0.03f;
    const int32_t za0 = zero_points ? 3 : 0;
    const void* x_host = f16 ? static_cast<const void*>(xh.data()) : static_cast<const void*>(xf.data());
    const void* bias_host = f16 ? static_cast<const void*>(bias_h.data()) : static_cast<const void*>(bias_f.data());
    const size_t fsz = f16 ? 2 : 4;
    const DataType fdt = f16 ? DataType::f16 : DataType::f32;

    // Expected: quantise with the oracle, then its int8 matmul with the dequantizing epilogue.
    std::vector<int8_t> aq(rows * k);
    const float s1[1] = {sa0};
    const int32_t z1[1] = {za0};
    oracle_quantize_linear(x_host, f16, 1, per_token ? rows : 1, per_token ? k : rows * k, per_token ? sa.data() : s1,
                           per_token ? static_cast<const void*>(za.data()) : static_cast<const void*>(z1), 2, aq.data(),
                           0, 1);
    std::vector<uint8_t> want(rows * n * fsz);
    oracle_gemm_i8_args o{};
    o.a = aq.data(); o.w = w.data(); o.out = want.data();
    o.m = rows; o.n = n; o.k = k;
    o.a_stride_m = k; o.a_stride_k = 1; o.w_stride_n = k; o.w_stride_k = 1; o.ldc = n;
    o.out_kind = f16 ? 4 : 3;
    o.bias = bias_host;
    o.relu = relu;
    o.scale_a = per_token ? sa.data() : nullptr;
    o.zp_a = per_token && zero_points ? za.data() : nullptr;
    o.scale_w = sw.data();
    o.scale_a_scalar = per_token ? 1.0f : sa0;
    o.scale_w_scalar = 1.0f;
    o.zp_a_scalar = per_token ? 0 : za0;
    o.out_scale = 1.0f;
    o.min_clip = -INFINITY; o.max_clip = INFINITY;
    oracle_gemm_i8(&o);

    DevBuf dx(x_host, rows * k * fsz), dw(w.data(), w.size()), dbias(bias_host, n * fsz), dout(want.size(), 0x5A);
    QuantParams qa = per_token ? arrays(sa.data(), zero_points ? za.data() : nullptr, rows, QuantGranularity::PerToken)
                               : per_tensor(sa0, za0);
    QuantParams qw = arrays(sw.data(), nullptr, n, QuantGranularity::PerChannel);
    const int64_t xs3[] = {batch, m, k}, xs2[] = {m, k}, ws[] = {n, k}, bs[] = {n}, os3[] = {batch, m, n}, os2[] = {m, n};
    const bool b3 = batch > 1;
    TensorView x = b3 ? TensorView(xs3, fdt, dx.p, TensorLayout::Dense, qa) : TensorView(xs2, fdt, dx.p, TensorLayout::Dense, qa);
    TensorView wv(ws, DataType::s8, dw.p, TensorLayout::Dense, qw);
    TensorView bv(bs, fdt, dbias.p);
    TensorView out = b3 ? TensorView(os3, fdt, dout.p) : TensorView(os2, fdt, dout.p);
    LinearAttributes attrs;
    attrs.epilogue.type = relu ? EpilogueActivateType::Relu : EpilogueActivateType::None;
    auto op = Linear::create(attrs, Backend::CUDA);
    const TensorDesc in_d[] = {x.desc(), wv.desc(), bv.desc()};
    EXPECT(op->getOutputTensorDesc(in_d)[0].dtype == fdt);
    ComputeContext ctx;
    ctx.expected_backend = Backend::CUDA;
    ctx.cuda_stream = stream;
    const TensorView ins[] = {x, wv, bv};
    EXPECT(op->compute(out, ins, ctx) == Status::ok);
    const auto got = dout.download<uint8_t>();
    EXPECT(got == want);
    {   // without parameters a float A is not a quantized tensor: rejected, nothing written
        DevBuf canary(want.size(), 0x3C);
        TensorView plain = b3 ? TensorView(xs3, fdt, dx.p) : TensorView(xs2, fdt, dx.p);
        TensorView o2v = b3 ? TensorView(os3, fdt, canary.p) : TensorView(os2, fdt, canary.p);
        const TensorView bad[] = {plain, wv, bv};
        EXPECT(op->compute(o2v, bad, ctx) == Status::invalid_argument);
        bool untouched = true;
        for (uint8_t b : canary.download<uint8_t>()) untouched = untouched && b == 0x3C;
        EXPECT(untouched);
    }
#ifdef NNB200_USE_NNOPS_HEADERS
    {   // the reference's CPU route on the same bytes
        std::vector<uint8_t> cpu(want.size());
        TensorView hx = b3 ? TensorView(xs3, fdt, const_cast<void*>(x_host), TensorLayout::Dense, qa)
                           : TensorView(xs2, fdt, const_cast<void*>(x_host), TensorLayout::Dense, qa);
        TensorView hw(ws, DataType::s8, w.data(), TensorLayout::Dense, qw);
        TensorView hb(bs, fdt, const_cast<void*>(bias_host));
        TensorView ho = b3 ? TensorView(os3, fdt, cpu.data()) : TensorView(os2, fdt, cpu.data());
        auto cpu_op = Linear::create(attrs, Backend::CPU);
        const TensorView hins[] = {hx, hw, hb};
        EXPECT(cpu_op->compute(ho, hins) == Status::ok);
        EXPECT(cpu == got);
    }
#endif
}

// ---- prepacked int8 weights (stand-alone API; the reference's CUDA operators have no packed form) ----
#ifndef NNB200_USE_NNOPS_HEADERS
static void prepack_case(bool matmul_kn, int64_t m, int64_t n, int64_t k, const char* name, cudaStream_t stream)
{
    g_case = name;
    std::mt19937_64 rng(m * 13 + n * 5 + k);
    std::vector<uint8_t> a(m * k);
    std::vector<int8_t> w(n * k), w_kn(k * n);
    for (auto& v : a) v = static_cast<uint8_t>(rng() % 256);
    for (auto& v : w) v = static_cast<int8_t>(static_cast<int>(rng() % 255) - 127);
    for (int64_t i = 0; i < n; ++i) {
        for (int64_t j = 0; j < k; ++j) w_kn[j * n + i] = w[i * k + j];
    }
    std::vector<float> sa(m), sw(n);
    std::vector<int32_t> za(m), zw(n), bias(n);
    std::uniform_real_distribution<float> us(0.001f, 0.02f), ua(0.01f, 0.03f);
    for (auto& v : sa) v = ua(rng);
    for (auto& v : sw) v = us(rng);
    for (auto& v : za) v = 100 + static_cast<int32_t>(rng() % 40);
    for (auto& v : zw) v = static_cast<int32_t>(rng() % 19) - 9;
    for (auto& v : bias) v = static_cast<int32_t>(rng() % 2001) - 1000;

    std::vector<int8_t> want(m * n);
    oracle_gemm_i8_args o{};
    o.a = a.data(); o.w = w.data(); o.out = want.data();
    o.m = m; o.n = n; o.k = k;
    o.a_stride_m = k; o.a_stride_k = 1; o.w_stride_n = k; o.w_stride_k = 1; o.ldc = n;
    o.a_unsigned = 1; o.out_kind = 1; o.bias = bias.data(); o.relu = 1;
    o.scale_a = sa.data(); o.scale_w = sw.data(); o.zp_a = za.data(); o.zp_w = zw.data();
    o.scale_a_scalar = 1.0f; o.scale_w_scalar = 1.0f;
    o.out_scale = 2.3f; o.out_zp = -3;
    o.min_clip = -INFINITY; o.max_clip = INFINITY;
    oracle_gemm_i8(&o);

    DevBuf da(a.data(), a.size()), dw(matmul_kn ? w_kn.data() : w.data(), w.size()), dbias(bias.data(), n * 4), dout(m * n, 0x5A);
    const int64_t as[] = {m, k}, ws_nk[] = {n, k}, ws_kn[] = {k, n}, bs[] = {n}, os[] = {m, n};
    const QuantParams qa = arrays(sa.data(), za.data(), m, QuantGranularity::PerToken);
    const QuantParams qw = arrays(sw.data(), zw.data(), n, QuantGranularity::PerChannel);
    TensorView wv = matmul_kn ? TensorView(ws_kn, DataType::s8, dw.p, TensorLayout::Dense, qw)
                              : TensorView(ws_nk, DataType::s8, dw.p, TensorLayout::Dense, qw);
    ComputeContext ctx;
    ctx.expected_backend = Backend::CUDA;
    ctx.cuda_stream = stream;
    LinearAttributes la;
    la.output_dtype = DataType::s8;
    la.epilogue.type = EpilogueActivateType::Relu;
    MatMulAttributes ma;
    ma.output_dtype = DataType::s8;
    ma.epilogue.type = EpilogueActivateType::Relu;
    auto lin = Linear::create(la, Backend::CUDA);
    auto mm = MatMul::create(ma, Backend::CUDA);
    OpBase* op = matmul_kn ? static_cast<OpBase*>(mm.get()) : static_cast<OpBase*>(lin.get());

    // Step 1: the query describes the blob.  Step 2: allocate that much and pack.
    TensorView packed;
    {
        const TensorView ins[] = {wv};
        TensorView outs[] = {packed};
        op->prepackWeights(ins, outs, ctx);
        packed = outs[0];
    }
    EXPECT(packed.is_empty() && packed.layout() == TensorLayout::PackedI8B200 && packed.shape(0) == n && packed.shape(1) == k);
    const size_t blob_bytes = static_cast<size_t>(packed.shape(0) * packed.pitch());
    EXPECT(blob_bytes == static_cast<size_t>(n) * static_cast<size_t>((k + 15) / 16 * 16 + 12));
    DevBuf blob(blob_bytes);
    TensorView filled(std::span<const int64_t>(packed.shape(), 2), DataType::s8, blob.p, packed.pitch(),
                      TensorLayout::PackedI8B200, packed.quant_params());
    {
        const TensorView ins[] = {wv};
        TensorView outs[] = {filled};
        op->prepackWeights(ins, outs, ctx);
    }
    TensorView out = TensorView(os, DataType::s8, dout.p, TensorLayout::Dense, per_tensor(2.3f, -3));
    const TensorView ins[] = {TensorView(as, DataType::u8, da.p, TensorLayout::Dense, qa), filled,
                              TensorView(bs, DataType::s32, dbias.p)};
    EXPECT(op->compute(out, ins, ctx) == Status::ok);
    EXPECT(dout.download<int8_t>() == want);
}
#endif

// ---- prepacked Q4_1 weights (stand-alone API): separated nibble and (d, m) planes ---------------
#ifndef NNB200_USE_NNOPS_HEADERS
static void prepack_q4_1_case(int64_t m, int64_t n, int64_t k, bool out_f16, const char* name, cudaStream_t stream)
{
    g_case = name;
    std::mt19937_64 rng(m * 7 + n + k);
    const int64_t nblk = (k + 31) / 32;
    std::vector<uint8_t> wb(n * nblk * 20);
    std::uniform_real_distribution<float> ud(0.005f, 0.02f), uu(0.8f, 1.2f);
    std::normal_distribution<float> na(0.0f, 1.0f);
    for (int64_t i = 0; i < n * nblk; ++i) {
        const uint16_t d = oracle_f32_to_f16(ud(rng));
        const uint16_t mn = oracle_f32_to_f16(-8.0f * oracle_f16_to_f32(d) * uu(rng));
        std::memcpy(&wb[i * 20], &d, 2);
        std::memcpy(&wb[i * 20 + 2], &mn, 2);
        for (int j = 0; j < 16; ++j) wb[i * 20 + 4 + j] = static_cast<uint8_t>(rng() & 0xFF);
    }
    std::vector<uint16_t> x(m * k);
    for (auto& v : x) v = oracle_f32_to_f16(na(rng));
    const size_t osz = out_f16 ? 2 : 4;
    DevBuf dx(x.data(), x.size() * 2), dw(wb.data(), wb.size()), d_raw(m * n * osz), d_packed(m * n * osz);
    const int64_t xs[] = {m, k}, ws[] = {n, k}, os[] = {m, n};
    const DataType odt = out_f16 ? DataType::f16 : DataType::f32;
    ComputeContext ctx;
    ctx.expected_backend = Backend::CUDA;
    ctx.cuda_stream = stream;
    auto op = Linear::create(LinearAttributes{}, Backend::CUDA);
    TensorView wv = view(ws, DataType::q4_1, dw.p);

    TensorView packed;
    {
        const TensorView ins[] = {wv};
        TensorView outs[] = {packed};
        op->prepackWeights(ins, outs, ctx);
        packed = outs[0];
    }
    EXPECT(packed.is_empty() && packed.layout() == TensorLayout::PackedQ4_1B200 && packed.shape(0) == n && packed.shape(1) == k);
    const size_t blob_bytes = static_cast<size_t>(packed.shape(0) * packed.pitch());
    EXPECT(blob_bytes >= static_cast<size_t>(n * nblk * 20) && packed.pitch() % 20 == 0);
    DevBuf blob(blob_bytes);
    TensorView filled(std::span<const int64_t>(packed.shape(), 2), DataType::q4_1, blob.p, packed.pitch(),
                      TensorLayout::PackedQ4_1B200, QuantParams{});
    {
        const TensorView ins[] = {wv};
        TensorView outs[] = {filled};
        op->prepackWeights(ins, outs, ctx);
    }
    TensorView out_raw = view(os, odt, d_raw.p), out_packed = view(os, odt, d_packed.p);
    const TensorView raw_ins[] = {view(xs, DataType::f16, dx.p), wv};
    const TensorView packed_ins[] = {view(xs, DataType::f16, dx.p), filled};
    EXPECT(op->compute(out_raw, raw_ins, ctx) == Status::ok);
    EXPECT(op->compute(out_packed, packed_ins, ctx) == Status::ok);
    // Same arithmetic on both forms wherever one engine serves both; everywhere within tolerance of the oracle.
    std::vector<uint8_t> want(m * n * osz);
    oracle_q4_1_matmul(x.data(), 1, k, wb.data(), nblk, want.data(), out_f16, n, m, n, k, 0, nullptr);
    const auto got = d_packed.download<uint8_t>();
    double rms = 0.0, worst = 0.0;
    for (int64_t i = 0; i < m * n; ++i) {
        const float w_ = out_f16 ? oracle_f16_to_f32(reinterpret_cast<const uint16_t*>(want.data())[i])
                                 : reinterpret_cast<const float*>(want.data())[i];
        const float g_ = out_f16 ? oracle_f16_to_f32(reinterpret_cast<const uint16_t*>(got.data())[i])
                                 : reinterpret_cast<const float*>(got.data())[i];
        rms += static_cast<double>(w_) * w_;
        worst = std::max(worst, static_cast<double>(std::fabs(g_ - w_)));
    }
    rms = std::sqrt(rms / static_cast<double>(m * n));
    EXPECT(worst <= (out_f16 ? 2e-2 : 4e-3) * rms);
}
#endif

// ---- QuantizeLinear / DequantizeLinear ------------------------------------------------------

// Known answers of the reference's operator test (tests/test_quant_linear.cpp:198-226, 439-467):
// per-channel along axis 1 of a [2,3] tensor, with the half-to-even tie 0.5 -> 0.
static void kat_quant_linear()
{
    g_case = "quantize_linear_2d_per_channel";
    const int64_t shape[] = {2, 3}, ps[] = {3};
    const float x_h[6] = {0.0f, 1.0f, 2.0f, 10.0f, 11.0f, 12.0f}, scale_h[3] = {1.0f, 2.0f, 3.0f};
    const int8_t zp_h[3] = {0, 0, 0};
    DevBuf x(x_h, sizeof(x_h)), sc(scale_h, sizeof(scale_h)), zp(zp_h, sizeof(zp_h)), y(6, 0x55);
    QuantLinearAttributes attrs;
    attrs.axis = 1;
    attrs.output_dtype = DataType::s8;
    auto op = QuantizeLinear::create(attrs, Backend::CUDA);
    const TensorView ins[] = {view(shape, DataType::f32, x.p), view(ps, DataType::f32, sc.p), view(ps, DataType::s8, zp.p)};
    const TensorDesc in_d[] = {ins[0].desc(), ins[1].desc(), ins[2].desc()};
    const auto od = op->getOutputTensorDesc(in_d);
    EXPECT(od[0].dtype == DataType::s8 && od[0].rank == 2 && od[0].dims[0] == 2 && od[0].dims[1] == 3);
    TensorView out = view(shape, DataType::s8, y.p);
    EXPECT(op->compute(out, ins) == Status::ok);
    const auto q = y.download<int8_t>();
    EXPECT(q[0] == 0 && q[1] == 0 && q[2] == 1 && q[3] == 10 && q[4] == 6 && q[5] == 4);

    g_case = "dequantize_linear_2d_per_channel";
    const int8_t xq_h[6] = {0, 0, 1, 10, 5, 4};
    DevBuf xq(xq_h, sizeof(xq_h)), f(24);
    attrs.output_dtype = DataType::f32;
    auto dq = DequantizeLinear::create(attrs, Backend::CUDA);
    const TensorView dins[] = {view(shape, DataType::s8, xq.p), view(ps, DataType::f32, sc.p), view(ps, DataType::s8, zp.p)};
    TensorView fout = view(shape, DataType::f32, f.p);
    EXPECT(dq->compute(fout, dins) == Status::ok);
    const auto r = f.download<float>();
    EXPECT(r[0] == 0.0f && r[1] == 0.0f && r[2] == 3.0f && r[3] == 10.0f && r[4] == 10.0f && r[5] == 12.0f);

    g_case = "quant_linear_contract";
    // A 64-bit float side is no dtype of this operator; a wrong scale dtype is an argument error.
    const TensorView bad_scale[] = {view(shape, DataType::f32, x.p), view(ps, DataType::s8, sc.p), view(ps, DataType::s8, zp.p)};
    EXPECT(op->compute(out, bad_scale) == Status::invalid_argument);
    const TensorView two[] = {view(shape, DataType::f32, x.p), view(ps, DataType::f32, sc.p)};
    EXPECT(op->compute(out, std::span<const TensorView>(two, 2)) == Status::invalid_argument);
    const auto after = y.download<int8_t>();
    EXPECT(after == q);  // rejected calls wrote nothing
}

struct QuantCase {
    std::vector<int64_t> shape;
    int64_t axis;
    int64_t params;  // 1 = per tensor
    bool f16, u8;
};

static void quant_linear_case(const QuantCase& c, const char* name, cudaStream_t stream)
{
    g_case = name;
    int64_t numel = 1;
    for (int64_t d : c.shape) numel *= d;
    int64_t outer = 1, rows = 1, inner = numel;
    if (c.params > 1 && c.axis < 0) {
        inner = c.shape.back();
        rows = numel / inner;
    } else if (c.params > 1) {
        inner = 1;
        for (size_t d = 0; d < c.shape.size(); ++d) {
            if (static_cast<int64_t>(d) < c.axis) outer *= c.shape[d];
            if (static_cast<int64_t>(d) > c.axis) inner *= c.shape[d];
        }
        rows = c.shape[static_cast<size_t>(c.axis)];
    }
    std::mt19937_64 rng(numel * 7 + c.params);
    std::normal_distribution<float> nd(0.0f, 60.0f);
    std::uniform_real_distribution<float> us(0.05f, 3.0f);
    std::vector<float> scale(c.params);
    std::vector<uint8_t> zp(c.params);
    for (auto& v : scale) v = us(rng);
    for (auto& v : zp) v = static_cast<uint8_t>(rng() % 256);
    std::vector<float> xf(numel);
    for (int64_t i = 0; i < numel; ++i) {
        xf[i] = (i % 5 == 0) ? (static_cast<float>(static_cast<int>(rng() % 180) - 90) + 0.5f) * scale[0] : nd(rng);
    }
    std::vector<uint16_t> xh(numel);
    for (int64_t i = 0; i < numel; ++i) xh[i] = oracle_f32_to_f16(xf[i]);
    const void* x_host = c.f16 ? static_cast<const void*>(xh.data()) : static_cast<const void*>(xf.data());
    const size_t fsz = c.f16 ? 2 : 4;
    const DataType fdt = c.f16 ? DataType::f16 : DataType::f32;
    const DataType qdt = c.u8 ? DataType::u8 : DataType::s8;

    std::vector<uint8_t> want_q(numel), xq(numel);
    oracle_quantize_linear(x_host, c.f16, outer, rows, inner, scale.data(), zp.data(), c.u8, want_q.data(), c.u8, 1);
    for (auto& v : xq) v = static_cast<uint8_t>(rng() % 256);
    std::vector<uint8_t> want_f(numel * fsz);
    oracle_dequantize_linear(xq.data(), c.u8, outer, rows, inner, scale.data(), zp.data(), c.u8, want_f.data(), c.f16);

    DevBuf dx(x_host, numel * fsz), dsc(scale.data(), scale.size() * 4), dzp(zp.data(), zp.size()), dq(numel, 0x11);
    DevBuf dxq(xq.data(), numel), df(numel * fsz, 0x11);
    const std::span<const int64_t> sh(c.shape.data(), c.shape.size());
    const int64_t ps[] = {c.params};
    QuantLinearAttributes attrs;
    attrs.axis = c.axis;
    attrs.output_dtype = qdt;
    ComputeContext ctx;
    ctx.expected_backend = Backend::CUDA;
    ctx.cuda_stream = stream;
    {
        auto op = QuantizeLinear::create(attrs, Backend::CUDA);
        TensorView out(sh, qdt, dq.p);
        const TensorView ins[] = {TensorView(sh, fdt, dx.p), view(ps, DataType::f32, dsc.p), view(ps, qdt, dzp.p)};
        EXPECT(op->compute(out, ins, ctx) == Status::ok);
        EXPECT(dq.download<uint8_t>() == want_q);
    }
    attrs.output_dtype = fdt;
    {
        auto op = DequantizeLinear::create(attrs, Backend::CUDA);
        TensorView out(sh, fdt, df.p);
        const TensorView ins[] = {TensorView(sh, qdt, dxq.p), view(ps, DataType::f32, dsc.p), view(ps, qdt, dzp.p)};
        EXPECT(op->compute(out, ins, ctx) == Status::ok);
        EXPECT(df.download<uint8_t>() == want_f);
    }
#ifdef NNB200_USE_NNOPS_HEADERS
    // The reference's own CPU operators on the same bytes.
    {
        std::vector<uint8_t> cpu_q(numel), cpu_f(numel * fsz);
        attrs.output_dtype = qdt;
        auto qop = QuantizeLinear::create(attrs, Backend::CPU);
        TensorView qo(sh, qdt, cpu_q.data());
        const TensorView qins[] = {TensorView(sh, fdt, const_cast<void*>(x_host)), view(ps, DataType::f32, scale.data()),
                                   view(ps, qdt, zp.data())};
        EXPECT(qop->compute(qo, qins) == Status::ok);
        EXPECT(cpu_q == want_q);
        attrs.output_dtype = fdt;
        auto dop = DequantizeLinear::create(attrs, Backend::CPU);
        TensorView fo(sh, fdt, cpu_f.data());
        const TensorView dins[] = {TensorView(sh, qdt, xq.data()), view(ps, DataType::f32, scale.data()),
                                   view(ps, qdt, zp.data())};
        EXPECT(dop->compute(fo, dins) == Status::ok);
        EXPECT(cpu_f == want_f);
    }
#endif
}

// ---- int8 Conv2D (reference tests/test_cuda_conv2d.cpp:252-500) -----------------------------

struct ConvCase {
    int64_t n, ic, ih, iw, oc, kh, kw, sh, sw, dh, dw, ph, pw, groups;
    DataType adt, odt;
    bool bias, relu;
    int auto_pad;   // 0 = explicit padding, 1 = SAME_UPPER
    bool packed;    // run a second time through prepackWeights
};

// Expected value: the gather written out (taps outside the image hold the activation's zero
// point) and the C oracle's int8 matmul per group.
static std::vector<uint8_t> conv_expected(const ConvCase& c, int64_t oh, int64_t ow, int64_t ph, int64_t pw,
                                          const std::vector<uint8_t>& x, const std::vector<int8_t>& w,
                                          const void* bias_host, int32_t zp_x, const std::vector<float>& sw,
                                          const std::vector<int32_t>& zw, float out_scale, int32_t out_zp)
{
    const int64_t icg = c.ic / c.groups, ocg = c.oc / c.groups, k = c.kh * c.kw * icg, pixels = c.n * oh * ow;
    const size_t osz = data_type_size(c.odt);
    const bool int_out = kind_of(c.odt) <= 2;
    std::vector<uint8_t> want(static_cast<size_t>(pixels * c.oc) * osz, 0);
    std::vector<uint8_t> col(static_cast<size_t>(pixels * k));
    std::vector<int8_t> wt(static_cast<size_t>(ocg * k));
    for (int64_t g = 0; g < c.groups; ++g) {
        for (int64_t p = 0; p < pixels; ++p) {
            const int64_t b = p / (oh * ow), y = (p / ow) % oh, xo = p % ow;
            for (int64_t a = 0; a < c.kh; ++a) {
                for (int64_t bb = 0; bb < c.kw; ++bb) {
                    const int64_t iy = y * c.sh - ph + a * c.dh, ix = xo * c.sw - pw + bb * c.dw;
                    for (int64_t ch = 0; ch < icg; ++ch) {
                        uint8_t v = static_cast<uint8_t>(zp_x);
                        if (iy >= 0 && iy < c.ih && ix >= 0 && ix < c.iw) {
                            v = x[static_cast<size_t>(((b * c.ih + iy) * c.iw + ix) * c.ic + g * icg + ch)];
                        }
                        col[static_cast<size_t>(p * k + (a * c.kw + bb) * icg + ch)] = v;
                    }
                }
            }
        }
        for (int64_t o = 0; o < ocg; ++o) {
            for (int64_t kk = 0; kk < k; ++kk) {
                wt[static_cast<size_t>(o * k + kk)] = w[static_cast<size_t>(kk * c.oc + g * ocg + o)];
            }
        }
        oracle_gemm_i8_args o{};
        o.a = col.data(); o.w = wt.data();
        o.out = want.data() + static_cast<size_t>(g * ocg) * osz;
        o.m = pixels; o.n = ocg; o.k = k;
        o.a_stride_m = k; o.a_stride_k = 1; o.w_stride_n = k; o.w_stride_k = 1; o.ldc = c.oc;
        o.a_unsigned = c.adt == DataType::u8;
        o.out_kind = kind_of(c.odt);
        o.bias = bias_host ? static_cast<const uint8_t*>(bias_host) + static_cast<size_t>(g * ocg) * (int_out ? 4 : osz) : nullptr;
        o.relu = c.relu;
        o.scale_w = sw.data() + g * ocg;
        o.zp_w = zw.data() + g * ocg;
        o.scale_a_scalar = 0.0078125f; o.scale_w_scalar = 1.0f;
        o.zp_a_scalar = zp_x;
        o.out_scale = out_scale; o.out_zp = out_zp;
        o.min_clip = -INFINITY; o.max_clip = INFINITY;
        oracle_gemm_i8(&o);
    }
    return want;
}

static void conv2d_i8_case(const ConvCase& c, const char* name, cudaStream_t stream)
{
    g_case = name;
    std::mt19937_64 rng(c.ic * 977 + c.oc * 31 + c.ih);
    const int64_t icg = c.ic / c.groups;
    std::vector<uint8_t> x(static_cast<size_t>(c.n * c.ih * c.iw * c.ic));
    for (auto& v : x) v = static_cast<uint8_t>(rng() & 0xFF);
    std::vector<int8_t> w(static_cast<size_t>(c.kh * c.kw * icg * c.oc));
    for (auto& v : w) v = static_cast<int8_t>(static_cast<int>(rng() % 255) - 127);
    std::vector<float> sw(c.oc);
    std::vector<int32_t> zw(c.oc);
    for (int64_t i = 0; i < c.oc; ++i) {
        sw[i] = 0.008f + 0.001f * static_cast<float>(i % 5);
        zw[i] = static_cast<int32_t>(i % 7) - 3;
    }
    const bool int_out = kind_of(c.odt) <= 2;
    const size_t osz = data_type_size(c.odt);
    std::vector<int32_t> bias_i(c.oc);
    std::vector<float> bias_f(c.oc);
    std::vector<uint16_t> bias_h(c.oc);
    for (int64_t i = 0; i < c.oc; ++i) {
        bias_i[i] = static_cast<int32_t>(rng() % 2001) - 1000;
        bias_f[i] = 0.0005f * static_cast<float>(bias_i[i]);
        bias_h[i] = oracle_f32_to_f16(bias_f[i]);
    }
    const void* bias_host = !c.bias ? nullptr
                            : int_out ? static_cast<const void*>(bias_i.data())
                                      : (c.odt == DataType::f32 ? static_cast<const void*>(bias_f.data())
                                                                : static_cast<const void*>(bias_h.data()));
    const int32_t zp_x = c.adt == DataType::u8 ? 128 : -6;
    const float out_scale = 0.03f;
    const int32_t out_zp = c.odt == DataType::u8 ? 110 : 0;

    Conv2DAttributes attrs;
    attrs.kernel_size = {c.kh, c.kw};
    attrs.stride = {c.sh, c.sw};
    attrs.dilation = {c.dh, c.dw};
    attrs.padding = {c.ph, c.pw};
    attrs.groups = c.groups;
    attrs.output_dtype = c.odt;
    attrs.auto_pad = c.auto_pad == 1 ? Conv2DAttributes::AutoPad::SAME_UPPER : Conv2DAttributes::AutoPad::NOTSET;
    if (c.relu) attrs.epilogue.type = EpilogueActivateType::Relu;

    QuantParams qa = per_tensor(0.0078125f, zp_x);
    QuantParams qw = arrays(sw.data(), zw.data(), c.oc, QuantGranularity::PerChannel);   // HOST arrays: the contract
    const QuantParams qc = per_tensor(out_scale, out_zp);
    DevBuf dx(x.data(), x.size()), dw(w.data(), w.size());
    DevBuf dbias(bias_host ? bias_host : static_cast<const void*>(bias_i.data()), static_cast<size_t>(c.oc) * (int_out ? 4 : osz));
    const int64_t xs[] = {c.n, c.ih, c.iw, c.ic}, ws[] = {c.kh, c.kw, icg, c.oc}, bs[] = {c.oc};
    TensorView xv(xs, c.adt, dx.p, TensorLayout::NHWC, qa);
    TensorView wv(ws, DataType::s8, dw.p, TensorLayout::HWIO, qw);
    TensorView bv(bs, int_out ? DataType::s32 : c.odt, dbias.p);

    auto op = Conv2D::create(attrs, Backend::CUDA);
    std::vector<TensorDesc> in_d = {xv.desc(), wv.desc()};
    std::vector<TensorView> ins = {xv, wv};
    if (c.bias) {
        in_d.push_back(bv.desc());
        ins.push_back(bv);
    }
    const TensorDesc od = op->getOutputTensorDesc(in_d).front();
    EXPECT(od.rank == 4 && od.dtype == c.odt && od.dims[0] == c.n && od.dims[3] == c.oc);
    const int64_t oh = od.dims[1], ow = od.dims[2];
    int64_t ph = c.ph, pw = c.pw;
    if (c.auto_pad == 1) {
        const int64_t th = std::max<int64_t>(0, (oh - 1) * c.sh + (c.kh - 1) * c.dh + 1 - c.ih);
        const int64_t tw = std::max<int64_t>(0, (ow - 1) * c.sw + (c.kw - 1) * c.dw + 1 - c.iw);
        ph = th / 2;
        pw = tw / 2;
    }
    const auto want = conv_expected(c, oh, ow, ph, pw, x, w, bias_host, zp_x, sw, zw, out_scale, out_zp);
    DevBuf dout(want.size(), 0x5A);
    const int64_t os[] = {c.n, oh, ow, c.oc};
    TensorView ov(os, c.odt, dout.p, TensorLayout::NHWC, qc);
    ComputeContext ctx;
    ctx.expected_backend = Backend::CUDA;
    ctx.cuda_stream = stream;
    EXPECT(op->compute(ov, ins, ctx) == Status::ok);
    const auto got = dout.download<uint8_t>();
    EXPECT(got == want);

    if (c.packed) {
        // Two-step prepack: query, allocate, fill; the packed call is bit-identical.
        TensorView packed;
        const TensorView pin[] = {wv};
        TensorView pout[] = {packed};
        op->prepackWeights(pin, pout, ctx);
        EXPECT(pout[0].is_empty() && pout[0].rank() == 2 && pout[0].layout() == TensorLayout::PackedHWIOCuda &&
               pout[0].shape(0) == c.oc);
        DevBuf blob(static_cast<size_t>(pout[0].numel()));
        const int64_t pshape[] = {pout[0].shape(0), pout[0].shape(1)};
        TensorView filled(pshape, DataType::s8, blob.p, pout[0].shape(1), TensorLayout::PackedHWIOCuda, qw);
        TensorView pout2[] = {filled};
        op->prepackWeights(pin, pout2, ctx);
        DevBuf dout2(want.size(), 0x5A);
        TensorView ov2(os, c.odt, dout2.p, TensorLayout::NHWC, qc);
        std::vector<TensorView> ins2 = ins;
        ins2[1] = filled;
        EXPECT(op->compute(ov2, ins2, ctx) == Status::ok);
        EXPECT(dout2.download<uint8_t>() == want);
    }

#ifdef NNB200_USE_NNOPS_HEADERS
    // The reference's own CPU route on the same bytes.
    std::vector<uint8_t> cpu(want.size(), 0x5A);
    TensorView hx(xs, c.adt, x.data(), TensorLayout::NHWC, qa);
    TensorView hw(ws, DataType::s8, w.data(), TensorLayout::HWIO, qw);
    TensorView hb(bs, int_out ? DataType::s32 : c.odt, const_cast<void*>(bias_host));
    TensorView ho(os, c.odt, cpu.data(), TensorLayout::NHWC, qc);
    std::vector<TensorView> hins = {hx, hw};
    if (c.bias) hins.push_back(hb);
    auto cpu_op = Conv2D::create(attrs, Backend::CPU);
    EXPECT(cpu_op->compute(ho, hins) == Status::ok);
    EXPECT(cpu == got);
#endif
}

static void conv2d_contract_cases()
{
    g_case = "conv2d_contract";
    // An s32 destination has no Conv2D route (tests/test_cuda_conv2d.cpp:503-528); neither has a
    // Winograd request or a residual add on the quantized route.
    std::vector<uint8_t> a(1 * 8 * 8 * 4, 1);
    std::vector<int8_t> w(3 * 3 * 4 * 6, 1);
    DevBuf da(a.data(), a.size()), dw(w.data(), w.size()), dout(6 * 6 * 6 * 4, 0x5A);
    const int64_t as[] = {1, 8, 8, 4}, ws[] = {3, 3, 4, 6}, cs[] = {1, 6, 6, 6};
    TensorView av(as, DataType::u8, da.p, TensorLayout::NHWC, per_tensor(0.01f, 128));
    TensorView wv(ws, DataType::s8, dw.p, TensorLayout::HWIO, per_tensor(0.01f, 0));
    ComputeContext ctx;
    ctx.expected_backend = Backend::CUDA;
    const TensorView ins[] = {av, wv};
    {
        TensorView cv(cs, DataType::s32, dout.p, TensorLayout::NHWC);
        Conv2DAttributes attrs;
        attrs.kernel_size = {3, 3};
        attrs.output_dtype = DataType::s32;
        auto op = Conv2D::create(attrs, Backend::CUDA);
        EXPECT(op->compute(cv, ins, ctx) == Status::unsupported);
    }
    {
        TensorView cv(cs, DataType::s8, dout.p, TensorLayout::NHWC, per_tensor(0.05f, 0));
        Conv2DAttributes attrs;
        attrs.kernel_size = {3, 3};
        attrs.output_dtype = DataType::s8;
        attrs.add_to = true;
        auto op = Conv2D::create(attrs, Backend::CUDA);
        EXPECT(op->compute(cv, ins, ctx) == Status::unsupported);
    }
    const auto canary = dout.download<uint8_t>();
    bool untouched = true;
    for (uint8_t v : canary) untouched = untouched && v == 0x5A;
    EXPECT(untouched);   // a rejected call writes nothing
}

int main()
{
    int dev_count = 0;
    if (cudaGetDeviceCount(&dev_count) != cudaSuccess || dev_count == 0) {
        std::printf("SKIP: no CUDA device\n");
        return 77;
    }
    cudaStream_t stream;
    CUDA_OK(cudaStreamCreate(&stream));

    kat_basic_s32();
    kat_zero_points();
    kat_u8_zero_points();
    kat_requant();

    const DataType kinds[] = {DataType::s32, DataType::s8, DataType::u8, DataType::f32, DataType::f16};
    for (DataType dt : kinds) {
        const std::string n1 = "linear_i8_per_channel_" + std::to_string(int(dt));
        linear_i8_case({1, 200, 330, 512, dt, true, true, true, false, false, 0, 0, 0}, n1.c_str(), nullptr);
        const std::string n2 = "linear_i8_zero_points_" + std::to_string(int(dt));
        linear_i8_case({1, 77, 130, 272, dt, false, true, true, true, false, 0, 0, 0}, n2.c_str(), stream);
    }
    linear_i8_case({1, 150, 200, 260, DataType::s8, true, false, true, false, false, 28, 12, 24}, "linear_i8_pitched", stream);
    linear_i8_case({1, 130, 140, 100, DataType::s32, false, false, false, true, false, 0, 0, 0}, "linear_i8_unaligned_k", nullptr);
    linear_i8_case({3, 64, 96, 128, DataType::s8, true, true, true, true, false, 0, 0, 0}, "linear_i8_batched", stream);
    linear_i8_case({1, 8, 520, 1024, DataType::s8, true, false, true, false, false, 0, 0, 0}, "linear_i8_decode_m8", nullptr);
    linear_i8_case({1, 256, 384, 512, DataType::s8, true, true, true, true, true, 0, 0, 0}, "linear_i8_device_arrays", stream);
    linear_i8_case({1, 512, 1024, 1024, DataType::s8, true, false, true, false, false, 0, 0, 0}, "linear_i8_512x1024x1024", nullptr);

    linear_q4_1_case(4, 260, 1024, false, "linear_q4_1_gemv_f32");
    linear_q4_1_case(1, 512, 4096, true, "linear_q4_1_gemv_f16");
    linear_q4_1_case(160, 384, 512, true, "linear_q4_1_gemm_f16");
    linear_q4_1_case(130, 300, 1000, false, "linear_q4_1_gemm_f32_ragged");

    contract_cases();

    linear_fp_act_case(1, 200, 330, 512, false, true, true, true, "linear_fp_act_f32_per_token_zp", stream);
    linear_fp_act_case(1, 77, 130, 272, true, false, true, false, "linear_fp_act_f16_per_tensor_zp", nullptr);
    linear_fp_act_case(1, 8, 520, 1024, true, true, false, true, "linear_fp_act_f16_decode_m8", stream);
    linear_fp_act_case(3, 64, 96, 128, false, true, true, false, "linear_fp_act_f32_batched_per_token", stream);
    linear_fp_act_case(1, 130, 140, 100, false, false, false, true, "linear_fp_act_f32_unaligned_k", nullptr);

#ifndef NNB200_USE_NNOPS_HEADERS
    prepack_case(false, 77, 130, 272, "prepack_linear_nk", stream);
    prepack_case(true, 200, 330, 1000, "prepack_matmul_kn_storage", stream);
    prepack_case(false, 4, 520, 1024, "prepack_linear_decode", nullptr);
    prepack_q4_1_case(1, 520, 4096, false, "prepack_q4_1_gemv_f32", stream);
    prepack_q4_1_case(3, 260, 1024, true, "prepack_q4_1_gemv_f16", nullptr);
    prepack_q4_1_case(300, 384, 512, true, "prepack_q4_1_two_pass_f16", stream);
#endif

    conv2d_i8_case({1, 16, 8, 8, 8, 3, 3, 1, 1, 1, 1, 1, 1, 1, DataType::u8, DataType::s8, true, true, 0, true}, "conv2d_i8_3x3_u8_s8", stream);
    conv2d_i8_case({1, 16, 8, 8, 8, 3, 3, 2, 1, 1, 1, 1, 1, 1, DataType::u8, DataType::f16, true, true, 0, false}, "conv2d_i8_stride_f16", nullptr);
    conv2d_i8_case({1, 16, 8, 8, 8, 3, 3, 1, 1, 2, 1, 1, 1, 1, DataType::s8, DataType::f16, true, true, 0, false}, "conv2d_i8_dilated_f16", stream);
    conv2d_i8_case({1, 16, 12, 12, 16, 3, 3, 1, 1, 1, 1, 1, 1, 2, DataType::u8, DataType::u8, true, true, 0, true}, "conv2d_i8_groups_u8", stream);
    conv2d_i8_case({1, 16, 8, 8, 16, 3, 3, 1, 1, 1, 1, 1, 1, 16, DataType::s8, DataType::u8, true, true, 0, true}, "conv2d_i8_one_channel_groups", nullptr);
    conv2d_i8_case({2, 64, 28, 28, 128, 1, 1, 1, 1, 1, 1, 0, 0, 1, DataType::s8, DataType::s8, true, false, 0, true}, "conv2d_i8_pointwise", stream);
    conv2d_i8_case({1, 32, 32, 32, 24, 3, 3, 1, 1, 1, 1, 1, 1, 1, DataType::s8, DataType::s8, true, true, 0, false}, "conv2d_i8_oc24", stream);
    conv2d_i8_case({1, 256, 14, 14, 256, 3, 3, 1, 1, 1, 1, 1, 1, 1, DataType::s8, DataType::s8, true, true, 0, true}, "conv2d_i8_k2304", stream);
    conv2d_i8_case({1, 64, 56, 56, 64, 3, 3, 1, 1, 1, 1, 1, 1, 1, DataType::u8, DataType::s8, true, true, 0, false}, "conv2d_i8_3136_pixels", stream);
    conv2d_i8_case({1, 128, 7, 7, 128, 3, 3, 1, 1, 1, 1, 1, 1, 1, DataType::s8, DataType::f32, false, false, 0, false}, "conv2d_i8_f32_no_bias", nullptr);
    conv2d_i8_case({2, 3, 33, 31, 32, 7, 7, 2, 2, 1, 1, 0, 0, 1, DataType::u8, DataType::s8, true, true, 1, true}, "conv2d_i8_stem_same_upper", stream);
    conv2d_contract_cases();

    kat_quant_linear();
    quant_linear_case({{64, 4096}, -1, 1, false, false}, "quant_linear_per_tensor_f32_s8", stream);
    quant_linear_case({{70001}, -1, 1, true, true}, "quant_linear_per_tensor_ragged_f16_u8", nullptr);
    quant_linear_case({{200, 1028}, -1, 200, false, true}, "quant_linear_per_token_f32_u8", stream);
    quant_linear_case({{37, 75}, -1, 37, true, false}, "quant_linear_per_token_ragged_f16_s8", nullptr);
    quant_linear_case({{5, 12, 24}, 1, 12, false, false}, "quant_linear_per_channel_axis1", stream);
    quant_linear_case({{4, 100, 64}, 0, 4, true, true}, "quant_linear_per_channel_axis0_f16", stream);
    quant_linear_case({{6, 50}, 1, 50, false, true}, "quant_linear_per_channel_last_axis", nullptr);

    CUDA_OK(cudaDeviceSynchronize());
    CUDA_OK(cudaStreamDestroy(stream));
    std::printf("%s: %d checks, %d failed\n", g_failed == 0 ? "PASS" : "FAIL", g_checks, g_failed);
    return g_failed == 0 ? 0 : 1;
}
