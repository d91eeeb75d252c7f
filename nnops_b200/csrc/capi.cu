// extern "C" entry points of libnnb200 (declared in include/nnb200.h): argument checks,
// engine choice, per-device state, TMA descriptor encoding.

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstring>
#include <mutex>

#include "internal.cuh"
#include "ptx.cuh"

namespace nnb200 {

namespace {

// One error word per device; kernels reach it through DeviceInfo::error_word.
__device__ int32_t g_error_word;

std::atomic<uint64_t> g_launches{0};

DeviceInfo g_devices[kMaxDevices];
std::mutex g_device_mutex;
std::atomic<bool> g_device_ok[kMaxDevices];

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn()
{
    // The driver entry point is looked up at run time so the library does not link libcuda.
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &qres) !=
                cudaSuccess ||
            qres != cudaDriverEntryPointSuccess) {
            return static_cast<EncodeTiledFn>(nullptr);
        }
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

}  // namespace

const DeviceInfo* current_device_info()
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        return nullptr;
    }
    // Only a successful look-up is remembered: one that failed (the device not usable yet, a
    // call made during stream capture) clears the CUDA error it raised and is tried again by
    // the next call.
    if (g_device_ok[dev].load(std::memory_order_acquire)) {
        return &g_devices[dev];
    }
    std::lock_guard<std::mutex> lock(g_device_mutex);
    if (g_device_ok[dev].load(std::memory_order_relaxed)) {
        return &g_devices[dev];
    }
    DeviceInfo d;
    d.device = dev;
    bool ok = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess;
    ok = ok && cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess;
    ok = ok && cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev) == cudaSuccess;
    void* p = nullptr;
    // The symbol's name is a host-side handle; kernels need its device address, which
    // differs per device, so it is resolved with that device current.
    ok = ok && cudaGetSymbolAddress(&p, g_error_word) == cudaSuccess;
    d.error_word = static_cast<int32_t*>(p);
    if (ok) {
        const int32_t zero = 0;
        ok = cudaMemcpy(d.error_word, &zero, sizeof(zero), cudaMemcpyHostToDevice) == cudaSuccess;
    }
    if (!ok) {
        (void)cudaGetLastError();
        return nullptr;
    }
    g_devices[dev] = d;
    g_device_ok[dev].store(true, std::memory_order_release);
    return &g_devices[dev];
}

namespace {
std::mutex g_poison_mutex;
PeerPoison g_poison[kMaxDevices];
}

PeerPoison peer_poison_for_current_device(bool create)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        return PeerPoison{};
    }
    std::lock_guard<std::mutex> lock(g_poison_mutex);
    if (g_poison[dev].host == nullptr && create) {
        void* h = nullptr;
        void* d = nullptr;
        if (cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
            (void)cudaGetLastError();
            return PeerPoison{};
        }
        std::memset(h, 0, 64);
        if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) {
            (void)cudaGetLastError();
            cudaFreeHost(h);
            return PeerPoison{};
        }
        g_poison[dev].host = static_cast<volatile int32_t*>(h);
        g_poison[dev].device = static_cast<int32_t*>(d);
    }
    return g_poison[dev];
}

namespace {
std::atomic<int> g_knobs[NNB200_KNOB_COUNT] = {{-1}, {-1}, {-1}, {-1}, {-1}, {-1}, {-1}, {-1}, {-1}};
}

int knob(int id)
{
    return (id >= 0 && id < NNB200_KNOB_COUNT) ? g_knobs[id].load(std::memory_order_relaxed) : -1;
}

void note_launch(int n)
{
    g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed);
}

bool make_tma_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t cols, uint64_t rows,
                 uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows, bool swizzle128)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) {
        return false;
    }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUtensorMapDataType dt = elem_bytes == 1   ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_UINT32;
    const CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// An NHWC 8-bit activation as a 4-D tensor {c, w, h, n} (innermost first) with byte strides for
// w, h, n; box = {box_c, box_w, box_h, 1}, 128-byte swizzle, zero fill outside the tensor.
bool make_tma_nhwc_u8(CUtensorMap* map, const void* base, uint64_t c, uint64_t w, uint64_t h, uint64_t n,
                      uint64_t stride_w, uint64_t stride_h, uint64_t stride_n, uint32_t box_c, uint32_t box_w,
                      uint32_t box_h, uint32_t step_w, uint32_t step_h)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr || box_w * step_w > 256 || box_h * step_h > 256) {
        return false;
    }
    const cuuint64_t dims[4] = {c, w, h, n};
    const cuuint64_t strides[3] = {stride_w, stride_h, stride_n};
    // The box is given as the span it covers in the tensor; the element strides thin it out.
    const cuuint32_t box[4] = {box_c, box_w * step_w, box_h * step_h, 1};
    const cuuint32_t elem_strides[4] = {1, step_w, step_h, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, elem_strides,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

namespace {

bool valid_i8_args(const nnb200_gemm_i8_args* a)
{
    if (a == nullptr || a->m < 0 || a->n < 0 || a->k < 0 || a->batch < 0) {
        return false;
    }
    if (a->out_kind < NNB200_OUT_S32 || a->out_kind > NNB200_OUT_F16) {
        return false;
    }
    if (a->m == 0 || a->n == 0 || a->batch == 0) {
        return true;
    }
    if (a->a == nullptr || a->w == nullptr || a->out == nullptr || a->k == 0) {
        return false;
    }
    if (a->ldc < a->n) {
        return false;
    }
    if ((a->a_stride_k != 1 && a->a_stride_m != 1) || (a->w_stride_k != 1 && a->w_stride_n != 1)) {
        return false;  // one of the two strides of each operand is the contiguous one
    }
    // Natural alignment of everything a kernel reads or writes as 2- or 4-byte words, and the
    // workspace's 16 bytes: a misaligned pointer is refused here instead of faulting on the GPU.
    const auto misaligned = [](const void* p, uintptr_t to) { return (reinterpret_cast<uintptr_t>(p) & (to - 1)) != 0; };
    const uintptr_t out_align = a->out_kind == NNB200_OUT_S32 || a->out_kind == NNB200_OUT_F32 ? 4
                              : a->out_kind == NNB200_OUT_F16 ? 2 : 1;
    const uintptr_t bias_align = a->out_kind == NNB200_OUT_F16 ? 2 : 4;
    if (misaligned(a->out, out_align) || misaligned(a->bias, bias_align) || misaligned(a->scale_a, 4) ||
        misaligned(a->scale_w, 4) || misaligned(a->zp_a, 4) || misaligned(a->zp_w, 4) || misaligned(a->r_w, 4) ||
        misaligned(a->workspace, 16)) {
        return false;
    }
    return true;
}

bool needs_compensation(const nnb200_gemm_i8_args* a)
{
    return a->zp_a_scalar != 0 || a->zp_w_scalar != 0 || (a->zp_a != nullptr && a->zp_a_nonzero != 0) ||
           (a->zp_w != nullptr && a->zp_w_nonzero != 0);
}

I8Problem problem_of(const nnb200_gemm_i8_args* a, int64_t b)
{
    I8Problem p;
    p.a = static_cast<const uint8_t*>(a->a) + b * a->a_batch_stride;
    p.w = static_cast<const uint8_t*>(a->w) + b * a->w_batch_stride;
    p.m = a->m;
    p.n = a->n;
    p.k = a->k;
    p.a_stride_m = a->a_stride_m;
    p.a_stride_k = a->a_stride_k;
    p.w_stride_n = a->w_stride_n;
    p.w_stride_k = a->w_stride_k;
    p.a_unsigned = a->a_unsigned;
    return p;
}

// The call writes a column window of a sharded output (peer stores or multicast stores).
bool sharded_out(const nnb200_gemm_i8_args* a)
{
    return a->num_peer_outs != 0 || a->multicast_out != nullptr;
}

int pick_i8_engine(const nnb200_gemm_i8_args* a, const I8Problem& p)
{
    if (a->force_engine == NNB200_ENGINE_GENERIC) {
        return NNB200_ENGINE_GENERIC;
    }
    if (a->force_engine == NNB200_ENGINE_NARROW) {
        return narrow_i8_supported(p) ? NNB200_ENGINE_NARROW : NNB200_ENGINE_GENERIC;
    }
    if (a->force_engine == NNB200_ENGINE_UMMA) {
        return umma_i8_supported(p) ? NNB200_ENGINE_UMMA : NNB200_ENGINE_GENERIC;
    }
    if (a->force_engine == NNB200_ENGINE_DECODE) {
        return decode_i8_supported(p) ? NNB200_ENGINE_DECODE : NNB200_ENGINE_GENERIC;
    }
    if (a->force_engine == NNB200_ENGINE_SKINNY) {
        return (!sharded_out(a) && skinny_i8_supported(p)) ? NNB200_ENGINE_SKINNY : NNB200_ENGINE_GENERIC;
    }
    // Few activation rows: the cost is streaming W once, and what decides is how evenly an engine
    // spreads that stream over the SMs (crossovers measured on four layer shapes):
    //   * up to 8 rows the streaming warp-MMA engine (16 channels per CTA);
    //   * 9..16 rows: the same while the layer has at most 96 tiles of 128 channels, beyond that the
    //     tensor-core engine with the weights as the 128-row operand;
    //   * 17..128 rows: a layer with so few channels that even 64-wide tiles of the square engine
    //     leave SMs idle is served best by exactly those; otherwise weights-as-rows up to 64 rows,
    //     and above while the layer has 256-channel tiles for less than half the SMs.
    if (!sharded_out(a)) {
        const bool decode_ok = decode_i8_supported(p);
        const bool skinny_ok = skinny_i8_supported(p);
        const DeviceInfo* dev = current_device_info();
        const int64_t sms = dev != nullptr ? dev->sm_count : 148;
        const int64_t tiles128 = (p.n + 127) / 128;
        if (decode_ok && (p.m <= 8 || !skinny_ok || tiles128 <= 96)) {
            return NNB200_ENGINE_DECODE;
        }
        if (skinny_ok) {
            const bool narrow_layer = p.m > 16 && (p.n + 63) / 64 <= sms;
            if (!narrow_layer && (p.m <= 64 || (p.n + 255) / 256 < sms / 2)) {
                return NNB200_ENGINE_SKINNY;
            }
        }
    }
    if (!sharded_out(a) && narrow_i8_supported(p)) {
        return NNB200_ENGINE_NARROW;
    }
    if (umma_i8_supported(p)) {
        return NNB200_ENGINE_UMMA;
    }
    return NNB200_ENGINE_GENERIC;
}

size_t out_elem_bytes(int kind)
{
    return (kind == NNB200_OUT_S32 || kind == NNB200_OUT_F32) ? 4 : (kind == NNB200_OUT_F16 ? 2 : 1);
}

// Self-test of the bounded pipeline waits: one thread waits on a barrier nothing ever arrives
// at.  The wait has to run out after `limit_cycles`, raise the CTA's abort flag and record
// kErrSelfTest in the device's error word; the kernel then returns normally.
__global__ void wait_selftest_kernel(long long limit_cycles, int32_t* error_word)
{
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&bar, 1);
        mbar_init_fence();
        if (!mbar_wait(&bar, 0, &abort_flag, limit_cycles)) {
            atomicCAS(error_word, 0, kErrSelfTest);
        }
    }
}

}  // namespace
}  // namespace nnb200

using namespace nnb200;

extern "C" {

size_t nnb200_gemm_i8_min_workspace_bytes(const nnb200_gemm_i8_args* a)
{
    if (!valid_i8_args(a) || a->m == 0 || a->n == 0 || a->batch == 0) {
        return 0;
    }
    if (!needs_compensation(a)) {
        return 0;
    }
    // R_a [batch][m] and R_w [batch][n], each padded to 256 bytes.
    const size_t ra = (static_cast<size_t>(a->m) * 4 + 255) & ~size_t(255);
    const size_t rw = (static_cast<size_t>(a->n) * 4 + 255) & ~size_t(255);
    return static_cast<size_t>(a->batch) * (ra + rw);
}

// Scratch that lets the few-row tensor-core engine share K evenly among all SMs (optional), and
// whether having it changes the engine: on a layer with so few channels that the square engine
// was chosen for its narrow tiles (17..128 rows), weights-as-rows with shared K is faster still
// when K is long (N=4096, K=14336, 24 rows: 24.4 against 35.9 us) -- but only with the scratch.
struct I8SplitPlan {
    size_t bytes;         // scratch wanted beyond the required minimum (0 = no use for it)
    bool switches_engine; // with the scratch the call runs on the weights-as-rows engine instead
};

static I8SplitPlan i8_split_plan(const nnb200_gemm_i8_args* a)
{
    I8SplitPlan plan{0, false};
    if (a->batch != 1 || sharded_out(a)) {
        return plan;
    }
    const DeviceInfo* dev = current_device_info();
    if (dev == nullptr) {
        return plan;
    }
    const I8Problem p = problem_of(a, 0);
    const int engine = pick_i8_engine(a, p);
    if (engine == NNB200_ENGINE_SKINNY) {
        plan.bytes = skinny_i8_split_bytes(p, *dev);
    } else if (engine == NNB200_ENGINE_UMMA && a->force_engine == NNB200_ENGINE_AUTO && p.m >= 17 && p.m <= 128) {
        plan.bytes = skinny_i8_split_bytes(p, *dev);  // 0 unless weights-as-rows is supported and the split pays
        plan.switches_engine = plan.bytes > 0;
    } else if (engine == NNB200_ENGINE_DECODE && a->force_engine == NNB200_ENGINE_AUTO && p.m > 8 &&
               p.n * p.k >= (int64_t{80} << 20)) {
        // 9..16 rows on a layer of modest width: the streaming engine costs ~0.23 us per MB of weights,
        // weights-as-rows with shared K ~0.16 us per MB plus 5 us more up front; from about 80 MB the
        // latter wins (N=4096, K=28672, 12 rows: 30.5 against 33.6 us).
        plan.bytes = skinny_i8_split_bytes(p, *dev);
        plan.switches_engine = plan.bytes > 0;
    }
    return plan;
}

// The part of the caller's workspace that serves the split, or null when it is absent, too small or misaligned.
static void* i8_split_scratch(const nnb200_gemm_i8_args* a, size_t required, size_t split_bytes)
{
    if (split_bytes == 0 || a->workspace == nullptr || a->workspace_bytes < required + split_bytes ||
        ((reinterpret_cast<uintptr_t>(a->workspace) + required) & 15u) != 0) {
        return nullptr;
    }
    return static_cast<uint8_t*>(a->workspace) + required;
}

// Engine of batch element 0 given the workspace the block carries.
static int i8_engine_with_workspace(const nnb200_gemm_i8_args* a, void** split_scratch)
{
    const I8SplitPlan plan = i8_split_plan(a);
    void* scratch = i8_split_scratch(a, nnb200_gemm_i8_min_workspace_bytes(a), plan.bytes);
    if (split_scratch != nullptr) {
        *split_scratch = scratch;
    }
    if (plan.switches_engine && scratch != nullptr) {
        return NNB200_ENGINE_SKINNY;
    }
    return pick_i8_engine(a, problem_of(a, 0));
}

size_t nnb200_gemm_i8_workspace_bytes(const nnb200_gemm_i8_args* a)
{
    if (!valid_i8_args(a) || a->m == 0 || a->n == 0 || a->batch == 0) {
        return 0;
    }
    return nnb200_gemm_i8_min_workspace_bytes(a) + i8_split_plan(a).bytes;
}

int nnb200_gemm_i8_engine(const nnb200_gemm_i8_args* a)
{
    if (!valid_i8_args(a)) {
        return -1;
    }
    if (a->m == 0 || a->n == 0 || a->batch == 0) {
        return pick_i8_engine(a, problem_of(a, 0));
    }
    return i8_engine_with_workspace(a, nullptr);
}

int nnb200_gemm_i8(const nnb200_gemm_i8_args* a, void* stream_v)
{
    if (!valid_i8_args(a)) {
        return NNB200_INVALID_ARGUMENT;
    }
    if (a->m == 0 || a->n == 0 || a->batch == 0) {
        return NNB200_OK;
    }
    const DeviceInfo* dev = current_device_info();
    if (dev == nullptr) {
        return NNB200_INTERNAL;
    }
    if (dev->cc_major != 10) {
        return NNB200_UNSUPPORTED;  // sm_100a only: there is no other code path
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const bool comp = needs_compensation(a);
    const size_t need = nnb200_gemm_i8_min_workspace_bytes(a);
    if (need > 0 && (a->workspace == nullptr || a->workspace_bytes < need)) {
        return NNB200_INVALID_ARGUMENT;
    }
    // The rest of the workspace, when there is enough of it, lets the few-row engine share K
    // among the SMs (and on narrow layers with a long K makes it the engine of choice).
    void* split_scratch = nullptr;
    const int engine0 = i8_engine_with_workspace(a, &split_scratch);
    const size_t ra_bytes = (static_cast<size_t>(a->m) * 4 + 255) & ~size_t(255);
    const size_t rw_bytes = (static_cast<size_t>(a->n) * 4 + 255) & ~size_t(255);

    if (sharded_out(a)) {
        // A rank barrier that ran out of time earlier leaves the gathered outputs suspect.
        const PeerPoison poison = peer_poison_for_current_device(false);
        if (poison.host != nullptr && *poison.host != 0) {
            return NNB200_INTERNAL;
        }
        // Sharded write-back: validated here so that a refused call has launched nothing.
        const auto mis16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; };
        bool ok = a->num_peer_outs >= 0 && a->num_peer_outs <= 7 && a->batch == 1 &&
                  (a->out_kind == NNB200_OUT_S8 || a->out_kind == NNB200_OUT_U8) && (a->ldc % 16) == 0 &&
                  (a->n % 16) == 0 && !mis16(a->out) &&
                  pick_i8_engine(a, problem_of(a, 0)) == NNB200_ENGINE_UMMA;
        for (int i = 0; ok && i < a->num_peer_outs; ++i) {
            ok = a->peer_out[i] != nullptr && !mis16(a->peer_out[i]);
        }
        if (a->multicast_out != nullptr) {
            ok = ok && a->num_peer_outs == 0 && !mis16(a->multicast_out);
        }
        if (!ok) {
            return NNB200_UNSUPPORTED;
        }
    }

    // Launchability of every batch element is settled before the first launch, so that a
    // refusal leaves the outputs untouched: the generic engine's grid has 65535 rows of 32.
    for (int64_t b = 0; b < a->batch; ++b) {
        const int e = a->batch == 1 ? engine0 : pick_i8_engine(a, problem_of(a, b));
        if (e == NNB200_ENGINE_GENERIC && (a->m + 31) / 32 > 65535) {
            return NNB200_UNSUPPORTED;
        }
    }

    for (int64_t b = 0; b < a->batch; ++b) {
        const I8Problem p = problem_of(a, b);
        I8Epilogue ep;
        std::memset(&ep, 0, sizeof(ep));
        ep.out = static_cast<uint8_t*>(a->out) + static_cast<size_t>(b * a->out_batch_stride) * out_elem_bytes(a->out_kind);
        ep.ldc = a->ldc;
        ep.out_kind = a->out_kind;
        ep.bias = a->bias;
        const bool int_out = a->out_kind <= NNB200_OUT_U8;
        ep.relu = int_out ? (a->relu != 0) : 0;
        ep.activation = int_out ? NNB200_ACT_NONE : a->activation;
        ep.act_alpha = a->act_alpha;
        ep.act_beta = a->act_beta;
        ep.min_clip = a->min_clip;
        ep.max_clip = a->max_clip;
        ep.scale_a = a->scale_a;
        ep.scale_w = a->scale_w;
        ep.zp_a = a->zp_a;
        ep.zp_w = a->zp_w;
        ep.scale_a_scalar = a->scale_a_scalar;
        ep.scale_w_scalar = a->scale_w_scalar;
        ep.zp_a_scalar = a->zp_a_scalar;
        ep.zp_w_scalar = a->zp_w_scalar;
        ep.compensate = comp ? 1 : 0;
        ep.k = static_cast<int32_t>(a->k);
        ep.out_scale = a->out_scale;
        ep.out_zp = a->out_zp;
        ep.mc_out = a->multicast_out;
        ep.num_peers = a->num_peer_outs;
        for (int i = 0; i < a->num_peer_outs; ++i) {
            ep.peer_out[i] = a->peer_out[i];
        }
        if (comp) {
            uint8_t* ws = static_cast<uint8_t*>(a->workspace) + static_cast<size_t>(b) * (ra_bytes + rw_bytes);
            int32_t* r_a = reinterpret_cast<int32_t*>(ws);
            int32_t* r_w = reinterpret_cast<int32_t*>(ws + ra_bytes);
            const bool have_rw = a->r_w != nullptr && (a->batch == 1 || a->w_batch_stride == 0);
            // R_a only multiplies weight zero points: without any, the sweep over A is skipped.
            // Likewise R_w only multiplies activation zero points.
            const bool need_ra = a->zp_w_scalar != 0 || (a->zp_w != nullptr && a->zp_w_nonzero != 0);
            const bool need_rw = a->zp_a_scalar != 0 || (a->zp_a != nullptr && a->zp_a_nonzero != 0);
            const bool sweep_w = need_rw && !have_rw;
            if (need_ra || sweep_w) {
                const int st = launch_i8_sums(p, need_ra ? r_a : nullptr, sweep_w ? r_w : nullptr, stream);
                if (st != NNB200_OK) {
                    return st;
                }
            }
            ep.r_a = need_ra ? r_a : nullptr;
            ep.r_w = !need_rw ? nullptr : (have_rw ? a->r_w : r_w);
        }
        int st;
        switch (a->batch == 1 ? engine0 : pick_i8_engine(a, p)) {
        case NNB200_ENGINE_UMMA: st = launch_gemm_i8_umma(p, ep, *dev, stream); break;
        case NNB200_ENGINE_NARROW: st = launch_gemm_i8_narrow(p, ep, *dev, stream); break;
        case NNB200_ENGINE_DECODE: st = launch_gemm_i8_decode(p, ep, *dev, stream); break;
        case NNB200_ENGINE_SKINNY: st = launch_gemm_i8_skinny(p, ep, *dev, split_scratch, stream); break;
        default: st = launch_gemm_i8_generic(p, ep, *dev, stream); break;
        }
        if (st != NNB200_OK) {
            return st;
        }
    }
    return NNB200_OK;
}

static bool valid_q4_args(const nnb200_q4_1_args* q)
{
    if (q == nullptr || q->m < 0 || q->n < 0 || q->k < 0) {
        return false;
    }
    if (q->m == 0 || q->n == 0) {
        return true;
    }
    if (q->a == nullptr || q->w_blocks == nullptr || q->out == nullptr || q->k == 0) {
        return false;
    }
    const int64_t nblk = (q->k + 31) / 32;
    if (q->w_dm != nullptr &&
        (q->ld_dm < nblk || (reinterpret_cast<uintptr_t>(q->w_dm) & 15u) != 0 ||
         (reinterpret_cast<uintptr_t>(q->w_blocks) & 15u) != 0 || (q->ld_dm % 4) != 0)) {
        return false;   // the planes of a packed weight are 16-byte aligned, rows included
    }
    return q->lda >= q->k && q->ldc >= q->n && q->ldw_blocks >= nblk;
}

// Rows of activations from which expanding the weights once and running a dense GEMM beats
// decoding them inside the GEMM (measured on config 4's weights: equal at 128 rows, 64 us
// against 100 us at 256).
static constexpr int64_t kTwoPassMinRows = 256;
// f32 activations have no fused tensor-core form (their only other route walks the weights once
// per 8 rows): the two-pass form, with the activations split into [hi | lo] f16, serves them from here up.
static constexpr int64_t kTwoPassMinRowsF32 = 17;

static int64_t two_pass_min_rows(const nnb200_q4_1_args* q)
{
    return q->a_f16 != 0 ? kTwoPassMinRows : kTwoPassMinRowsF32;
}

size_t nnb200_q4_1_workspace_bytes(const nnb200_q4_1_args* q)
{
    if (!valid_q4_args(q) || q->m == 0 || q->n == 0) {
        return 0;
    }
    // Optional: without it a tall call runs the fused kernel.
    const bool wanted = q->force_engine == 5 || (q->force_engine == 0 && q->m >= two_pass_min_rows(q));
    return wanted ? q4_1_two_pass_scratch_bytes(*q) : 0;
}

int nnb200_q4_1_engine(const nnb200_q4_1_args* q)
{
    if (!valid_q4_args(q)) {
        return -1;
    }
    if (q->w_dm != nullptr) {
        // Packed weights (separate nibble and (d, m) planes): the two-pass GEMM for tall calls that
        // bring its scratch, else the deferred-scaling GEMV; -1 when neither can take the call.
        if (q->force_engine == 0 || q->force_engine == 5) {
            if (q->m >= two_pass_min_rows(q) && q4_1_two_pass_supported(*q)) {
                return 5;
            }
        }
        if (q->force_engine == 0 || q->force_engine == 2 || q->force_engine == 6) {
            return q4_1_gemv_dsq_supported(*q) ? 6 : -1;
        }
        return -1;
    }
    // 1 = fused tensor-core GEMM (tcgen05), 3 = GEMV on CUDA cores, 4 = GEMV with warp-level MMA
    // after per-weight dequantisation, 5 = two-pass GEMM (expand to f16 scratch, dense tcgen05
    // GEMM), 6 = GEMV with warp-level MMA on raw nibbles and deferred scaling.
    int gemv = 3;
    if (q->force_engine != 3) {
        // Deferred scaling pays one fix-up per (channel, block, activation column), so it wins where
        // the columns are few: one f16 row (4.6 against 4.7 us on a 10 MB matrix, 33 against 51 us on
        // 147 MB) and one f32 row (two columns); from two f16 rows on the per-weight form is faster
        // (M = 8 on 10 MB: 6.0 against 9.7 us).  Knob Q4_GEMV: 1 never, 2 whenever it can run.
        const int kn = knob(NNB200_KNOB_Q4_GEMV);
        const bool few_columns = q->m == 1;
        const bool prefer_dsq = q->force_engine == 6 || (q->force_engine != 4 && kn != 1 && (kn == 2 || few_columns));
        if (prefer_dsq && q4_1_gemv_dsq_supported(*q)) {
            gemv = 6;
        } else if (q4_1_gemv_mma_supported(*q)) {
            gemv = 4;
        }
    }
    if (q->force_engine == 2 || q->force_engine == 3 || q->force_engine == 4 || q->force_engine == 6) {
        return gemv;
    }
    const bool gemm_ok = q4_1_gemm_umma_supported(*q);
    const bool two_pass_ok = q4_1_two_pass_supported(*q);
    if (q->force_engine == 5) {
        return two_pass_ok ? 5 : (gemm_ok ? 1 : gemv);
    }
    if (q->force_engine == 1) {
        return gemm_ok ? 1 : gemv;
    }
    if (q->m >= two_pass_min_rows(q) && two_pass_ok) {
        return 5;
    }
    return (q->m > 8 && gemm_ok) ? 1 : gemv;
}

int nnb200_linear_q4_1(const nnb200_q4_1_args* q, void* stream_v)
{
    if (!valid_q4_args(q)) {
        return NNB200_INVALID_ARGUMENT;
    }
    if (q->m == 0 || q->n == 0) {
        return NNB200_OK;
    }
    if ((reinterpret_cast<uintptr_t>(q->w_blocks) & 3u) != 0) {
        return NNB200_UNSUPPORTED;  // blocks are read as 32-bit words
    }
    const DeviceInfo* dev = current_device_info();
    if (dev == nullptr) {
        return NNB200_INTERNAL;
    }
    if (dev->cc_major != 10) {
        return NNB200_UNSUPPORTED;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    switch (nnb200_q4_1_engine(q)) {
    case -1: return NNB200_UNSUPPORTED;   // packed weights in a shape no engine takes them in
    case 1: return launch_q4_1_gemm_umma(*q, *dev, stream);
    case 5: return launch_q4_1_two_pass(*q, *dev, stream);
    case 4: return launch_q4_1_gemv_mma(*q, *dev, stream);
    case 6: return launch_q4_1_gemv_dsq(*q, *dev, stream);
    default: return launch_q4_1_gemv(*q, *dev, stream);
    }
}

int nnb200_q4_1_decode(const void* w_blocks, int64_t ldw_blocks, int64_t rows, int64_t k, void* out, int32_t out_f16,
                       int64_t ld_out, void* stream)
{
    if (rows < 0 || k < 0 || (rows > 0 && k > 0 && (w_blocks == nullptr || out == nullptr)) || ld_out < k) {
        return NNB200_INVALID_ARGUMENT;
    }
    if ((reinterpret_cast<uintptr_t>(w_blocks) & 3u) != 0) {
        return NNB200_UNSUPPORTED;
    }
    return launch_q4_1_decode(w_blocks, ldw_blocks, rows, k, out, out_f16, ld_out, static_cast<cudaStream_t>(stream));
}

size_t nnb200_i8_pack_bytes(int64_t n, int64_t k)
{
    if (n <= 0 || k <= 0) {
        return 0;
    }
    return static_cast<size_t>(n) * static_cast<size_t>(i8_pack_pitch(k) + 12);
}

size_t nnb200_q4_1_pack_bytes(int64_t n, int64_t k)
{
    if (n <= 0 || k <= 0) {
        return 0;
    }
    return static_cast<size_t>(n) * (static_cast<size_t>(q4_1_pack_qs_pitch(k)) * 16 + static_cast<size_t>(q4_1_pack_dm_pitch(k)) * 4);
}

int nnb200_q4_1_packed_view(const void* blob, int64_t n, int64_t k, nnb200_q4_1_packed* view)
{
    if (blob == nullptr || view == nullptr || n <= 0 || k <= 0) {
        return NNB200_INVALID_ARGUMENT;
    }
    const uint8_t* base = static_cast<const uint8_t*>(blob);
    view->qs = base;
    view->qs_pitch = q4_1_pack_qs_pitch(k);
    view->dm = base + static_cast<size_t>(n) * static_cast<size_t>(view->qs_pitch) * 16;
    view->dm_pitch = q4_1_pack_dm_pitch(k);
    return NNB200_OK;
}

int nnb200_q4_1_pack(const void* w_blocks, int64_t ldw_blocks, int64_t n, int64_t k, void* blob, size_t blob_bytes,
                     void* stream)
{
    if (n < 0 || k < 0) {
        return NNB200_INVALID_ARGUMENT;
    }
    if (n == 0 || k == 0) {
        return NNB200_OK;
    }
    if (w_blocks == nullptr || blob == nullptr || ldw_blocks < (k + 31) / 32 ||
        (reinterpret_cast<uintptr_t>(w_blocks) & 3u) != 0 || (reinterpret_cast<uintptr_t>(blob) & 15u) != 0 ||
        blob_bytes < nnb200_q4_1_pack_bytes(n, k)) {
        return NNB200_INVALID_ARGUMENT;
    }
    const DeviceInfo* dev = current_device_info();
    if (dev == nullptr) {
        return NNB200_INTERNAL;
    }
    return launch_q4_1_pack(w_blocks, ldw_blocks, n, k, blob, static_cast<cudaStream_t>(stream));
}

int nnb200_i8_packed_view(const void* blob, int64_t n, int64_t k, nnb200_i8_packed* view)
{
    if (blob == nullptr || view == nullptr || n <= 0 || k <= 0) {
        return NNB200_INVALID_ARGUMENT;
    }
    const uint8_t* base = static_cast<const uint8_t*>(blob);
    const int64_t pitch = i8_pack_pitch(k);
    view->w = base;
    view->pitch = pitch;
    view->scale_w = reinterpret_cast<const float*>(base + n * pitch);
    view->zp_w = reinterpret_cast<const int32_t*>(base + n * pitch + n * 4);
    view->r_w = reinterpret_cast<const int32_t*>(base + n * pitch + n * 8);
    return NNB200_OK;
}

int nnb200_i8_pack(const void* w, int64_t n, int64_t k, int64_t w_stride_n, int64_t w_stride_k, const float* scale_w,
                   float scale_w_scalar, const int32_t* zp_w, int32_t zp_w_scalar, void* blob, size_t blob_bytes,
                   void* stream)
{
    if (n < 0 || k < 0) {
        return NNB200_INVALID_ARGUMENT;
    }
    if (n == 0 || k == 0) {
        return NNB200_OK;
    }
    if (w == nullptr || blob == nullptr || blob_bytes < nnb200_i8_pack_bytes(n, k) ||
        (reinterpret_cast<uintptr_t>(blob) & 15u) != 0 || (w_stride_n != 1 && w_stride_k != 1)) {
        return NNB200_INVALID_ARGUMENT;
    }
    const DeviceInfo* dev = current_device_info();
    if (dev == nullptr) {
        return NNB200_INTERNAL;
    }
    if (dev->cc_major != 10) {
        return NNB200_UNSUPPORTED;
    }
    return launch_i8_pack(w, n, k, w_stride_n, w_stride_k, scale_w, scale_w_scalar, zp_w, zp_w_scalar, blob,
                          static_cast<cudaStream_t>(stream));
}

static int quant_linear_call(const nnb200_quant_linear_args* q, void* stream, bool quantize)
{
    if (q == nullptr || q->outer < 0 || q->rows < 0 || q->inner < 0) {
        return NNB200_INVALID_ARGUMENT;
    }
    if (q->outer == 0 || q->rows == 0 || q->inner == 0) {
        return NNB200_OK;
    }
    if (q->x == nullptr || q->y == nullptr || q->scale == nullptr || q->zero_point == nullptr ||
        q->zp_unsigned < NNB200_ZP_S8 || q->zp_unsigned > NNB200_ZP_S32) {
        return NNB200_INVALID_ARGUMENT;
    }
    if (q->zp_unsigned == NNB200_ZP_S32 && (reinterpret_cast<uintptr_t>(q->zero_point) & 3u) != 0) {
        return NNB200_INVALID_ARGUMENT;
    }
    // The element count must fit the kernels' 64-bit signed indexing.
    if (q->outer > INT64_MAX / q->rows || q->outer * q->rows > INT64_MAX / q->inner) {
        return NNB200_INVALID_ARGUMENT;
    }
    const DeviceInfo* dev = current_device_info();
    if (dev == nullptr) {
        return NNB200_INTERNAL;
    }
    if (dev->cc_major != 10) {
        return NNB200_UNSUPPORTED;
    }
    return quantize ? launch_quantize_linear(*q, *dev, static_cast<cudaStream_t>(stream))
                    : launch_dequantize_linear(*q, *dev, static_cast<cudaStream_t>(stream));
}

int nnb200_quantize_linear(const nnb200_quant_linear_args* q, void* stream)
{
    return quant_linear_call(q, stream, true);
}

int nnb200_dequantize_linear(const nnb200_quant_linear_args* q, void* stream)
{
    return quant_linear_call(q, stream, false);
}

int nnb200_interleave_shards(const void* gathered, void* out, int64_t m, int64_t row_bytes_per_shard, int32_t shards,
                              int64_t out_pitch_bytes, void* stream)
{
    if (m < 0 || row_bytes_per_shard < 0 || shards < 1 || out_pitch_bytes < row_bytes_per_shard * shards) {
        return NNB200_INVALID_ARGUMENT;
    }
    if (m == 0 || row_bytes_per_shard == 0) {
        return NNB200_OK;
    }
    if (gathered == nullptr || out == nullptr) {
        return NNB200_INVALID_ARGUMENT;
    }
    if ((row_bytes_per_shard & 15) != 0 || (out_pitch_bytes & 15) != 0 ||
        (reinterpret_cast<uintptr_t>(gathered) & 15u) != 0 || (reinterpret_cast<uintptr_t>(out) & 15u) != 0) {
        return NNB200_UNSUPPORTED;
    }
    const DeviceInfo* dev = current_device_info();
    if (dev == nullptr) {
        return NNB200_INTERNAL;
    }
    return launch_interleave_shards(gathered, out, m, row_bytes_per_shard, shards, out_pitch_bytes, *dev,
                                    static_cast<cudaStream_t>(stream));
}

int nnb200_rank_barrier(int32_t* const* flags_by_rank, int32_t world, int32_t rank, int64_t limit_cycles, void* stream)
{
    if (flags_by_rank == nullptr || world < 1 || world > 8 || rank < 0 || rank >= world || limit_cycles < 0) {
        return NNB200_INVALID_ARGUMENT;
    }
    for (int r = 0; r < world; ++r) {
        if (flags_by_rank[r] == nullptr || (reinterpret_cast<uintptr_t>(flags_by_rank[r]) & 3u) != 0) {
            return NNB200_INVALID_ARGUMENT;
        }
    }
    const DeviceInfo* dev = current_device_info();
    if (dev == nullptr) {
        return NNB200_INTERNAL;
    }
    // An earlier barrier on this device ran out of time: some rank's tiles may never have
    // landed, so every later sharded call is refused until nnb200_take_device_error has been
    // called (which reports code 8 and clears the state).
    const PeerPoison poison = peer_poison_for_current_device(true);
    if (poison.host == nullptr) {
        return NNB200_INTERNAL;
    }
    if (*poison.host != 0) {
        return NNB200_INTERNAL;
    }
    return launch_rank_barrier(flags_by_rank, world, rank, limit_cycles, poison.device, *dev,
                               static_cast<cudaStream_t>(stream));
}

int nnb200_take_device_error(int32_t* code)
{
    const DeviceInfo* dev = current_device_info();
    if (dev == nullptr || code == nullptr) {
        return NNB200_INTERNAL;
    }
    if (cudaDeviceSynchronize() != cudaSuccess) {
        return NNB200_INTERNAL;
    }
    if (cudaMemcpy(code, dev->error_word, sizeof(int32_t), cudaMemcpyDeviceToHost) != cudaSuccess) {
        return NNB200_INTERNAL;
    }
    const PeerPoison poison = peer_poison_for_current_device(false);
    if (poison.host != nullptr) {
        *poison.host = 0;
    }
    const int32_t zero = 0;
    return cuda_status(cudaMemcpy(dev->error_word, &zero, sizeof(zero), cudaMemcpyHostToDevice));
}

int nnb200_selftest_wait_limit(int64_t limit_cycles, void* stream)
{
    const DeviceInfo* dev = current_device_info();
    if (dev == nullptr) {
        return NNB200_INTERNAL;
    }
    if (limit_cycles < 1 || limit_cycles > 200'000'000) {
        return NNB200_INVALID_ARGUMENT;
    }
    wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_cycles, dev->error_word);
    note_launch();
    return cuda_status(cudaGetLastError());
}

int nnb200_copy_h2d_async(void* dst_device, const void* src_host, size_t bytes, void* stream)
{
    if (bytes == 0) {
        return NNB200_OK;
    }
    if (dst_device == nullptr || src_host == nullptr) {
        return NNB200_INVALID_ARGUMENT;
    }
    return cuda_status(
        cudaMemcpyAsync(dst_device, src_host, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
}

namespace {
// Stream-ordered scratch comes from a private pool per device that keeps its memory between
// calls (release threshold: never).  The device's default pool hands freed memory back to the
// driver at every synchronisation, which made each staged call pay for fresh physical memory
// (0.4 ms per int8 Linear with host-side scale arrays).  The reference does the same
// (src/backend/cuda/matmul/gemm_common.cuh:296-318).
std::mutex g_pool_mutex;
cudaMemPool_t g_pool[nnb200::kMaxDevices];
bool g_pool_ready[nnb200::kMaxDevices];

cudaMemPool_t scratch_pool_for_current_device()
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= nnb200::kMaxDevices) {
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_pool_mutex);
    if (!g_pool_ready[dev]) {
        cudaMemPoolProps props = {};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = dev;
        cudaMemPool_t pool = nullptr;
        if (cudaMemPoolCreate(&pool, &props) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        uint64_t keep = UINT64_MAX;
        if (cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep) != cudaSuccess) {
            (void)cudaGetLastError();
        }
        g_pool[dev] = pool;
        g_pool_ready[dev] = true;
    }
    return g_pool[dev];
}
}  // namespace

int nnb200_scratch_alloc_async(void** out, size_t bytes, void* stream)
{
    if (out == nullptr) {
        return NNB200_INVALID_ARGUMENT;
    }
    *out = nullptr;
    if (bytes == 0) {
        return NNB200_OK;
    }
    cudaMemPool_t pool = scratch_pool_for_current_device();
    const cudaError_t e = pool != nullptr ? cudaMallocFromPoolAsync(out, bytes, pool, static_cast<cudaStream_t>(stream))
                                          : cudaMallocAsync(out, bytes, static_cast<cudaStream_t>(stream));
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        return NNB200_OUT_OF_MEMORY;
    }
    return cuda_status(e);
}

int nnb200_scratch_free_async(void* p, void* stream)
{
    if (p == nullptr) {
        return NNB200_OK;
    }
    return cuda_status(cudaFreeAsync(p, static_cast<cudaStream_t>(stream)));
}

int nnb200_peer_buffer_alloc(void** ptr, size_t bytes)
{
    if (ptr == nullptr || bytes == 0) {
        return NNB200_INVALID_ARGUMENT;
    }
    *ptr = nullptr;
    const cudaError_t e = cudaMalloc(ptr, bytes);
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        return NNB200_OUT_OF_MEMORY;
    }
    return cuda_status(e);
}

int nnb200_peer_buffer_free(void* ptr)
{
    return ptr == nullptr ? NNB200_OK : cuda_status(cudaFree(ptr));
}

int nnb200_peer_buffer_export(const void* ptr, uint8_t handle[64])
{
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (ptr == nullptr || handle == nullptr) {
        return NNB200_INVALID_ARGUMENT;
    }
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(ptr));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return NNB200_INTERNAL;
    }
    std::memcpy(handle, &h, sizeof(h));
    return NNB200_OK;
}

int nnb200_peer_buffer_open(const uint8_t handle[64], void** ptr)
{
    if (ptr == nullptr || handle == nullptr) {
        return NNB200_INVALID_ARGUMENT;
    }
    *ptr = nullptr;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    // Opened with the ACCESSING device current: the driver maps the exporter's memory for this
    // device and enables the peer path between the two GPUs.
    const cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        cudaGetLastError();
        *ptr = nullptr;
        return e == cudaErrorPeerAccessUnsupported ? NNB200_UNSUPPORTED : NNB200_INTERNAL;
    }
    return NNB200_OK;
}

int nnb200_peer_buffer_close(void* ptr)
{
    return ptr == nullptr ? NNB200_OK : cuda_status(cudaIpcCloseMemHandle(ptr));
}

int nnb200_enable_peer_access(int32_t peer_device)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        return NNB200_INTERNAL;
    }
    if (peer_device == dev) {
        return NNB200_OK;
    }
    int can = 0;
    if (cudaDeviceCanAccessPeer(&can, dev, peer_device) != cudaSuccess || can == 0) {
        cudaGetLastError();
        return NNB200_UNSUPPORTED;
    }
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
        return NNB200_OK;
    }
    return cuda_status(e);
}

int nnb200_is_device_pointer(const void* p)
{
    if (p == nullptr) {
        return 0;
    }
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) ? 1 : 0;
}

uint64_t nnb200_launch_count(void)
{
    return g_launches.load(std::memory_order_relaxed);
}

int nnb200_measure_i8_mma_peak(int32_t iters, int32_t pattern, double* ops, void* stream)
{
    if (iters < 1 || iters > (1 << 21) || pattern < 0 || pattern > 3) {
        return NNB200_INVALID_ARGUMENT;   // the upper bound keeps the launch well inside the bounded wait
    }
    const DeviceInfo* dev = current_device_info();
    if (dev == nullptr) {
        return NNB200_INTERNAL;
    }
    if (dev->cc_major != 10) {
        return NNB200_UNSUPPORTED;
    }
    return launch_mma_i8_peak(iters, pattern, ops, *dev, static_cast<cudaStream_t>(stream));
}

int nnb200_set_knob(int id, int value)
{
    if (id < 0 || id >= NNB200_KNOB_COUNT) {
        return INT32_MIN;
    }
    return g_knobs[id].exchange(value < 0 ? -1 : value, std::memory_order_relaxed);
}

int nnb200_get_knob(int id)
{
    return (id >= 0 && id < NNB200_KNOB_COUNT) ? knob(id) : INT32_MIN;
}

const char* nnb200_version(void)
{
    return "nnb200 0.1 (sm_100a)";
}

}  // extern "C"
