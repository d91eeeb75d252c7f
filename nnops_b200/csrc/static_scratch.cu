// nnb200_gemm_i8_static_scratch: the zero-point-compensated int8 matmul for callers that
// cannot hand the library any scratch memory.
//
// Who needs this: an inference-engine plugin or a real-time loop that is given its input
// and output buffers by the host framework and is not allowed to call cudaMalloc (or any
// allocating routine) itself -- allocation takes a device-wide lock, may synchronise, and
// can fail long after start-up.  The compensated matmul needs two small int32 vectors of
// scratch (row sums of A and of W); nnb200_gemm_i8 takes them from the caller's workspace,
// this entry point keeps them in a fixed array inside the library image instead.
//
// Every GPU on which the library's device code gets loaded holds its own copy of the array
// until the process exits (with lazy module loading that is from the first use of a kernel or
// symbol of this file on that GPU, otherwise from library load).  All calls on one GPU share
// that copy: two calls that overlap on the GPU race on it, so the caller serialises them.

#include <cuda_runtime.h>

#include <mutex>

#include "internal.cuh"

namespace nnb200 {

namespace {

// Device-resident scratch, one copy per GPU.  In host code this name is only a handle for
// the symbol; the address kernels can use is looked up per device below.
static __device__ __align__(256) unsigned char g_static_scratch[NNB200_STATIC_SCRATCH_BYTES];

std::mutex g_scratch_mutex;
void* g_scratch_ptr[kMaxDevices];   // non-null once the lookup has succeeded on that device

// Device address of the current device's copy of the array; nullptr on failure.  The lookup
// runs with the caller's device current and is remembered only when it succeeds: a first call
// made too early (during stream capture, say) fails, clears the CUDA error it raised, and a
// later call tries again.
void* static_scratch_for_current_device()
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        g_scratch_ptr[dev] = p;
    }
    return g_scratch_ptr[dev];
}

}  // namespace
}  // namespace nnb200

extern "C" int nnb200_gemm_i8_static_scratch(const nnb200_gemm_i8_args* args, void* stream)
{
    using namespace nnb200;
    if (args == nullptr) {
        return NNB200_INVALID_ARGUMENT;
    }
    nnb200_gemm_i8_args local = *args;
    local.workspace = nullptr;
    local.workspace_bytes = 0;
    const size_t need = nnb200_gemm_i8_min_workspace_bytes(&local);
    if (need > static_cast<size_t>(NNB200_STATIC_SCRATCH_BYTES)) {
        // Too large for the fixed array: refuse before anything is launched.
        return NNB200_OUT_OF_MEMORY;
    }
    if (need > 0) {
        const DeviceInfo* info = current_device_info();
        if (info != nullptr && info->cc_major != 10) {
            return NNB200_UNSUPPORTED;  // the library image only holds sm_100a code, this array included
        }
        void* p = static_scratch_for_current_device();
        if (p == nullptr) {
            return NNB200_INTERNAL;
        }
        local.workspace = p;
        local.workspace_bytes = need;  // exactly the sums' share: the optional K-sharing scratch is not offered here
    }
    // The sums kernels overwrite every entry of R_a / R_w they later read, so the previous
    // call's contents never leak into this one and nothing has to be cleared.
    return nnb200_gemm_i8(&local, stream);
}
