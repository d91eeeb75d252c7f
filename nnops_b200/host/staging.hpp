// Helpers shared by the host-side backend files (linear / matmul / conv2d): status mapping,
// output-kind mapping, and stream-ordered staging of host-side quantization arrays.
#pragma once

#ifdef NNB200_USE_NNOPS_HEADERS
#include "nnops/ops/linear.hpp"
#else
#include "nnops_b200/nnops_api.hpp"
#endif

#include "nnb200.h"

#include <algorithm>
#include <cstddef>
#include <cstdint>

namespace nnops::backend::cuda {

namespace b200_detail {

inline Status to_status(int code)
{
    return code >= 0 && code <= 5 ? static_cast<Status>(code) : Status::internal;
}

inline bool out_kind_of(DataType dt, int& kind)
{
    switch (dt) {
    case DataType::s32: kind = NNB200_OUT_S32; return true;
    case DataType::s8: kind = NNB200_OUT_S8; return true;
    case DataType::u8: kind = NNB200_OUT_U8; return true;
    case DataType::f32: kind = NNB200_OUT_F32; return true;
    case DataType::f16: kind = NNB200_OUT_F16; return true;
    default: return false;
    }
}

// One quantization array as the kernels want it: a device pointer (or null + scalar).
struct DeviceArray {
    const void* ptr = nullptr;
    bool any_nonzero = true;
};

// Stream-ordered staging of host-side quantization arrays plus the kernels' own scratch.
class Staging {
public:
    explicit Staging(void* stream) : stream_(stream) {}
    ~Staging()
    {
        if (base_ != nullptr) {
            nnb200_scratch_free_async(base_, stream_);
        }
    }
    Staging(const Staging&) = delete;
    Staging& operator=(const Staging&) = delete;

    /// Reserve room; call for every array before allocate().
    void reserve(const void* host, size_t bytes)
    {
        if (host != nullptr && nnb200_is_device_pointer(host) == 0) {
            total_ += (bytes + 255) & ~size_t(255);
        }
    }
    void reserve_raw(size_t bytes) { total_ += (bytes + 255) & ~size_t(255); }
    int allocate() { return total_ == 0 ? NNB200_OK : nnb200_scratch_alloc_async(&base_, total_, stream_); }

    /// Device address of `host` (copied if it is host memory); int32 arrays report whether any
    /// entry is non-zero so the backend can skip the zero-point sweeps.
    int place(const void* host, size_t bytes, bool scan_int32, DeviceArray& out)
    {
        out.ptr = nullptr;
        out.any_nonzero = true;
        if (host == nullptr) {
            return NNB200_OK;
        }
        if (nnb200_is_device_pointer(host) != 0) {
            out.ptr = host;
            return NNB200_OK;
        }
        if (scan_int32) {
            const int32_t* v = static_cast<const int32_t*>(host);
            out.any_nonzero = std::any_of(v, v + bytes / 4, [](int32_t x) { return x != 0; });
        }
        void* dst = static_cast<char*>(base_) + used_;
        used_ += (bytes + 255) & ~size_t(255);
        out.ptr = dst;
        return nnb200_copy_h2d_async(dst, host, bytes, stream_);
    }
    // Null when the request exceeds what was reserved.
    void* take_raw(size_t bytes)
    {
        const size_t padded = (bytes + 255) & ~size_t(255);
        if (base_ == nullptr || used_ + padded > total_) {
            return nullptr;
        }
        void* p = static_cast<char*>(base_) + used_;
        used_ += padded;
        return p;
    }

private:
    void* stream_;
    void* base_ = nullptr;
    size_t total_ = 0;
    size_t used_ = 0;
};

}  // namespace b200_detail

}  // namespace nnops::backend::cuda
