// Prepacked int8 weights: the device blob behind the operators' two-step prepackWeights
// contract (reference include/nnops/core/op_base.hpp:72-80: an empty outputs[0] asks for the
// packed form's geometry, a populated one is filled).  The reference's CUDA front end answers
// "no packed form" (src/ops/linear.cpp:125-128) and its launcher therefore pays on EVERY call
// for staging the per-channel arrays from pageable host memory and for sweeping W again to get
// its row sums (src/backend/cuda/matmul/matmul_i8.cuh:323-376, matmul_i8_common.cuh:270-350).
//
// Blob for a weight of N channels and K inputs, N * (pitch + 12) bytes, pitch = K rounded up to 16:
//
//   [0, N*pitch)            W as [N][pitch] s8, k-contiguous, zero padded -- whatever pose the
//                           source had ([N,K] or [K,N], any pitch), so the tensor-core and decode
//                           engines' alignment rules always hold afterwards
//   + N*4                   scale_w[N] f32   (1.0 when the weight is per-tensor)
//   + N*4                   zp_w[N]    s32   (0 likewise)
//   + N*4                   r_w[N]     s32   sum_k W[n][k], so a call with activation zero points
//                                            does not read W twice
//
// One kernel transposes / copies 64 x 64 tiles through shared memory (coalesced along whichever
// direction the source is contiguous in) and accumulates the row sums with integer atomics
// (exact and order-independent).

#include <cstring>

#include "internal.cuh"

namespace nnb200 {

namespace {

constexpr int kTile = 64;

__global__ void __launch_bounds__(256) pack_i8_kernel(const int8_t* __restrict__ w, const int64_t n, const int64_t k,
                                                      const int64_t stride_n, const int64_t stride_k,
                                                      int8_t* __restrict__ dst, const int64_t pitch,
                                                      int32_t* __restrict__ r_w)
{
    __shared__ int8_t tile[kTile][kTile + 4];  // [n][k]
    const int64_t n0 = static_cast<int64_t>(blockIdx.y) * kTile;
    const int64_t k0 = static_cast<int64_t>(blockIdx.x) * kTile;
    const bool k_fast = stride_k == 1 || stride_n != 1;  // walk k fastest unless only n is contiguous
    for (int i = threadIdx.x; i < kTile * kTile; i += 256) {
        const int r = k_fast ? i / kTile : i % kTile;  // n index inside the tile
        const int c = k_fast ? i % kTile : i / kTile;  // k index inside the tile
        int8_t v = 0;
        if (n0 + r < n && k0 + c < k) {
            v = w[(n0 + r) * stride_n + (k0 + c) * stride_k];
        }
        tile[r][c] = v;
    }
    __syncthreads();
    // Write dense rows (pad columns beyond k, up to the pitch, with zeros) and sum each row:
    // four threads per row, 16 bytes each.
    const int r = threadIdx.x >> 2;
    const int q = threadIdx.x & 3;
    const bool row_ok = n0 + r < n;  // rows past n hold zeros in the tile
    int32_t sum = 0;
    uint32_t words[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t word = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int8_t v = tile[r][q * 16 + j * 4 + b];
            sum += v;
            word |= static_cast<uint32_t>(static_cast<uint8_t>(v)) << (8 * b);
        }
        words[j] = word;
    }
    const int64_t col = k0 + q * 16;
    if (row_ok && col < pitch) {  // pitch is a multiple of 16: the 16-byte piece is entirely inside or outside
        *reinterpret_cast<uint4*>(dst + (n0 + r) * pitch + col) = make_uint4(words[0], words[1], words[2], words[3]);
    }
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);  // every lane takes part; invalid rows contribute zeros
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    if (row_ok && q == 0 && sum != 0) {
        atomicAdd(&r_w[n0 + r], sum);
    }
}

__global__ void __launch_bounds__(256) fill_params_kernel(float* scale, int32_t* zp, int64_t n, float s, int32_t z,
                                                          int fill_scale, int fill_zp)
{
    const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i < n) {
        if (fill_scale) {
            scale[i] = s;
        }
        if (fill_zp) {
            zp[i] = z;
        }
    }
}

}  // namespace

int64_t i8_pack_pitch(int64_t k)
{
    return (k + 15) / 16 * 16;
}

int launch_i8_pack(const void* w, int64_t n, int64_t k, int64_t stride_n, int64_t stride_k, const float* scale_w,
                   float scale_scalar, const int32_t* zp_w, int32_t zp_scalar, void* blob, cudaStream_t stream)
{
    const int64_t pitch = i8_pack_pitch(k);
    uint8_t* base = static_cast<uint8_t*>(blob);
    float* scale_d = reinterpret_cast<float*>(base + n * pitch);
    int32_t* zp_d = reinterpret_cast<int32_t*>(base + n * pitch + n * 4);
    int32_t* rw_d = reinterpret_cast<int32_t*>(base + n * pitch + n * 8);
    if (cudaMemsetAsync(rw_d, 0, static_cast<size_t>(n) * 4, stream) != cudaSuccess) {
        return NNB200_INTERNAL;
    }
    // Per-channel arrays may live on the host or on the device: a default-kind copy takes both.
    if (scale_w != nullptr &&
        cudaMemcpyAsync(scale_d, scale_w, static_cast<size_t>(n) * 4, cudaMemcpyDefault, stream) != cudaSuccess) {
        return NNB200_INTERNAL;
    }
    if (zp_w != nullptr &&
        cudaMemcpyAsync(zp_d, zp_w, static_cast<size_t>(n) * 4, cudaMemcpyDefault, stream) != cudaSuccess) {
        return NNB200_INTERNAL;
    }
    if (scale_w == nullptr || zp_w == nullptr) {
        fill_params_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
            scale_d, zp_d, n, scale_scalar, zp_scalar, scale_w == nullptr, zp_w == nullptr);
        note_launch();
    }
    // The grid covers the padded pitch so the pad columns are written (as zeros) too.
    const dim3 grid(static_cast<unsigned>((pitch + kTile - 1) / kTile), static_cast<unsigned>((n + kTile - 1) / kTile));
    if (grid.y > 65535u) {
        return NNB200_UNSUPPORTED;
    }
    pack_i8_kernel<<<grid, 256, 0, stream>>>(static_cast<const int8_t*>(w), n, k, stride_n, stride_k,
                                             reinterpret_cast<int8_t*>(base), pitch, rw_d);
    note_launch();
    return cuda_status(cudaGetLastError());
}

// ---- Q4_1: (d, m) plane and nibble plane ------------------------------------------------------
// One thread per block: five 4-byte reads of the raw stream, one 16-byte and one 4-byte store.
namespace {

__global__ void __launch_bounds__(256) pack_q4_1_kernel(const uint32_t* __restrict__ w, const int64_t ldw_words,
                                                        const int64_t n, const int64_t nblk,
                                                        uint4* __restrict__ qs, const int64_t qs_pitch,
                                                        uint32_t* __restrict__ dm, const int64_t dm_pitch)
{
    const int64_t total = n * nblk;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t row = i / nblk;
        const int64_t b = i - row * nblk;
        const uint32_t* src = w + row * ldw_words + b * 5;
        dm[row * dm_pitch + b] = src[0];
        qs[row * qs_pitch + b] = make_uint4(src[1], src[2], src[3], src[4]);
    }
}

}  // namespace

int64_t q4_1_pack_qs_pitch(int64_t k) { return (k + 31) / 32; }                    // in 16-byte blocks
int64_t q4_1_pack_dm_pitch(int64_t k) { return (((k + 31) / 32) + 3) / 4 * 4; }    // in 4-byte entries: 16-byte rows

int launch_q4_1_pack(const void* w_blocks, int64_t ldw_blocks, int64_t n, int64_t k, void* blob, cudaStream_t stream)
{
    const int64_t nblk = (k + 31) / 32;
    if (n == 0 || nblk == 0) {
        return NNB200_OK;
    }
    const int64_t qs_pitch = q4_1_pack_qs_pitch(k);
    const int64_t dm_pitch = q4_1_pack_dm_pitch(k);
    uint8_t* base = static_cast<uint8_t*>(blob);
    uint4* qs = reinterpret_cast<uint4*>(base);
    uint32_t* dm = reinterpret_cast<uint32_t*>(base + static_cast<size_t>(n) * qs_pitch * 16);
    // The pad entries of the (d, m) rows are never read; clear them anyway so the blob is reproducible.
    if (dm_pitch != nblk) {
        if (cudaMemsetAsync(dm, 0, static_cast<size_t>(n) * dm_pitch * 4, stream) != cudaSuccess) {
            return NNB200_INTERNAL;
        }
    }
    const int64_t total = n * nblk;
    const unsigned grid = static_cast<unsigned>(total / 256 + 1 > 4096 ? 4096 : total / 256 + 1);
    pack_q4_1_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint32_t*>(w_blocks), ldw_blocks * 5, n, nblk, qs, qs_pitch,
                                               dm, dm_pitch);
    note_launch();
    return cuda_status(cudaGetLastError());
}

}  // namespace nnb200
