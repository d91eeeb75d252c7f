// Reassembly of a column-sharded output after an all-gather.
//
// N-sharded Linear: rank r owns output channels [r*n_per, (r+1)*n_per) and produces a dense
// [M, n_per] slab.  An all-gather concatenates the slabs rank-major, [g][M][n_per]; this
// kernel rewrites them as the row-major [M, g*n_per] matrix the single-GPU call would have
// produced.  Pure data movement: 16-byte loads and stores, grid sized from the SM count.
// (The reference has no multi-GPU code; this sits above its operator API.)

#include "internal.cuh"

namespace nnb200 {

namespace {

__global__ void __launch_bounds__(256) interleave_shards_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                                int64_t m, int64_t vec_per_row, int g,
                                                                int64_t dst_pitch_vec)
{
    // src: [g][m][vec_per_row]   dst: [m][g * vec_per_row (pitch dst_pitch_vec)]
    const int64_t total = static_cast<int64_t>(g) * m * vec_per_row;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t v = i % vec_per_row;
        const int64_t row = (i / vec_per_row) % m;
        const int64_t r = i / (vec_per_row * m);
        dst[row * dst_pitch_vec + r * vec_per_row + v] = src[i];
    }
}

}  // namespace

int launch_interleave_shards(const void* src, void* dst, int64_t m, int64_t row_bytes_per_shard, int g,
                             int64_t dst_pitch_bytes, const DeviceInfo& dev, cudaStream_t stream)
{
    const int64_t vec_per_row = row_bytes_per_shard / 16;
    const int64_t total = static_cast<int64_t>(g) * m * vec_per_row;
    if (total == 0) {
        return NNB200_OK;
    }
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = static_cast<int64_t>(dev.sm_count) * 16;
    if (blocks > cap) {
        blocks = cap;
    }
    interleave_shards_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const uint4*>(src), static_cast<uint4*>(dst), m, vec_per_row, g, dst_pitch_bytes / 16);
    note_launch();
    return cuda_status(cudaGetLastError());
}

}  // namespace nnb200
