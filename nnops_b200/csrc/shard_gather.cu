// Reassembly of a column-sharded output after an all-gather.
//
// N-sharded Linear: rank r owns output channels [r*n_per, (r+1)*n_per) and produces a dense
// [M, n_per] slab.  An all-gather concatenates the slabs rank-major, [g][M][n_per]; this
// kernel rewrites them as the row-major [M, g*n_per] matrix the single-GPU call would have
// produced.  Pure data movement: 16-byte loads and stores, grid sized from the SM count.
// (The reference has no multi-GPU code; this sits above its operator API.)

#include "internal.cuh"
#include "ptx.cuh"

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

// Flags of one rank: slot r holds the last epoch rank r announced here, slot kEpochSlot this
// rank's own call count.
constexpr int kEpochSlot = 8;

struct RankFlags {
    int32_t* by_rank[8];
};

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v)
{
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p)
{
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One warp per GPU.  Lane 0 advances this rank's epoch; lane r (r != rank) announces it in rank
// r's flag array and then polls the local slot r until rank r has announced the same epoch.
// The epoch lives in device memory, so a captured launch stays valid on replay.  The wait is
// bounded: on expiry the lane records kErrPeerWait, sets the host-visible poison word (so that
// the host refuses the next sharded call without having to synchronise) and the kernel
// returns.  A rank that finds the poison already set does not wait at all: its output is
// already suspect, and skipping keeps a poisoned pipeline from stalling one limit per step.
__global__ void rank_barrier_kernel(const RankFlags flags, const int world, const int rank, const long long limit_cycles,
                                    int32_t* error_word, int32_t* poison)
{
    const int lane = static_cast<int>(threadIdx.x);
    int32_t* mine = flags.by_rank[rank];
    int32_t epoch = 0;
    if (lane == 0) {
        epoch = mine[kEpochSlot] + 1;
        mine[kEpochSlot] = epoch;
    }
    epoch = __shfl_sync(0xFFFFFFFFu, epoch, 0);
    const bool poisoned = poison != nullptr && *reinterpret_cast<volatile int32_t*>(poison) != 0;
    if (lane < world && lane != rank) {
        st_release_sys(flags.by_rank[lane] + rank, epoch);
        if (poisoned) {
            atomicCAS(error_word, 0, kErrPeerWait);
            return;
        }
        const long long t0 = clock64();
        uint32_t spins = 0;
        while (static_cast<int32_t>(static_cast<uint32_t>(ld_acquire_sys(mine + lane)) - static_cast<uint32_t>(epoch)) < 0) {
            if ((++spins & 0x3Fu) == 0 && clock64() - t0 > limit_cycles) {
                atomicCAS(error_word, 0, kErrPeerWait);
                if (poison != nullptr) {
                    *reinterpret_cast<volatile int32_t*>(poison) = 1;
                    __threadfence_system();
                }
                break;
            }
        }
    }
}

}  // namespace

int launch_rank_barrier(int32_t* const* flags_by_rank, int world, int rank, long long limit_cycles,
                        int32_t* poison, const DeviceInfo& dev, cudaStream_t stream)
{
    RankFlags f;
    for (int r = 0; r < 8; ++r) {
        f.by_rank[r] = r < world ? flags_by_rank[r] : nullptr;
    }
    // Ranks of one job drift apart by far more than a pipeline stage ever waits (a lazy module
    // load, a collector pause, a data loader on one rank), so the default limit here is about
    // half a minute of SM clocks, not the two seconds of the in-kernel pipeline waits.
    constexpr long long kRankBarrierLimitCycles = 60'000'000'000LL;
    rank_barrier_kernel<<<1, 32, 0, stream>>>(f, world, rank, limit_cycles > 0 ? limit_cycles : kRankBarrierLimitCycles,
                                              dev.error_word, poison);
    note_launch();
    return cuda_status(cudaGetLastError());
}

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
