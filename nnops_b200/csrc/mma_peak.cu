// Measured int8 tensor rate: tcgen05.mma kind::i8 issued back to back on operand tiles that
// never leave shared memory.
//
// The roofline of the int8 GEMM needs a denominator that is a property of the part, not of a
// library: one CTA per SM holds one 128 x 128-byte A tile and one 256 x 128-byte W tile in shared
// memory (zero-filled or pseudo-random, in the 128-byte-swizzled K-major layout the GEMM uses), and a single
// thread issues `iters` groups of four M128 x N256 x K32 MMAs -- exactly the instruction, shape,
// descriptors and two alternating TMEM accumulators of gemm_i8_umma_kernel -- with nothing to
// wait for: no TMA, no epilogue, no global traffic.  What limits it is the tensor pipe and the
// power cap, which is what "peak" means for the GEMM.  Timed by the caller with events around
// the launch.  (The reference has no counterpart: it predates tcgen05.)

#include "internal.cuh"
#include "ptx.cuh"
#include "ptx_pair.cuh"

namespace nnb200 {

namespace {

constexpr int kPeakM = 128;
constexpr int kPeakN = 256;
constexpr int kPeakKBytes = 128;                        // one swizzle row = four K32 steps
constexpr int kPeakATile = kPeakM * kPeakKBytes;        // 16 KB
constexpr int kPeakBTile = kPeakN * kPeakKBytes;        // 32 KB
constexpr int kPeakSmem = kPeakATile + kPeakBTile + 1024;   // + alignment slack
constexpr int kPeakTmemCols = 512;                      // two 256-column accumulators

__global__ void __launch_bounds__(128, 1) mma_i8_peak_kernel(const int iters, const int pattern, const uint32_t idesc,
                                                             int32_t* error_word)
{
    extern __shared__ __align__(1024) uint8_t peak_smem[];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;

    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(peak_smem) + 1023) & ~uintptr_t(1023));
    // pattern 0: zeros (the pipe's issue rate, next to no switching power); 1: pseudo-random
    // bytes (what the same instruction stream holds once the operands toggle and the power cap
    // sets the clock).
    for (int i = threadIdx.x; i < (kPeakATile + kPeakBTile) / 16; i += blockDim.x) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (pattern != 0) {
            uint32_t h = static_cast<uint32_t>(i) * 2654435761u + blockIdx.x * 40503u + 0x9E3779B9u;
            h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
            v = make_uint4(h, h * 3266489917u + 1u, (h ^ 0xA5A5A5A5u) * 668265263u, h * 374761393u + 7u);
        }
        reinterpret_cast<uint4*>(tiles)[i] = v;
    }
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        abort_word = 0;
        mbar_init(&done_bar, 1);
        mbar_init_fence();
    }
    if (warp == 0) {
        tmem_alloc(&tmem_slot, kPeakTmemCols);
        tmem_relinquish();
    }
    fence_proxy_async_smem();   // the zero fill (generic proxy) must be visible to the MMA's reads
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;

    if (threadIdx.x == 0) {
        const uint64_t a_desc = umma_desc_sw128_kmajor(smem_u32(tiles));
        const uint64_t b_desc = umma_desc_sw128_kmajor(smem_u32(tiles + kPeakATile));
        for (int it = 0; it < iters; ++it) {
            const uint32_t d_tmem = tmem_base + static_cast<uint32_t>((it & 1) * kPeakN);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                umma_i8(d_tmem, a_desc + static_cast<uint64_t>(ks * 2), b_desc + static_cast<uint64_t>(ks * 2), idesc,
                        (it > 1 || ks > 0) ? 1u : 0u);
            }
        }
        umma_commit(&done_bar);   // arrives when every MMA above has completed
        if (!mbar_wait(&done_bar, 0, &abort_word)) {
            atomicCAS(error_word, 0, kErrMmaWait);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kPeakTmemCols);
    }
}

// The same loop in the CTA-pair form (cta_group::2): two CTAs of a cluster hold 128 rows of A and
// HALF of the 256 W rows each, the leader issues M256 x N256 x K32 MMAs that run on both SMs'
// tensor cores, each of which reads the other half of W out of its neighbour's shared memory.
// It answers whether that instruction form, with nothing else in the way, sustains the rate of
// the single-CTA form.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1)
mma_i8_peak_pair_kernel(const int iters, const int pattern, const uint32_t idesc, int32_t* error_word)
{
    extern __shared__ __align__(1024) uint8_t peak_smem[];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;

    constexpr int kBHalf = kPeakBTile / 2;
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(peak_smem) + 1023) & ~uintptr_t(1023));
    for (int i = threadIdx.x; i < (kPeakATile + kBHalf) / 16; i += blockDim.x) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (pattern != 0) {
            uint32_t h = static_cast<uint32_t>(i) * 2654435761u + blockIdx.x * 40503u + 0x9E3779B9u;
            h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
            v = make_uint4(h, h * 3266489917u + 1u, (h ^ 0xA5A5A5A5u) * 668265263u, h * 374761393u + 7u);
        }
        reinterpret_cast<uint4*>(tiles)[i] = v;
    }
    const int warp = threadIdx.x >> 5;
    const uint32_t rank = cluster_cta_rank();
    if (threadIdx.x == 0) {
        abort_word = 0;
        mbar_init(&done_bar, 1);
        mbar_init_fence();
    }
    if (warp == 0) {
        tmem_alloc_pair(&tmem_slot, kPeakTmemCols);
        tmem_relinquish_pair();
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;

    if (threadIdx.x == 0 && rank == 0) {
        const uint64_t a_desc = umma_desc_sw128_kmajor(smem_u32(tiles));
        const uint64_t b_desc = umma_desc_sw128_kmajor(smem_u32(tiles + kPeakATile));
        for (int it = 0; it < iters; ++it) {
            const uint32_t d_tmem = tmem_base + static_cast<uint32_t>((it & 1) * kPeakN);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                umma_i8_pair(d_tmem, a_desc + static_cast<uint64_t>(ks * 2), b_desc + static_cast<uint64_t>(ks * 2), idesc,
                             (it > 1 || ks > 0) ? 1u : 0u);
            }
        }
        umma_commit_pair(map_to_cta(smem_u32(&done_bar), 0));
        if (!mbar_wait_cluster(&done_bar, 0, &abort_word)) {
            atomicCAS(error_word, 0, kErrMmaWait);
        }
    }
    tc_fence_before_sync();
    cluster_sync_all();   // the leader's MMAs read the follower's tiles: nobody leaves before they are done
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kPeakTmemCols);
    }
}

}  // namespace

// Launch the probe on every SM.  *ops_out = integer operations (2 per multiply-add) the launch
// performs; the caller divides by the time between its events.
int launch_mma_i8_peak(int iters, int pattern, double* ops_out, const DeviceInfo& dev, cudaStream_t stream)
{
    static bool attr_done[kMaxDevices];
    if (!attr_done[dev.device]) {
        if (cudaFuncSetAttribute(mma_i8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeakSmem) != cudaSuccess) {
            (void)cudaGetLastError();
            return NNB200_INTERNAL;
        }
        attr_done[dev.device] = true;
    }
    if ((pattern & 2) != 0) {
        // CTA-pair form: one cluster of two per SM pair.
        static bool pair_attr_done[kMaxDevices];
        if (!pair_attr_done[dev.device]) {
            if (cudaFuncSetAttribute(mma_i8_peak_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeakSmem) !=
                cudaSuccess) {
                (void)cudaGetLastError();
                return NNB200_INTERNAL;
            }
            pair_attr_done[dev.device] = true;
        }
        const int ctas = dev.sm_count & ~1;
        const uint32_t idesc_pair = umma_idesc(2, 1, 1, 2 * kPeakM, kPeakN);
        mma_i8_peak_pair_kernel<<<ctas, 128, kPeakSmem, stream>>>(iters, pattern & 1, idesc_pair, dev.error_word);
        note_launch();
        if (ops_out != nullptr) {
            *ops_out = 2.0 * kPeakM * kPeakN * 32.0 * 4.0 * static_cast<double>(iters) * ctas;
        }
        return cuda_status(cudaGetLastError());
    }
    const uint32_t idesc = umma_idesc(2, 1, 1, kPeakM, kPeakN);   // s32 accumulate, s8 x s8
    mma_i8_peak_kernel<<<dev.sm_count, 128, kPeakSmem, stream>>>(iters, pattern, idesc, dev.error_word);
    note_launch();
    if (ops_out != nullptr) {
        *ops_out = 2.0 * kPeakM * kPeakN * 32.0 * 4.0 * static_cast<double>(iters) * dev.sm_count;
    }
    return cuda_status(cudaGetLastError());
}

}  // namespace nnb200
