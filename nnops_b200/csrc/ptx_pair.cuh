// Inline-PTX wrappers for CTA pairs (thread-block clusters of two) driving one tcgen05.mma over
// both SMs (cta_group::2): cluster rank / address mapping, cluster barriers, remote mbarrier
// arrives, TMA loads that report to the pair leader's barrier, and the paired TMEM / MMA /
// commit forms.  Loads stay plain point-to-point copies from this GPU's own memory into the
// issuing CTA's shared memory; only the completion signal goes to the other CTA.
#pragma once

#include "ptx.cuh"

namespace nnb200 {

__device__ __forceinline__ uint32_t cluster_cta_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Address of the same shared-memory location in CTA `rank` of this cluster (shared::cluster window).
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}

// Whole-CTA, both CTAs of the cluster: every thread arrives, then waits.
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Arrive on an mbarrier that may live in the other CTA (address from map_to_cta).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// try_wait with cluster-scope acquire: the arrivals may come from the other CTA.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// The same with a suspend-time hint (see mbar_try_wait_suspend).
__device__ __forceinline__ bool mbar_try_wait_cluster_suspend(uint64_t* bar, uint32_t parity, uint32_t ns)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}

// Bounded wait, as mbar_wait, with the cluster-scope probe.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag)
{
    if (mbar_try_wait_cluster(bar, parity)) {
        return true;
    }
    const long long t0 = clock64();
    uint32_t spins = 0;
    for (;;) {
        if (mbar_try_wait_cluster_suspend(bar, parity, kWaitSuspendNs)) {
            return true;
        }
        if ((++spins & 0xFu) == 0) {
            if (*abort_flag != 0) {
                return false;
            }
            if (clock64() - t0 > kWaitLimitCycles) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// 2-D tiled load into THIS CTA's shared memory whose byte count is reported to the mbarrier at
// `bar_cluster_addr` (the pair leader's full barrier, from map_to_cta).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int32_t x, int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}

// The same for a 4-D tensor map (an NHWC activation: {c, w, h, n}); coordinates may lie outside
// the tensor, where the load delivers the fill value.
__device__ __forceinline__ void tma_load_4d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int32_t x, int32_t y, int32_t z, int32_t w)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}

// TMEM allocation for the pair: one warp of EACH of the two CTAs executes these.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// One thread of the pair's leader CTA: D (256 rows over both SMs' TMEM) (+)= A * B, with A's
// two 128-row halves and B's two N/2-row halves read from the two CTAs' shared memory at the
// same offsets.
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrive on the mbarrier at `bar_cluster_addr` (either CTA's) once every paired MMA this thread
// issued so far has completed in both SMs.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}

// The same arrival delivered to the barrier at this shared-memory offset in EVERY CTA named by
// cta_mask (bit i = cluster rank i), with one instruction instead of one commit per destination.
__device__ __forceinline__ void umma_commit_pair_mask(uint64_t* bar, uint16_t cta_mask)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     smem_u32(bar)),
                 "h"(cta_mask)
                 : "memory");
}

}  // namespace nnb200
