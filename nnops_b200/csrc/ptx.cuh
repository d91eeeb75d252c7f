// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarrier, TMA
// (cp.async.bulk.tensor), tcgen05 MMA / TMEM.  No multicast variants exist here on purpose:
// every CTA loads its own tiles from local memory.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace nnb200 {

// Error codes kernels record in the device error word.
enum DeviceError : int32_t {
    kErrNone = 0,
    kErrProducerWait = 1,  // TMA producer timed out on an empty-slot barrier
    kErrMmaWait = 2,       // MMA issuer timed out on a full-slot barrier
    kErrEpilogueWait = 3,  // epilogue timed out on an accumulator barrier
    kErrAccumWait = 4,     // MMA issuer timed out waiting for a free accumulator
    kErrDequantWait = 5,   // Q4_1 dequant warps timed out
    kErrDrainWait = 6,     // teardown timed out waiting for copies in flight
    kErrSelfTest = 7,      // the wait self-test's barrier ran out, as it must
    kErrPeerWait = 8,      // the device-side rank barrier timed out waiting for another GPU's flag
};

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one()
{
    uint32_t pred = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier ---------------------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// The same probe, allowed to suspend the thread in hardware for up to `ns` nanoseconds while the
// phase is incomplete (it still returns as soon as the phase completes).  Used inside the wait
// loops: a role that polls without the hint takes issue slots from the epilogue warps that share
// its scheduler.
__device__ __forceinline__ bool mbar_try_wait_suspend(uint64_t* bar, uint32_t parity, uint32_t ns)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}

// Upper bound on any single pipeline wait, in SM clock cycles (~2 s at 2 GHz).  A healthy
// kernel waits microseconds; the bound only exists so a mis-programmed pipeline returns an
// error instead of hanging the GPU.
constexpr long long kWaitLimitCycles = 4'000'000'000LL;
// How long one probe inside a wait loop may keep the thread suspended.
constexpr uint32_t kWaitSuspendNs = 20000;

// Wait for `parity` on `bar`.  Returns false if the wait ran out or another role already
// aborted (`*abort_flag` != 0); on running out it raises the flag itself.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          long long limit_cycles = kWaitLimitCycles)
{
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    const long long t0 = clock64();
    uint32_t spins = 0;
    for (;;) {
        if (mbar_try_wait_suspend(bar, parity, kWaitSuspendNs)) {
            return true;
        }
        if ((++spins & 0xFu) == 0) {
            if (*abort_flag != 0) {
                return false;
            }
            if (clock64() - t0 > limit_cycles) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// Warp-collective wait: lane 0 polls, the result is broadcast.  Keeps the number of threads
// hammering one barrier word at one per warp instead of thirty-two.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag)
{
    int ok = 1;
    if ((threadIdx.x & 31) == 0) {
        ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
    }
    ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
    return ok != 0;
}

// ---- TMA --------------------------------------------------------------------------------

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// 2-D tiled load into this CTA's shared memory; x is the innermost (contiguous) coordinate
// and must make x * elem_size a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int32_t x,
                                            int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// 4-D tiled load (an NHWC activation as {c, w, h, n}): x, the innermost coordinate, must make
// x * elem_size a multiple of 16 bytes; the others may be negative or past the end, and the
// part of the box outside the tensor is filled with zeros.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int32_t x, int32_t y,
                                            int32_t z, int32_t w)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}

// 2-D tiled store shared -> global (the destination may be a peer GPU's memory: stores, unlike
// multicast loads, are fine there).  Tracked by the issuing thread's bulk async-groups.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int32_t x, int32_t y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                 "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// At most N of this thread's bulk groups still have shared-memory reads outstanding.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// At most N of this thread's bulk groups are still incomplete (writes included).
template <int N>
__device__ __forceinline__ void bulk_wait_group()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// 1-D bulk copy global -> this CTA's shared memory; both addresses 16-byte aligned, size a
// multiple of 16 bytes; completion is counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// 16-byte asynchronous copy global -> shared without staging registers; bytes past
// `src_bytes` (0..16) are written as zeros.  Completion is tracked per thread in commit groups.
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src, uint32_t src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src),
                 "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit()
{
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait_group()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Generic-proxy writes to shared memory -> visible to the async proxy (UMMA / TMA reads).
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tcgen05 / TMEM -----------------------------------------------------------------------

// Whole-warp: allocate `ncols` (power of two, 32..512) TMEM columns; base address lands in *slot.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)),
                 "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

// Whole-warp (the allocating warp).
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Arrive on `bar` once every MMA this thread issued so far has finished reading shared
// memory / writing TMEM.  Implies tcgen05.fence::before_thread_sync.
__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile written by TMA with the
// 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.  The tile base must be
// 1024-byte aligned; stepping along K inside the 128-byte row adds the byte offset to the
// start address.
__device__ __forceinline__ uint64_t umma_desc_sw128_kmajor(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
    d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused for swizzled K-major)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset: 8 rows * 128 B
    d |= static_cast<uint64_t>(1) << 46;                      // descriptor version (sm_100)
    d |= static_cast<uint64_t>(2) << 61;                      // layout: 128-byte swizzle
    return d;
}

// Shared-memory matrix descriptor for an MN-major operand tile (the operand's M or N index is
// the contiguous one in memory: A stored [K][M], W stored [K][N]) written by TMA with the
// 128-byte swizzle: rows of 128 bytes along M/N, one row per k, eight k-rows per 1024-byte
// swizzle group (stride byte offset), and `block_bytes` between consecutive 128-byte column
// blocks of a tile wider than 128 (leading byte offset).  Stepping along K by 32 rows adds
// 32 * 128 bytes to the start address.
__device__ __forceinline__ uint64_t umma_desc_sw128_mnmajor(uint32_t smem_addr, uint32_t block_bytes)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
    d |= static_cast<uint64_t>((block_bytes >> 4) & 0x3FFFu) << 16;  // leading byte offset: next 128-byte block
    d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset: 8 k-rows * 128 B
    d |= static_cast<uint64_t>(1) << 46;                      // descriptor version (sm_100)
    d |= static_cast<uint64_t>(2) << 61;                      // layout: 128-byte swizzle
    return d;
}

// Instruction-descriptor bits that declare an operand MN-major instead of K-major.
constexpr uint32_t kUmmaAMajorMN = 1u << 15;
constexpr uint32_t kUmmaBMajorMN = 1u << 16;

// Instruction descriptor, dense, both operands K-major.
//   d_fmt: 0 = f16, 1 = f32, 2 = s32;  a_fmt / b_fmt: kind::i8 0 = u8, 1 = s8; kind::f16 0 = f16, 1 = bf16.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t d_fmt, uint32_t a_fmt, uint32_t b_fmt, uint32_t m,
                                                  uint32_t n)
{
    return (d_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem], issued by one thread.
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Warp-wide: 32 lanes x 32 consecutive 32-bit columns; lane i receives row (lane base + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]),
          "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),
          "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// One 256-bit store (sm_100): a full 32-byte sector per lane.  `p` must be 32-byte aligned.
__device__ __forceinline__ void st_global_32(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t e,
                                             uint32_t f, uint32_t g, uint32_t h)
{
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d),
                 "r"(e), "r"(f), "r"(g), "r"(h)
                 : "memory");
}

// 16-byte store to a MULTICAST address (a mapping of a multicast object bound to one buffer per
// GPU): the NVSwitch writes the bytes into every bound buffer.  Only valid on such addresses.
__device__ __forceinline__ void multimem_st_16(void* mc_addr, uint4 v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
}

// Named barrier over a subset of the CTA's warps.
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t nthreads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace nnb200
