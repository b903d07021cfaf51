// Thin inline-PTX wrappers for the sm_100a features the GEMM kernel uses: mbarrier,
// TMA (cp.async.bulk.tensor), tcgen05 (alloc / mma / commit / ld / fences) and proxy fences.
// Every spin is bounded: a wait that outlives QM_WAIT_LIMIT_NS returns false instead of hanging.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace qm {
namespace ptx {

#ifndef QM_WAIT_LIMIT_NS
#define QM_WAIT_LIMIT_NS 200000000ull  // 0.2 s per wait, far beyond any legitimate stall (whole kernels take < 30 ms)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint64_t globaltimer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- mbarrier ------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrive on the barrier at the same shared-memory offset in CTA `cta` of this cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t cta)
{
    asm volatile(
        "{\n"
        " .reg .b32 ra;\n"
        " mapa.shared::cluster.u32 ra, %0, %1;\n"
        " mbarrier.arrive.shared::cluster.b64 _, [ra];\n"
        "}\n" ::"r"(bar),
        "r"(cta)
        : "memory");
}

__device__ __forceinline__ uint32_t mapa_cluster(uint32_t addr, uint32_t cta)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
    return r;
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Cluster-scope acquire, needed when the arrivals come from the peer CTA.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false if the limit expired or another role raised `abort_flag`.
template <bool kCluster = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag)
{
    auto poll = [&]() { return kCluster ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity); };
    if (poll()) return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (!poll()) {
        if ((++spins & 63u) == 0u) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > QM_WAIT_LIMIT_NS) return false;
        }
    }
    return true;
}

// Non-suspending poll with cluster-scope acquire.  For barriers whose arrivals come from the peer
// CTA of a pair (remote mbarrier.arrive, tcgen05.commit issued by the other SM).
__device__ __forceinline__ bool mbar_test_wait_cluster(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool mbar_spin_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag)
{
    if (mbar_test_wait_cluster(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (!mbar_test_wait_cluster(bar, parity)) {
        if ((++spins & 255u) == 0u) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > QM_WAIT_LIMIT_NS) return false;
        }
    }
    return true;
}

// Whole-warp wait with one verdict for all lanes.  kRemote: lane 0 alone spins (without suspending, cluster-scope acquire)
// and broadcasts its verdict by shuffle; the other lanes make no acquire of their own, so this form is used only where what
// follows does not read memory that the barrier guards: tcgen05.ld of an accumulator (ordered by tcgen05.fence) or stores into
// a slot that the barrier declares free.
template <bool kRemote>
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int lane)
{
    if constexpr (!kRemote) {
        // Every lane polls, and all lanes leave the loop in the same iteration.  Why both halves are needed:
        //  * Visibility.  mbarrier.try_wait has acquire semantics for the thread that executes it and sees the phase
        //    complete: the writes the barrier guards (TMA bytes counted by complete_tx, a peer's shared-memory stores
        //    released by its arrive) are then visible to THAT thread.  A lane that only learned of the completion from a
        //    vote or a shuffle has made no acquire of its own, so each lane must see `true` from its own try_wait.  The
        //    loop ends only in an iteration in which every lane's own try_wait returned true.
        //  * Convergence.  The instructions that follow such a wait are warp-wide .sync.aligned ones (tcgen05.ld,
        //    tcgen05.st, tcgen05.wait), which require all 32 threads to execute the same instruction together; executed by
        //    a diverged warp their behaviour is undefined.  One try_wait can answer differently for different lanes when
        //    the phase completes while it is in flight, so a per-lane `while (!try_wait)` lets lanes leave in different
        //    iterations, and nothing obliges the compiler to reconverge them before an inline-asm instruction it knows
        //    nothing about.  __all_sync is a convergence point by definition: every lane that leaves the loop leaves it
        //    from the same vote, so the warp is converged at the next instruction.  (With a per-lane loop about one
        //    8192^3 launch in 120 had a few stale TMEM lanes, always the lowest lanes of one warp; with this form none.)
        //  * Ordering against the tensor core's asynchronous accesses is not this function's job: every call site that
        //    goes on to tcgen05.ld / tcgen05.st / tcgen05.mma issues tcgen05.fence::after_thread_sync after the wait, and
        //    tcgen05.fence::before_thread_sync before the arrive that hands the data on.
        if (__all_sync(0xFFFFFFFFu, mbar_try_wait(bar, parity))) return true;
        const uint64_t t0 = globaltimer_ns();
        uint32_t spins = 0;
        for (;;) {
            if (__all_sync(0xFFFFFFFFu, mbar_try_wait(bar, parity))) return true;
            if ((++spins & 63u) == 0u) {
                const bool stop = (*abort_flag != 0) || (globaltimer_ns() - t0 > QM_WAIT_LIMIT_NS);
                if (__any_sync(0xFFFFFFFFu, stop)) return false;
            }
        }
    } else {
        int ok = 1;
        if (lane == 0) ok = mbar_spin_wait(bar, parity, abort_flag) ? 1 : 0;
        return __shfl_sync(0xFFFFFFFFu, ok, 0) != 0;
    }
}

// ---- proxy / tcgen05 fences ------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- TMA -------------------------------------------------------------------------------
// 2-D tiled load global -> shared of this CTA, completion counted in bytes on `bar`.
// x is the innermost coordinate in elements (bytes here) and must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const void *tmap, int32_t x, int32_t y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void prefetch_tmap(const void *tmap)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// ---- TMEM ------------------------------------------------------------------------------
template <int kGroup>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols)
{
    if constexpr (kGroup == 1)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
                     : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
                     : "memory");
}

template <int kGroup>
__device__ __forceinline__ void tmem_relinquish()
{
    if constexpr (kGroup == 1)
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    else
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

template <int kGroup>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    if constexpr (kGroup == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---- tcgen05.mma / commit ----------------------------------------------------------------
// D[tmem] (+)= A[smem desc] * B[smem desc], int8 x int8 -> int32.  Issued by ONE thread.
template <int kGroup>
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    if constexpr (kGroup == 1)
        asm volatile(
            "{\n"
            " .reg .pred p;\n"
            " setp.ne.b32 p, %4, 0;\n"
            " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n"
            " .reg .pred p;\n"
            " setp.ne.b32 p, %4, 0;\n"
            " tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
}

// Makes `bar` (a shared::cluster address; a local shared::cta address is valid as such)
// complete one arrival once every tcgen05.mma this thread issued before has finished.
template <int kGroup>
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    if constexpr (kGroup == 1)
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    else
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- tcgen05.ld ------------------------------------------------------------------------
// Lane i of the warp reads TMEM lane (taddr.lane + i), 16 or 32 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&v)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- shared-memory vector access by 32-bit address ---------------------------------------
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ void sts128(uint32_t addr, uint4 v)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- programmatic dependent launch ----------------------------------------------------------
// launch_dependents: the next kernel in the stream (if it was launched with programmatic stream serialisation)
// may start once every CTA of this grid has executed this or exited.  wait: blocks until the grids this one
// depends on have completed and their memory is visible; returns at once when there is no such dependency.
__device__ __forceinline__ void grid_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void grid_dependency_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_arrive()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}

__device__ __forceinline__ void cluster_wait()
{
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

}  // namespace ptx
}  // namespace qm
