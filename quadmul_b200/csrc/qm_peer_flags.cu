// Completion flags between GPUs for the fused gather of the column-sharded GEMM.
//
// Every rank's GEMM epilogue stores its column slab straight into the destination rank's C (peer-mapped memory, plain
// stores).  The destination has to learn when each slab is complete.  Rank r, in stream order after its GEMM, runs
// flag_signal_kernel: a system-scope fence, then a release store of the step number into word r of a flag array that
// lives in the DESTINATION's memory.  The destination runs flags_wait_kernel: one thread per rank polls its word with
// acquire loads until it has reached the step number -- for a bounded time; when the limit expires the kernel records
// QM_ERR_TIMEOUT (wait site kWaitPeer) in the device status word and returns, so a rank that never signals costs the
// limit, not the GPU.  The two kernels run on different GPUs; nothing here makes one launch wait for another launch on
// the same GPU.  The reference has no multi-GPU path (kernel.cu:268-289 is one launch on one device).
#include "qm_internal.h"
#include "qm_ptx.cuh"
#include "qm_tc_common.cuh"

namespace qm {

namespace {

__global__ void flag_signal_kernel(int *flag, int value)
{
    if (threadIdx.x == 0) {
        __threadfence_system();  // the slab this rank's GEMM wrote is visible system-wide before the flag is
        asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
    }
}

__global__ void flags_wait_kernel(const int *flags, int count, int value, unsigned long long limit_ns, int *status)
{
    const int t = threadIdx.x;
    if (t >= count) return;
    const uint64_t t0 = ptx::globaltimer_ns();
    for (;;) {
        int v;
        asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(flags + t) : "memory");
        if (v - value >= 0) return;  // step numbers only grow; the difference survives wrap-around
        if (ptx::globaltimer_ns() - t0 > limit_ns) {
            if (atomicCAS(status, 0, (int)QM_ERR_TIMEOUT) == 0) status[1] = kWaitPeer | (t << 8);
            return;
        }
        __nanosleep(200);
    }
}

}  // namespace

int flag_signal_launch(int *flag, int value, cudaStream_t s)
{
    flag_signal_kernel<<<1, 32, 0, s>>>(flag, value);
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? QM_OK : record_cuda_error(e, "flag_signal_kernel launch");
}

int flags_wait_launch(const int *flags, int count, int value, int timeout_ms, int *status, cudaStream_t s)
{
    flags_wait_kernel<<<1, 64, 0, s>>>(flags, count, value, (unsigned long long)timeout_ms * 1000000ull, status);
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? QM_OK : record_cuda_error(e, "flags_wait_kernel launch");
}

}  // namespace qm
