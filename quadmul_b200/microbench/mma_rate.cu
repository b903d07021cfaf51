// Microbenchmark: clocks per tcgen05.mma.kind::i8 by shape and operand source (one CTA, one issuing thread).
// Measures a limit of the hardware that the decode kernel (csrc/qm_gemm_dec.cu) is designed around; not part of the library.
//   build: nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a --expt-relaxed-constexpr -o mma_rate.bin mma_rate.cu -lcuda
//   run:   ./mma_rate.bin
// Every in-kernel wait is bounded (qm_ptx.cuh); a time-out sets the status word that the host prints.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include "../csrc/qm_ptx.cuh"
#include "../csrc/qm_tc_common.cuh"
using namespace qm::ptx;

__device__ __forceinline__ void mma_ta(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc)
{
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}

__global__ void __launch_bounds__(128, 1) mma_rate(uint32_t idesc, int a_tmem, int nacc, int ncols, int reps, long long *out, int *status)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t tmem_slot_s;
    __shared__ int abort_s;
    __shared__ __align__(8) unsigned long long bar_s;
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t op0 = (raw + 1023u) & ~1023u;  // A tile: 128 rows x 128 B; B tile after it: 256 rows x 128 B
    const uint32_t bar = smem_u32(&bar_s);
    volatile int *abort_flag = &abort_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < (128 + 256) * 128 / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(smem_raw + (op0 - raw))[i] = 0x01010101u;
    if (threadIdx.x == 0) { mbar_init(bar, 1); abort_s = 0; fence_mbar_init(); fence_proxy_async_smem(); }
    if (warp == 0) { tmem_alloc<1>(smem_u32(&tmem_slot_s), 512); tmem_relinquish<1>(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot_s;
    if (warp == 1 && lane == 0) {
        const uint64_t dA = qm::tc::make_smem_desc(op0), dB = qm::tc::make_smem_desc(op0 + 128 * 128);
        uint32_t parity = 0;
        for (int round = 0; round < 3; ++round) {
            long long t0 = clock64();
            uint32_t dd[4];
            for (int j = 0; j < 4; ++j) dd[j] = tmem + (uint32_t)((j % nacc) * ncols);
            if (a_tmem) {
                for (int r = 0; r < reps; r += 4) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) mma_ta(dd[j], tmem + 256 + 8u * j, dB + 2u * j, idesc, 1u);
                }
            } else {
                for (int r = 0; r < reps; r += 4) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) umma_i8<1>(dd[j], dA + 2u * j, dB + 2u * j, idesc, 1u);
                }
            }
            long long t1 = clock64();
            umma_commit<1>(bar);
            if (!mbar_wait(bar, parity, abort_flag)) { *status = 1; break; }
            parity ^= 1u;
            long long t2 = clock64();
            out[2 * round] = t1 - t0;
            out[2 * round + 1] = t2 - t0;
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) { tc_fence_after_sync(); tmem_dealloc<1>(tmem, 512); }
}

int main()
{
    long long *out; cudaMalloc(&out, 64); int *status; cudaMalloc(&status, 4); cudaMemset(status, 0, 4);
    cudaFuncSetAttribute(mma_rate, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    const int reps = 512;
    printf("clks per MMA (issue loop / until commit arrives), %d MMAs, K = 32 int8\n", reps);
    for (int M : {128, 64})
        for (int N : {16, 32, 64, 128, 256})
            for (int a_tmem : {0, 1})
                for (int nacc : {1, 4}) {
                    if (nacc * N > 256) continue;
                    uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
                    mma_rate<<<1, 128, 64 * 1024>>>(idesc, a_tmem, nacc, N, reps, out, status);
                    cudaError_t e = cudaDeviceSynchronize();
                    long long h[6]; cudaMemcpy(h, out, 48, cudaMemcpyDeviceToHost);
                    int st; cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
                    printf("M=%3d N=%3d A=%s nacc=%d: issue %6.1f  total %6.1f  %s st=%d\n", M, N, a_tmem ? "tmem" : "smem", nacc,
                           (double)h[4] / reps, (double)h[5] / reps, e == cudaSuccess ? "" : cudaGetErrorString(e), st);
                    if (e != cudaSuccess || st) return 1;
                }
    return 0;
}
