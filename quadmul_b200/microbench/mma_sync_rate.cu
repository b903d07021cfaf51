// Microbenchmark: throughput of the warp-level mma.sync.m16n8k32 s8 x s8 -> s32 (the pre-tcgen05 tensor path) on one SM.
// Measures a limit of the hardware that decides whether a register-resident decode kernel could use it; not part of the library.
//   build: nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -o mma_sync_rate.bin mma_sync_rate.cu
//   run:   ./mma_sync_rate.bin
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>

__global__ void __launch_bounds__(1024, 1) mma_sync_rate(int reps, int *sink, long long *clocks)
{
    int d[4][4];
    for (int i = 0; i < 4; ++i)
        for (int j = 0; j < 4; ++j) d[i][j] = 0;
    uint32_t a0 = threadIdx.x, a1 = threadIdx.x * 3, a2 = threadIdx.x * 5, a3 = threadIdx.x * 7, b0 = threadIdx.x * 11, b1 = threadIdx.x * 13;
    __syncthreads();
    const long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+r"(d[i][0]), "+r"(d[i][1]), "+r"(d[i][2]), "+r"(d[i][3])
                         : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
    const long long t1 = clock64();
    __syncthreads();
    int s = 0;
    for (int i = 0; i < 4; ++i)
        for (int j = 0; j < 4; ++j) s += d[i][j];
    if (s == 0x7fffffff) *sink = s;
    if (threadIdx.x == 0) clocks[0] = t1 - t0;
}

int main()
{
    int *sink; long long *clk; cudaMalloc(&sink, 4); cudaMalloc(&clk, 8);
    const int reps = 2000;
    for (int warps : {1, 2, 4, 8, 16, 32}) {
        mma_sync_rate<<<1, warps * 32>>>(reps, sink, clk);
        mma_sync_rate<<<1, warps * 32>>>(reps, sink, clk);
        cudaError_t e = cudaDeviceSynchronize();
        long long h; cudaMemcpy(&h, clk, 8, cudaMemcpyDeviceToHost);
        const double mmas = (double)warps * reps * 4;
        printf("%2d warps: %8lld clocks for %.0f mma.sync m16n8k32 s8: %.2f clocks per warp-MMA, %.0f MAC/clk/SM %s\n", warps, h, mmas,
               h / (double)(reps * 4), mmas * 16 * 8 * 32 / h, e == cudaSuccess ? "" : cudaGetErrorString(e));
    }
    return 0;
}
