// Microbenchmark: how fast can TMA stream a row-major byte matrix into shared memory, by box shape.
// Measures a limit of the hardware that the decode kernel (csrc/qm_gemm_dec.cu) is designed around; not part of the library.
//   build: nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a --expt-relaxed-constexpr -o tma_stream.bin tma_stream.cu -lcuda
//   run:   ./tma_stream.bin   [bytes per matrix row, default 4096]
// Every in-kernel wait is bounded (qm_ptx.cuh); a time-out sets the status word that the host prints.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include "../csrc/qm_ptx.cuh"
using namespace qm::ptx;

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

__global__ void __launch_bounds__(64, 1)
stream_kernel(const __grid_constant__ CUtensorMap tmap, int tiles, int stages_per_tile, int box_rows, int box_w, int nbox,
              int S, int stage_bytes, int consume, int *status, unsigned *sink)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t d0 = (raw + 1023u) & ~1023u;
    const uint32_t bar0 = d0 + S * stage_bytes;
    __shared__ int abort_flag_s;
    volatile int *abort_flag = &abort_flag_s;
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (S + s); };
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
        abort_flag_s = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
                for (int kb = 0; kb < stages_per_tile; ++kb, ++it) {
                    const int s = it % S; const uint32_t ph = (it / S) & 1u;
                    if (!mbar_wait(empty(s), ph ^ 1u, abort_flag)) { atomicExch(status, 1); *abort_flag = 1; return; }
                    mbar_arrive_expect_tx(full(s), stage_bytes);
                    for (int b = 0; b < nbox; ++b)
                        tma_load_2d(d0 + s * stage_bytes + b * box_rows * box_w, &tmap, (kb * nbox + b) * box_w, t * box_rows, full(s));
                }
            }
        }
    } else {
        uint32_t it = 0; unsigned acc = 0;
        for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
            for (int kb = 0; kb < stages_per_tile; ++kb, ++it) {
                const int s = it % S; const uint32_t ph = (it / S) & 1u;
                if (!warp_wait<false>(full(s), ph, abort_flag, lane)) { if (lane == 0) { atomicExch(status, 2); *abort_flag = 1; } return; }
                if (consume) {
                    for (int o = lane * 16; o < stage_bytes; o += 512) { uint4 w = lds128(d0 + s * stage_bytes + o); acc += w.x ^ w.y ^ w.z ^ w.w; }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty(s));
            }
        }
        if (acc == 0x12345678u) *sink = acc;
    }
}

int main(int argc, char **argv)
{
    const long rows = 114688, kbytes = argc > 1 ? atol(argv[1]) : 4096;  // 470 MB at 4096
    const long total = rows * kbytes;
    uint8_t *d; cudaMalloc(&d, total); cudaMemset(d, 1, total);
    int *status; cudaMalloc(&status, 4); cudaMemset(status, 0, 4);
    unsigned *sink; cudaMalloc(&sink, 4);
    void *p = nullptr; cudaDriverEntryPointQueryResult q;
    cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    EncodeTiledFn enc = (EncodeTiledFn)p;
    cudaFuncSetAttribute(stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    struct Cfg { const char *name; int box_rows, box_w, nbox, ring_kb, ctas_per_sm, consume, flat; };
    Cfg cfgs[] = {
        {"128r x 64B x2 (current), ring 160K", 128, 64, 2, 160, 1, 0, 0},
        {"128r x 64B x2, consume", 128, 64, 2, 160, 1, 1, 0},
        {"128r x 128B x1, ring 160K", 128, 128, 1, 160, 1, 0, 0},
        {"128r x 256B x1, ring 160K", 128, 256, 1, 160, 1, 0, 0},
        {"128r x 64B x4, ring 160K", 128, 64, 4, 160, 1, 0, 0},
        {"64r x 256B x1, ring 160K", 64, 256, 1, 160, 1, 0, 0},
        {"32r x 256B x2, ring 160K", 32, 256, 2, 160, 1, 0, 0},
        {"128r x 64B x2, ring 80K, 2 CTA/SM", 128, 64, 2, 80, 2, 0, 0},
        {"128r x 64B x2, ring 64K", 128, 64, 2, 64, 1, 0, 0},
        {"128r x 64B x2, ring 96K", 128, 64, 2, 96, 1, 0, 0},
        {"flat 64r x 256B (contiguous 16K), ring 160K", 64, 256, 1, 160, 1, 0, 1},
        {"flat 64r x 256B, ring 80K, 2 CTA/SM", 64, 256, 1, 80, 2, 0, 1},
    };
    for (const Cfg &c : cfgs) {
        CUtensorMap tm;
        cuuint64_t dims[2], strides[1]; cuuint32_t box[2] = {(cuuint32_t)c.box_w, (cuuint32_t)c.box_rows}, estr[2] = {1, 1};
        long vrows, vk;
        if (c.flat) { vk = 256; vrows = total / 256; } else { vk = kbytes; vrows = rows; }
        dims[0] = vk; dims[1] = vrows; strides[0] = vk;
        CUresult r = enc(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, d, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { printf("%s: encode failed %d\n", c.name, (int)r); continue; }
        const int stage_bytes = c.box_rows * c.box_w * c.nbox;
        const int S = c.ring_kb * 1024 / stage_bytes;
        const int tiles = (int)(vrows / c.box_rows);
        const int stages_per_tile = (int)(vk / (c.box_w * c.nbox));
        const int smem = 1024 + S * stage_bytes + 2 * S * 8 + 64;
        const int grid = 148 * c.ctas_per_sm;
        cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
        for (int i = 0; i < 2; ++i)
            stream_kernel<<<grid, 64, smem>>>(tm, tiles, stages_per_tile, c.box_rows, c.box_w, c.nbox, S, stage_bytes, c.consume, status, sink);
        cudaEventRecord(e0);
        const int reps = 5;
        for (int i = 0; i < reps; ++i)
            stream_kernel<<<grid, 64, smem>>>(tm, tiles, stages_per_tile, c.box_rows, c.box_w, c.nbox, S, stage_bytes, c.consume, status, sink);
        cudaEventRecord(e1);
        cudaError_t e = cudaDeviceSynchronize();
        float ms; cudaEventElapsedTime(&ms, e0, e1);
        int st = 0; cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
        printf("%-48s S=%2d stage=%5d  %8.1f us  %7.1f GB/s  status=%d %s\n", c.name, S, stage_bytes, ms * 1e3 / reps,
               total / (ms / reps) / 1e6, st, e == cudaSuccess ? "" : cudaGetErrorString(e));
        if (e != cudaSuccess || st) break;
    }
    return 0;
}
