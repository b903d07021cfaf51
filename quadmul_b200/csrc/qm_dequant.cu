// Dequantisation of an int32 product that already sits in memory: out[r][c] = bf16(float(acc[r][c]) * scale_a[r] * scale_b[c]).
//
// The composed half of qm_gemm_s4_dequant_bf16 for shapes whose GEMM kernel has no fused epilogue (the 256 x 256
// large-shape kernel converts inside its epilogue and never writes the int32 matrix).  The reference has no scales and
// no floating-point output (pure integer GEMM, kernel.cu:155-184); its README names fusing as the intended use
// (README.md:7).  HBM-bound: 4 bytes read and 2 written per element; 8 elements per thread, 16-byte accesses where the
// pointers and pitches allow.
#include <cuda_bf16.h>

#include "qm_epilogue.cuh"
#include "qm_internal.h"

namespace qm {

namespace {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
dequant_kernel(const int32_t *__restrict__ acc, int64_t ld_acc, const float *__restrict__ scale_a, const float *__restrict__ scale_b,
               uint16_t *__restrict__ out, int64_t ldc, int m, int n, int vec_ok)
{
    const int64_t groups_per_row = (n + 7) / 8;
    const int64_t total = (int64_t)m * groups_per_row;
    for (int64_t g = (int64_t)blockIdx.x * kThreads + threadIdx.x; g < total; g += (int64_t)gridDim.x * kThreads) {
        const int r = (int)(g / groups_per_row);
        const int c0 = (int)(g % groups_per_row) * 8;
        const float sa = scale_a ? __ldg(scale_a + r) : 1.0f;
        const int32_t *src = acc + (int64_t)r * ld_acc + c0;
        uint16_t *dst = out + (int64_t)r * ldc + c0;
        if (vec_ok && c0 + 8 <= n) {
            const int4 x0 = __ldcs(reinterpret_cast<const int4 *>(src));
            const int4 x1 = __ldcs(reinterpret_cast<const int4 *>(src) + 1);
            float sb[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) sb[j] = scale_b ? __ldg(scale_b + c0 + j) : 1.0f;
            uint4 o;
            o.x = dequant_bf16_bits(x0.x, sa, sb[0]) | (dequant_bf16_bits(x0.y, sa, sb[1]) << 16);
            o.y = dequant_bf16_bits(x0.z, sa, sb[2]) | (dequant_bf16_bits(x0.w, sa, sb[3]) << 16);
            o.z = dequant_bf16_bits(x1.x, sa, sb[4]) | (dequant_bf16_bits(x1.y, sa, sb[5]) << 16);
            o.w = dequant_bf16_bits(x1.z, sa, sb[6]) | (dequant_bf16_bits(x1.w, sa, sb[7]) << 16);
            __stcs(reinterpret_cast<uint4 *>(dst), o);
        } else {
            for (int j = 0; j < 8 && c0 + j < n; ++j)
                dst[j] = (uint16_t)dequant_bf16_bits(src[j], sa, scale_b ? __ldg(scale_b + c0 + j) : 1.0f);
        }
    }
}

}  // namespace

int dequant_launch(const int32_t *acc, int64_t ld_acc, const float *scale_a, const float *scale_b, void *out_bf16, int64_t ldc,
                   int m, int n, cudaStream_t s)
{
    if (m <= 0 || n <= 0) return QM_OK;
    const int vec_ok = ((reinterpret_cast<uintptr_t>(acc) & 15u) == 0 && (ld_acc & 3) == 0 &&
                        (reinterpret_cast<uintptr_t>(out_bf16) & 15u) == 0 && (ldc & 7) == 0)
                           ? 1
                           : 0;
    const int64_t total = (int64_t)m * ((n + 7) / 8);
    int64_t blocks = (total + kThreads - 1) / kThreads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    dequant_kernel<<<(unsigned)blocks, kThreads, 0, s>>>(acc, ld_acc, scale_a, scale_b, static_cast<uint16_t *>(out_bf16), ldc, m, n,
                                                           vec_ok);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? QM_OK : record_cuda_error(e, "dequant_kernel launch");
}

}  // namespace qm
