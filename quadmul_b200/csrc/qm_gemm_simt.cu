// General-shape int4 GEMM on the integer dot-product units (dp4a).
//
// Takes what the tensor-core kernel cannot address: K not a multiple of 32, operands that are not
// 16-byte aligned, K >= 131072.  Same arithmetic contract as the reference's kernel
// (kernel.cu:62-266): C[m,n] = sum_k s4(A[m,k]) * s4(B[n,k]), exact int32.
//
// Operand bytes are staged through shared memory with byte loads (so any alignment works), each
// 32-bit word of 8 nibbles is split into the even and the odd elements scaled by 16
// (w << 4 & 0xF0F0F0F0, w & 0xF0F0F0F0 read as four int8 each), and dp4a accumulates 256 x the
// true sum; the factor is removed with an exact arithmetic shift every kFlushChunks chunks.
#include "qm_internal.h"

namespace qm {

namespace {

constexpr int kTile = 64;         // C tile is kTile x kTile per CTA
constexpr int kThreads = 256;     // 16 x 16 threads, 4 x 4 outputs each
constexpr int kChunkBytes = 32;   // packed bytes of K per stage (64 elements)
constexpr int kPitchWords = kChunkBytes / 4 + 1;
constexpr int kFlushChunks = 256; // 256 chunks * 64 elements * 64 (max |a*b|) * 256 = 2^28 < 2^31

__global__ void __launch_bounds__(kThreads) gemm_simt_kernel(const uint8_t *__restrict__ A, const uint8_t *__restrict__ B,
                                                             int32_t *__restrict__ C, int M, int N, int K, int64_t ldc)
{
    __shared__ uint32_t sA[kTile * kPitchWords];
    __shared__ uint32_t sB[kTile * kPitchWords];
    const int64_t kb = K / 2;  // packed bytes per row
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int row0 = blockIdx.y * kTile, col0 = blockIdx.x * kTile;

    int32_t total[4][4], acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) total[i][j] = acc[i][j] = 0;

    int chunks_since_flush = 0;
    for (int64_t b0 = 0; b0 < kb; b0 += kChunkBytes) {
        // stage: 64 rows x 32 bytes per operand = 2048 bytes; 8 bytes (2 words) per thread
        {
            uint8_t *dA = reinterpret_cast<uint8_t *>(sA), *dB = reinterpret_cast<uint8_t *>(sB);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                int idx = threadIdx.x * 8 + i;  // 0..2047
                int r = idx / kChunkBytes, c = idx % kChunkBytes;
                int64_t gb = b0 + c;
                uint8_t va = 0, vb = 0;
                if (gb < kb) {
                    if (row0 + r < M) va = A[(int64_t)(row0 + r) * kb + gb];
                    if (col0 + r < N) vb = B[(int64_t)(col0 + r) * kb + gb];
                }
                dA[r * kPitchWords * 4 + c] = va;
                dB[r * kPitchWords * 4 + c] = vb;
            }
        }
        __syncthreads();
#pragma unroll
        for (int w = 0; w < kChunkBytes / 4; ++w) {
            uint32_t alo[4], ahi[4], blo[4], bhi[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t a = sA[(ty * 4 + i) * kPitchWords + w];
                uint32_t b = sB[(tx * 4 + i) * kPitchWords + w];
                alo[i] = (a << 4) & 0xF0F0F0F0u;
                ahi[i] = a & 0xF0F0F0F0u;
                blo[i] = (b << 4) & 0xF0F0F0F0u;
                bhi[i] = b & 0xF0F0F0F0u;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = __dp4a((int)alo[i], (int)blo[j], acc[i][j]);
                    acc[i][j] = __dp4a((int)ahi[i], (int)bhi[j], acc[i][j]);
                }
        }
        __syncthreads();
        if (++chunks_since_flush == kFlushChunks) {
            chunks_since_flush = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    total[i][j] += acc[i][j] >> 8;  // exact: acc is a multiple of 256
                    acc[i][j] = 0;
                }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int r = row0 + ty * 4 + i;
        if (r >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int c = col0 + tx * 4 + j;
            if (c < N) C[(int64_t)r * ldc + c] = total[i][j] + (acc[i][j] >> 8);
        }
    }
}

}  // namespace

int simt_launch(const GemmArgs &g)
{
    dim3 grid((g.n + kTile - 1) / kTile, (g.m + kTile - 1) / kTile);
    if (grid.y > 65535u) return QM_ERR_SHAPE;
    gemm_simt_kernel<<<grid, kThreads, 0, g.stream>>>(g.A, g.B, g.C, g.m, g.n, g.k, g.ldc);
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? QM_OK : record_cuda_error(e, "gemm_simt_kernel launch");
}

}  // namespace qm
