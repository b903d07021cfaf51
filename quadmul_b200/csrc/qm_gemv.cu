// Packed-int4 GEMM for one to four rows of A (batch-1 decode): a weight-streaming dp4a kernel, no tensor cores.
//
// Same contract as the other GEMM kernels (exact int32 C = A * B^T on nibbles; replaces the reference's igemm<Config>,
// kernel.cu:62-266, whose table has no entry below M = 128).  With so few rows of A the tensor path has nothing to gain
// from the MMA and pays for its pipeline: a tcgen05.mma costs the same ~46 clocks for N = 16 tokens as for 64, and a
// launch is a chain of TMA -> converter -> TMEM -> MMA -> reduction hand-offs (8.0 us at 1 x 4096 x 4096, the same
// whether the weights come from HBM or from L2).  Here every warp streams whole rows of B with coalesced 16-byte loads
// (a warp reads 512 contiguous bytes per instruction, several rows in flight), splits each 16-byte chunk into the
// even and the odd elements times 16 as everywhere else in this library, and multiplies with dp4a against the rows of A,
// which are converted once per CTA into shared memory in the same order.  Per chunk and lane: 12 integer
// instructions for the split and 8 dp4a per row of A, i.e. up to ~45 packed bytes per clock and SM at one row, well
// above the ~44 bytes per clock and SM that HBM can deliver to 148 SMs.  A warp-shuffle reduction over the 32 K-slices
// and one store per output finish a row of B.
//
// The accumulators hold 256 x the true sums (K < 131072 keeps them inside int32, as on the tensor path).  Launches
// chain through programmatic dependent launch like the decode kernel's: before the grid dependency is resolved a warp
// only issues L2 prefetches for its first rows of B (a prefetch returns no data).
#include <atomic>
#include <cstdlib>

#include "qm_epilogue.cuh"
#include "qm_internal.h"
#include "qm_ptx.cuh"
#include "qm_tc_common.cuh"

namespace qm {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
// RU = rows of B a warp streams at a time.  Every chunk of a row of A is read from shared memory once per step, so the
// shared-memory traffic is 2 MR / RU times the weight bytes.  RU = 2 gives twice the warps for a given n (best for the
// small, latency-bound problems: 2 x 4096 x 4096 4.8 us against 5.8 us), RU = 4 halves the shared-memory traffic (best
// when the stream is long: 4 x 28672 x 8192 35 against 43 us); the launcher picks by n.
template <int MR, int RU>
__global__ void __launch_bounds__(kThreads)
gemv_kernel(const uint8_t *__restrict__ A, const uint8_t *__restrict__ B, int32_t *__restrict__ C, int64_t ldc, int m, int n, int k,
            uint16_t *__restrict__ out_bf16, const float *__restrict__ scale_a, const float *__restrict__ scale_b)
{
    extern __shared__ uint4 a_cv[];  // [MR][chunks][2]: even elements x 16, odd elements x 16 of each 16-byte chunk of A
    ptx::grid_launch_dependents();
    const int chunks = k / 32;  // 16-byte packed chunks per row
    const int64_t row_bytes = k / 2;
    constexpr int kRowsPerStep = RU;
    const int lane = threadIdx.x & 31;
    const int warp = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const int num_warps = gridDim.x * kWarps;
    // One row of A: every warp takes a contiguous range of rows of B, the ranges equal to within one row (1 x 8192 x 4096:
    // 4.98 -> 4.32 us against whole steps dealt out in turn, where the warps with one step more decide the time).  With more
    // rows of A the steps are dealt out in turn: there a range's last, partly empty step costs more than the balance gains
    // (4 x 11008 x 4096: 11.4 us in turn, 14.2 us with ranges).
    constexpr bool kRanges = MR == 1;
    const int row_end = kRanges ? (int)((int64_t)(warp + 1) * n / num_warps) : n;
    const int first_row0 = kRanges ? (int)((int64_t)warp * n / num_warps) : warp * kRowsPerStep;
    const int row_step = kRanges ? kRowsPerStep : num_warps * kRowsPerStep;
    // rows past the end of the range re-read the step's first row; their results are not stored
    auto row_ptr = [&](int row0, int u) { return reinterpret_cast<const uint4 *>(B + (int64_t)(row0 + u < row_end ? row0 + u : row0) * row_bytes); };
    if (first_row0 < row_end) {
        // L2 prefetch of this warp's first rows: returns no data, so it may run before the grid dependency is resolved
#pragma unroll
        for (int u = 0; u < kRowsPerStep; ++u)
            for (int64_t b = (int64_t)lane * 128; b < row_bytes; b += 32 * 128)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint8_t *>(row_ptr(first_row0, u)) + b));
    }
    ptx::grid_dependency_wait();  // nothing above read or wrote global memory

    for (int i = threadIdx.x; i < MR * chunks; i += kThreads) {
        const int r = i / chunks, c = i - r * chunks;
        uint4 w = make_uint4(0, 0, 0, 0);
        if (r < m) w = __ldg(reinterpret_cast<const uint4 *>(A + r * row_bytes) + c);
        uint4 lo, hi;
        tc::split_s4x32(w, lo, hi);
        a_cv[2 * i] = lo;
        a_cv[2 * i + 1] = hi;
    }
    __syncthreads();

    for (int row0 = first_row0; row0 < row_end; row0 += row_step) {
        int acc[kRowsPerStep][MR];
#pragma unroll
        for (int u = 0; u < kRowsPerStep; ++u)
#pragma unroll
            for (int r = 0; r < MR; ++r) acc[u][r] = 0;
        const uint4 *brow[kRowsPerStep];
#pragma unroll
        for (int u = 0; u < kRowsPerStep; ++u) brow[u] = row_ptr(row0, u);
        // acc += (chunk c of the rows of A) x (chunk c of the step's rows of B, already in registers)
        auto accumulate = [&](int c, const uint4(&w)[kRowsPerStep]) {
            uint4 wl[kRowsPerStep], wh[kRowsPerStep];
#pragma unroll
            for (int u = 0; u < kRowsPerStep; ++u) tc::split_s4x32(w[u], wl[u], wh[u]);
#pragma unroll
            for (int r = 0; r < MR; ++r) {
                const uint4 al = a_cv[2 * (r * chunks + c)], ah = a_cv[2 * (r * chunks + c) + 1];
#pragma unroll
                for (int u = 0; u < kRowsPerStep; ++u) {
                    int s = acc[u][r];
                    s = __dp4a((int)wl[u].x, (int)al.x, s);
                    s = __dp4a((int)wl[u].y, (int)al.y, s);
                    s = __dp4a((int)wl[u].z, (int)al.z, s);
                    s = __dp4a((int)wl[u].w, (int)al.w, s);
                    s = __dp4a((int)wh[u].x, (int)ah.x, s);
                    s = __dp4a((int)wh[u].y, (int)ah.y, s);
                    s = __dp4a((int)wh[u].z, (int)ah.z, s);
                    s = __dp4a((int)wh[u].w, (int)ah.w, s);
                    acc[u][r] = s;
                }
            }
        };
#pragma unroll(8 / kRowsPerStep)
        for (int c = lane; c < chunks; c += 32) {
            uint4 w[kRowsPerStep];
#pragma unroll
            for (int u = 0; u < kRowsPerStep; ++u) w[u] = __ldcs(brow[u] + c);
            accumulate(c, w);
        }
#pragma unroll
        for (int u = 0; u < kRowsPerStep; ++u)
#pragma unroll
            for (int r = 0; r < MR; ++r) {
                int s = acc[u][r];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
                acc[u][r] = s;
            }
        // lane (u, r) writes output (row r of A, row row0 + u of B)
        if (lane < kRowsPerStep * MR) {
            const int u = lane / MR, r = lane - u * MR;
            int s = 0;
#pragma unroll
            for (int uu = 0; uu < kRowsPerStep; ++uu)
#pragma unroll
                for (int rr = 0; rr < MR; ++rr)
                    if (uu == u && rr == r) s = acc[uu][rr];
            const int p = row0 + u;
            if (p < row_end && r < m) {
                s >>= 8;
                if (out_bf16)
                    out_bf16[(int64_t)r * ldc + p] =
                        (uint16_t)dequant_bf16_bits(s, scale_a ? __ldg(scale_a + r) : 1.0f, scale_b ? __ldg(scale_b + p) : 1.0f);
                else
                    C[(int64_t)r * ldc + p] = s;
            }
        }
    }
}

template <int MR, int RU>
int launch_gemv(const GemmArgs &g, const DeviceCtx &ctx)
{
    const size_t smem = (size_t)MR * (size_t)g.k;  // MR rows x k int8
    static std::atomic<bool> configured[64];  // set once per device; a repeated cudaFuncSetAttribute is harmless
    if (!configured[ctx.device & 63].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(gemv_kernel<MR, RU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemvMaxSmemBytes);
        if (e != cudaSuccess) return record_cuda_error(e, "cudaFuncSetAttribute(gemv shared memory)");
        configured[ctx.device & 63].store(true, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    // enough warps that every SM has ~16 rows of B in flight; never more warps than row pairs
    constexpr int kRowsPerStep = RU;
    const int64_t steps = ((int64_t)g.n + kRowsPerStep - 1) / kRowsPerStep;
    int64_t ctas = (steps + kWarps - 1) / kWarps;
    const int64_t max_ctas = (int64_t)(ctx.num_sms > 0 ? ctx.num_sms : 1) * (smem > 100 * 1024 ? 1 : (smem > 48 * 1024 ? 2 : 4));
    if (ctas > max_ctas) ctas = max_ctas;
    if (ctas < 1) ctas = 1;
    cfg.gridDim = dim3((unsigned)ctas, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = g.stream;
    cudaLaunchAttribute attr[1];
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    static const bool allow_pdl = !std::getenv("QM_NO_PDL");
    if (allow_pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 1;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_kernel<MR, RU>, g.A, g.B, g.C, g.ldc, g.m, g.n, g.k, static_cast<uint16_t *>(g.out_bf16),
                                       g.scale_a, g.scale_b);
    if (e != cudaSuccess) return record_cuda_error(e, "gemv_kernel launch");
    return QM_OK;
}

}  // namespace

bool gemv_eligible(const GemmArgs &g)
{
    return g.m >= 1 && g.m <= kGemvMaxRows && g.k % 32 == 0 && g.k < 131072 && (size_t)(g.m <= 1 ? 1 : (g.m <= 2 ? 2 : 4)) * g.k <= kGemvMaxSmemBytes &&
           (reinterpret_cast<uintptr_t>(g.A) & 15u) == 0 && (reinterpret_cast<uintptr_t>(g.B) & 15u) == 0;
}

int gemv_launch(const GemmArgs &g, const DeviceCtx &ctx)
{
    if (!gemv_eligible(g)) return QM_ERR_ARG;
    const bool long_stream = g.n >= 16384;
    if (g.m <= 1) return launch_gemv<1, 2>(g, ctx);
    if (g.m <= 2) return long_stream ? launch_gemv<2, 4>(g, ctx) : launch_gemv<2, 2>(g, ctx);
    return long_stream ? launch_gemv<4, 4>(g, ctx) : launch_gemv<4, 2>(g, ctx);
}

}  // namespace qm
