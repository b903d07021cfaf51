// Packed-int4 GEMM for up to 64 rows of A (in tiles of 16) on small weight matrices: register-resident decode kernel.
//
// Same contract as the other GEMM kernels (exact int32 C = A * B^T on nibbles; replaces the reference's igemm<Config>,
// kernel.cu:62-266).  At the decode sizes named for this library (16 x 4096 x 4096, 16 x 11008 x 4096: 8-23 MB of weights,
// 1.3-3.5 us of HBM time) a launch of the TMA/TMEM kernel is a chain of hand-offs that costs the same 8-11 us whether
// the weights come from HBM or from L2.  This kernel has no pipeline to fill: a CTA owns 32 rows of B, its 16 warps split
// K between them, and every lane asks for ALL of its weights (up to eight 16-byte loads) before anything else happens, so
// the whole 64 KB block of a CTA is in flight after a few instructions and the launch is one memory round trip long.
// While the loads fly the CTA copies the rows of A, packed as they are, into shared memory.  The products run on the
// warp-level tensor path, mma.sync.m16n8k32.s8 (2048 MAC per clock and SM measured on B200, a quarter of tcgen05 but four
// times what 16 tokens at HBM rate need): A fragment = 16 tokens x 32 K read from shared memory and split there and then
// into even elements x 16 and odd elements x 16 (as everywhere in this library), B fragment = 8 rows of B x 32 K straight
// from the registers the weights were loaded into, after the same split.  (Converting A once into shared memory instead
// cost more than it saved: 16 x 4096 x 4096 4.8 us against 3.9 us.)  Rows of A beyond 16 are further tiles that take
// their turn against the same weight registers (K <= 4096).  Lane (g, q) of a warp (g = lane / 4, q = lane % 4)
// loads chunk 4 t + q of row g of each of four 8-row groups, and for mma step s = 0..3 supplies word s of the even half as
// the fragment's k = 4q..4q+3 and word s of the odd half as k = 16+4q..16+4q+3; the A fragment is built from the same
// words of the same chunks, so every product pairs equal K indices.  The 16 partial 16 x 32 tiles of a CTA meet in shared
// memory, are summed by 512 threads (one output each), shifted by 8 and stored as 128-byte row segments.
//
// With at most eight rows of A the operands of the MMA change places (TOK8 below): 16 rows of B x 8 tokens per instruction,
// half as many instructions per round.
//
// Launches chain through programmatic dependent launch; before griddepcontrol.wait a CTA only prefetches its weights into
// L2 (no data is returned, so this is correct whatever the previous kernel writes).  Prefetches are bulk prefetches, one per
// row of a block, so that they do not compete with the loads for the load path.
#include <atomic>
#include <cstdlib>

#include "qm_epilogue.cuh"
#include "qm_internal.h"
#include "qm_ptx.cuh"
#include "qm_tc_common.cuh"

namespace qm {

namespace {

// Shape of the CTA: WARPS warps, RG 8-row groups of B per block, MS chunk steps in flight per warp.  The library runs
// <16, 4, 2>: 32 rows of B per block, one CTA per SM.  A lane has eight 16-byte loads in flight, a warp covers
// WARPS x MS x 128 elements of K per round, and there is one output per thread (16 tokens x 8 RG rows of B = 32 WARPS).
// (Measured and not kept: <8, 2, 4>, half-size CTAs two per SM, meant to overlap the rounds of a B that needs several;
// 16 x 11008 x 4096 10.9 us against 10.2 us for the one-CTA form, 16 x 4096 x 4096 6.0 against 4.9 us; and issuing the next
// block's loads before the reduction of the current one instead of prefetching it to L2: 10.9 against 10.2 us.)
template <int WARPS, int RG, int MS>
struct RmmaCfg {
    static_assert(WARPS == 4 * RG, "one output per thread");
    static constexpr int kWarps = WARPS;
    static constexpr int kThreads = WARPS * 32;
    static constexpr int kRowGroups = RG;        // 8-row groups of B per block
    static constexpr int kRowsPerCta = 8 * RG;
    static constexpr int kMaxSteps = MS;         // chunk steps a warp keeps in flight at once
    static constexpr int kRedBytes = WARPS * RG * 32 * 4 * 4;  // one 16 x (8 RG) int32 partial tile per warp
    static constexpr int kCtasPerSm = WARPS == 16 ? 1 : 2;
};

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t word(const uint4 &v, int s) { return s == 0 ? v.x : (s == 1 ? v.y : (s == 2 ? v.z : v.w)); }

// MODE 1 (PRE): B is the pre-laid-out form written by prelayout_kernel below, [block of 8 RG rows][round][warp][step][row group][lane]
// in 16-byte chunks: every load instruction of a warp reads 512 consecutive bytes, a warp's round is 4 KB and a CTA's round
// 64 KB of consecutive addresses.  MODE 2 (FULL): the plain layout of a B whose rows fill whole 32-row blocks and whose K fills
// whole rounds (n % (8 RG) == 0, k % (128 WARPS MS) == 0): the same loads as MODE 0 without their bounds checks.  MODE 3 (WIDE,
// MS == 2): such a B, 32-byte aligned, read with 256-bit loads: a warp takes two ADJACENT chunk steps of a round (256 elements
// of K) and lane (g, q) loads chunks 2q and 2q + 1 of its row in one instruction, so that the four lanes of a row read one
// whole 128-byte line where MODE 0 / 2 read 64 bytes of it; the rows of A are indexed by the same chunks, so every product
// still pairs equal K indices.
//
// TOK8 (m <= 8): the operands of the MMA change places.  Two 8-row groups of B are the 16 rows of the instruction's first
// operand (rows g and g + 8 of a lane come from the registers of group 2i and 2i + 1) and tokens 0..7 its eight columns, so a
// round takes half as many mma.sync (the instruction costs the same for 8 tokens as for 16) and half as many partial sums go
// through the reduction.
template <int WARPS, int RG, int MS, int MODE, bool TOK8>
__global__ void __launch_bounds__(WARPS * 32, (WARPS == 16 ? 1 : 2))
gemm_rmma_kernel(const uint8_t *__restrict__ A, const uint8_t *__restrict__ B, int32_t *__restrict__ C, int64_t ldc, int m, int n, int k,
                 uint16_t *__restrict__ out_bf16, const float *__restrict__ scale_a, const float *__restrict__ scale_b)
{
    using Cfg = RmmaCfg<WARPS, RG, MS>;
    constexpr int kWarps = Cfg::kWarps, kThreads = Cfg::kThreads, kRowGroups = Cfg::kRowGroups, kRowsPerCta = Cfg::kRowsPerCta,
                  kMaxSteps = Cfg::kMaxSteps;
    constexpr bool PRE = MODE == 1, WIDE = MODE == 3, FULL = MODE == 2 || WIDE;
    static_assert(!WIDE || MS == 2, "two chunks per 256-bit load");
    static_assert(!TOK8 || RG % 2 == 0, "row groups are paired");
    constexpr int kAcc = TOK8 ? kRowGroups / 2 : kRowGroups;  // accumulator tiles (m16n8) per warp
    extern __shared__ uint4 smem_u4[];
    // The rows of A stay PACKED in shared memory, [16 tiles rows][chunks + 4] 16-byte units (the 64 bytes of padding put the two
    // rows a quarter-warp reads at once on different banks); the A fragments are split when they are read.
    uint4 *a_pk = smem_u4;
    const int chunks = k / 32;
    const int tiles = (m + 15) / 16;  // token tiles of 16 rows of A
    // (WIDE reads chunks 2q + u: 32 bytes between the lanes of a row, so one chunk of padding puts the rows of a quarter-warp on
    // different banks)
    const int pk_stride = chunks + (WIDE ? 1 : 4);
    // [warp][row group][j][32]: accumulator register j of lane l at position (l + 4 (2 rg + (j & 1))) % 32, which makes both the
    // writes (one register of all lanes) and the reads (one token, 32 rows of B) hit 32 different banks
    int32_t *red = reinterpret_cast<int32_t *>(smem_u4 + (size_t)16 * tiles * pk_stride);
    const int64_t row_bytes = k / 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int steps = (chunks + 3) / 4;  // chunk steps of a row: step t covers chunks 4t .. 4t+3
    const int num_blocks = (n + kRowsPerCta - 1) / kRowsPerCta;
    const int rounds_k = (steps + kWarps * kMaxSteps - 1) / (kWarps * kMaxSteps);  // rounds of K a block takes (pre-laid-out form: padded)
    // this lane's first chunk of (block rb, round r, this warp) in the pre-laid-out form; chunk (u, rg) is 32 * (u * RG + rg) further
    auto pre_base = [&](int rb, int r) {
        return reinterpret_cast<const uint4 *>(B) + (((int64_t)rb * rounds_k + r) * kWarps + warp) * (32 * kMaxSteps * kRowGroups) + lane;
    };

    // chunk of a row that this lane handles in step u of the round that starts at step t0 (t0 = warp + round * kWarps * kMaxSteps)
    auto chunk_of = [&](int t0, int u) {
        if constexpr (WIDE) return 4 * (t0 - warp) + 8 * warp + 2 * q + u;
        else return 4 * (t0 + u * kWarps) + q;
    };

    // L2 prefetch of one block of weights: returns no data, touches nothing the program can observe.  One bulk prefetch per row
    // of the block (per 4 KB of a pre-laid-out block) instead of one instruction per 128-byte line keeps the load path free
    // for the loads themselves.
    auto prefetch_block = [&](int rb) {
        if (rb >= num_blocks) return;
        if constexpr (PRE) {
            // a block is rounds_k x kWarps x (32 kMaxSteps kRowGroups 16) contiguous bytes
            const int pieces = rounds_k * kWarps * (32 * kMaxSteps * kRowGroups * 16) / 4096;
            const uint8_t *base = reinterpret_cast<const uint8_t *>(B) + (int64_t)rb * pieces * 4096;
            for (int i = threadIdx.x; i < pieces; i += kThreads)
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + (int64_t)i * 4096), "r"(4096) : "memory");
        } else {
            for (int i = threadIdx.x; i < kRowsPerCta; i += kThreads) {
                const int row = rb * kRowsPerCta + i;
                if (row < n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(B + (int64_t)row * row_bytes), "r"((int)row_bytes) : "memory");
            }
        }
    };
    ptx::grid_launch_dependents();
    prefetch_block((int)blockIdx.x);
    ptx::grid_dependency_wait();  // nothing above read or wrote global memory

    // all rows of A, packed as they are, -> shared memory (zero beyond m); all threads, followed by a barrier
    auto copy_a_packed = [&]() {
        for (int i = threadIdx.x; i < 16 * tiles * chunks; i += kThreads) {
            const int r = i / chunks, c = i - r * chunks;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < m) v = __ldg(reinterpret_cast<const uint4 *>(A + (int64_t)r * row_bytes) + c);
            a_pk[r * pk_stride + c] = v;
        }
        __syncthreads();
    };
    // all loads of up to kMaxSteps chunk steps of block rb, starting at step t0
    auto load_round = [&](uint4(&w)[kMaxSteps][kRowGroups], int rb, int t0) {
        if constexpr (PRE) {
            // padded with zeros beyond n and k: no bounds to check
            const uint4 *src = pre_base(rb, (t0 - warp) / (kWarps * kMaxSteps));
#pragma unroll
            for (int u = 0; u < kMaxSteps; ++u)
#pragma unroll
                for (int rg = 0; rg < kRowGroups; ++rg) w[u][rg] = __ldcs(src + 32 * (u * kRowGroups + rg));
        } else if constexpr (WIDE) {
#pragma unroll
            for (int rg = 0; rg < kRowGroups; ++rg) {
                const uint8_t *src = B + (int64_t)(rb * kRowsPerCta + rg * 8 + g) * row_bytes + (int64_t)chunk_of(t0, 0) * 16;
                asm volatile("ld.global.cs.v8.u32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                             : "=r"(w[0][rg].x), "=r"(w[0][rg].y), "=r"(w[0][rg].z), "=r"(w[0][rg].w), "=r"(w[1][rg].x), "=r"(w[1][rg].y),
                               "=r"(w[1][rg].z), "=r"(w[1][rg].w)
                             : "l"(src));
            }
        } else {
#pragma unroll
            for (int u = 0; u < kMaxSteps; ++u) {
                const int t = t0 + u * kWarps;
                const int c = 4 * t + q;
#pragma unroll
                for (int rg = 0; rg < kRowGroups; ++rg) {
                    const int row = rb * kRowsPerCta + rg * 8 + g;
                    if constexpr (FULL) {
                        w[u][rg] = __ldcs(reinterpret_cast<const uint4 *>(B + (int64_t)row * row_bytes) + c);
                    } else {
                        w[u][rg] = make_uint4(0, 0, 0, 0);
                        if (t < steps && c < chunks && row < n) w[u][rg] = __ldcs(reinterpret_cast<const uint4 *>(B + (int64_t)row * row_bytes) + c);
                    }
                }
            }
        }
    };
    // d += (token tile tt of the packed rows of A in shared memory, split here) x (the weights of one round)
    auto mma_round_packed = [&](int(&d)[kAcc][4], const uint4(&w)[kMaxSteps][kRowGroups], int t0, int tt) {
#pragma unroll
        for (int u = 0; u < kMaxSteps; ++u) {
            const int t = t0 + u * kWarps;
            const int c = chunk_of(t0, u);
            if (FULL || t < steps) {  // uniform over the warp (a whole round has every step)
                uint4 p0 = make_uint4(0, 0, 0, 0), p1 = p0;
                if (FULL || c < chunks) {
                    p0 = a_pk[(16 * tt + g) * pk_stride + c];
                    if constexpr (!TOK8) p1 = a_pk[(16 * tt + g + 8) * pk_stride + c];
                }
                if constexpr (TOK8) {
                    // second operand: token g, k = 4q..4q+3 from the even half and 16+4q.. from the odd half of the chunk
                    uint4 tlo, thi;
                    tc::split_s4x32(p0, tlo, thi);
#pragma unroll
                    for (int i = 0; i < kAcc; ++i) {
                        uint4 wl0, wh0, wl1, wh1;
                        tc::split_s4x32(w[u][2 * i], wl0, wh0);
                        tc::split_s4x32(w[u][2 * i + 1], wl1, wh1);
#pragma unroll
                        for (int s = 0; s < 4; ++s)
                            mma_s8(d[i], word(wl0, s), word(wl1, s), word(wh0, s), word(wh1, s), word(tlo, s), word(thi, s));
                    }
                    continue;
                }
                uint4 alo0, ahi0, alo1, ahi1;
                tc::split_s4x32(p0, alo0, ahi0);
                tc::split_s4x32(p1, alo1, ahi1);
#pragma unroll
                for (int rg = 0; rg < kRowGroups; ++rg) {
                    uint4 wl, wh;
                    tc::split_s4x32(w[u][rg], wl, wh);
#pragma unroll
                    for (int s = 0; s < 4; ++s)
                        mma_s8(d[rg], word(alo0, s), word(alo1, s), word(ahi0, s), word(ahi1, s), word(wl, s), word(wh, s));
                }
            }
        }
    };
    // partial tiles of all warps -> shared memory -> one output per thread (token tile tt, block rb); two barriers
    auto reduce_store = [&](const int(&d)[kAcc][4], int rb, int tt) {
        int sum = 0, tok, col;
        bool mine = true;
        if constexpr (TOK8) {
            // [warp][pair i][j][32]: register j of lane l at position (l + 2 i + (j >> 1)) % 32.  Lane (g, q) holds rows g (j = 0, 1)
            // and g + 8 (j = 2, 3) of the 16 rows of pair i, tokens 2q (j even) and 2q + 1 (j odd).
#pragma unroll
            for (int i = 0; i < kAcc; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) red[((warp * kAcc + i) * 4 + j) * 32 + ((lane + 2 * i + (j >> 1)) & 31)] = d[i][j];
            __syncthreads();
            // 8 tokens x kRowsPerCta rows of B: the first 8 kRowsPerCta threads take one output each
            tok = threadIdx.x / kRowsPerCta, col = threadIdx.x % kRowsPerCta;
            mine = tok < 8;
            if (mine) {
                const int rg = col >> 3, i = rg >> 1, half = rg & 1;
                const int src_lane = (col & 7) * 4 + (tok >> 1);
                const int j = 2 * half + (tok & 1);
#pragma unroll
                for (int ww = 0; ww < kWarps; ++ww) sum += red[((ww * kAcc + i) * 4 + j) * 32 + ((src_lane + 2 * i + half) & 31)];
            }
        } else {
#pragma unroll
            for (int rg = 0; rg < kRowGroups; ++rg)
#pragma unroll
                for (int j = 0; j < 4; ++j) red[((warp * kRowGroups + rg) * 4 + j) * 32 + ((lane + 4 * (2 * rg + (j & 1))) & 31)] = d[rg][j];
            __syncthreads();
            tok = threadIdx.x / kRowsPerCta, col = threadIdx.x % kRowsPerCta;  // 16 tokens x kRowsPerCta rows of B
            const int rg = col >> 3, cc = col & 7;
            // accumulator layout of m16n8: lane (g, q) holds (row g, col 2q), (g, 2q+1), (g+8, 2q), (g+8, 2q+1)
            const int src_lane = (tok & 7) * 4 + (cc >> 1);
            const int j = (cc & 1) + (tok >= 8 ? 2 : 0);
#pragma unroll
            for (int ww = 0; ww < kWarps; ++ww) sum += red[((ww * kRowGroups + rg) * 4 + j) * 32 + ((src_lane + 4 * (2 * rg + (j & 1))) & 31)];
        }
        sum >>= 8;
        const int token = 16 * tt + tok;
        const int p = rb * kRowsPerCta + col;
        if (mine && token < m && p < n) {
            if (out_bf16)
                out_bf16[(int64_t)token * ldc + p] =
                    (uint16_t)dequant_bf16_bits(sum, scale_a ? __ldg(scale_a + token) : 1.0f, scale_b ? __ldg(scale_b + p) : 1.0f);
            else
                C[(int64_t)token * ldc + p] = sum;
        }
        __syncthreads();  // `red` and the rows of A are rewritten next
    };

    const bool resident = steps <= kWarps * kMaxSteps;     // a block's weights fit one round of registers (the host requires it for tiles > 1)
    bool a_ready = false;
    for (int rb = blockIdx.x; rb < num_blocks; rb += gridDim.x) {
        int d[kAcc][4];
        uint4 w[kMaxSteps][kRowGroups];
        if (resident) {
            // the weights stay in registers while the token tiles pass through shared memory one after the other
            load_round(w, rb, warp);
            prefetch_block(rb + (int)gridDim.x);  // the next block goes to L2 meanwhile
            if (!a_ready) {
                copy_a_packed();
                a_ready = true;
            }
            for (int tt = 0; tt < tiles; ++tt) {
#pragma unroll
                for (int rg = 0; rg < kAcc; ++rg)
#pragma unroll
                    for (int j = 0; j < 4; ++j) d[rg][j] = 0;
                mma_round_packed(d, w, warp, tt);
                reduce_store(d, rb, tt);
            }
        } else {
#pragma unroll
            for (int rg = 0; rg < kAcc; ++rg)
#pragma unroll
                for (int j = 0; j < 4; ++j) d[rg][j] = 0;
            for (int t0 = warp; t0 < steps; t0 += kWarps * kMaxSteps) {
                load_round(w, rb, t0);
                if (t0 == warp) prefetch_block(rb + (int)gridDim.x);
                if (!a_ready) {  // every warp has at least one round here (steps > kWarps * kMaxSteps)
                    copy_a_packed();
                    a_ready = true;
                }
                mma_round_packed(d, w, t0, 0);
            }
            reduce_store(d, rb, 0);
        }
    }
}

}  // namespace

bool rmma_eligible(const GemmArgs &g)
{
    // more than one 16-row tile of A needs a block's weights resident in registers: at most kWarps * kMaxSteps chunk steps
    const int max_k = g.m <= 16 ? kRmmaMaxK : kRmmaMaxKTiled;
    return g.m >= 1 && g.m <= kRmmaMaxRows && g.k % 32 == 0 && g.k <= max_k && (reinterpret_cast<uintptr_t>(g.A) & 15u) == 0 &&
           (reinterpret_cast<uintptr_t>(g.B) & 15u) == 0;
}

// B (n x k/2 bytes) -> the pre-laid-out form of gemm_rmma_kernel<WARPS, RG, MS, true>; one thread per 16-byte chunk of B'.
template <int WARPS, int RG, int MS>
__global__ void __launch_bounds__(256) prelayout_kernel(const uint8_t *__restrict__ B, uint4 *__restrict__ Bp, int n, int k, int rounds_k,
                                                        int64_t total_chunks)
{
    const int chunks = k / 32;
    const int64_t row_bytes = k / 2;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_chunks; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t x = i;
        const int lane = (int)(x % 32); x /= 32;
        const int rg = (int)(x % RG); x /= RG;
        const int u = (int)(x % MS); x /= MS;
        const int w = (int)(x % WARPS); x /= WARPS;
        const int r = (int)(x % rounds_k);
        const int64_t rb = x / rounds_k;
        const int g = lane >> 2, q = lane & 3;
        const int64_t row = rb * (8 * RG) + rg * 8 + g;
        const int c = 4 * (w + (r * MS + u) * WARPS) + q;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < n && c < chunks) v = __ldg(reinterpret_cast<const uint4 *>(B + row * row_bytes) + c);
        Bp[i] = v;
    }
}

template <int WARPS, int RG, int MS, int MODE, bool TOK8>
static int rmma_launch_tok(const GemmArgs &g, const DeviceCtx &ctx)
{
    using Cfg = RmmaCfg<WARPS, RG, MS>;
    auto kernel = gemm_rmma_kernel<WARPS, RG, MS, MODE, TOK8>;
    const int tiles = (g.m + 15) / 16;
    const size_t smem = (size_t)16 * tiles * (g.k / 2 + 64) + Cfg::kRedBytes;  // packed rows of A, padded by 64 bytes
    static std::atomic<bool> configured[64];  // set once per device; a repeated cudaFuncSetAttribute is harmless
    if (!configured[ctx.device & 63].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kRmmaMaxRows * (kRmmaMaxKTiled / 2 + 64) + Cfg::kRedBytes);  // also covers 16 rows at kRmmaMaxK
        if (e != cudaSuccess) return record_cuda_error(e, "cudaFuncSetAttribute(rmma shared memory)");
        configured[ctx.device & 63].store(true, std::memory_order_release);
    }
    const int blocks = (g.n + Cfg::kRowsPerCta - 1) / Cfg::kRowsPerCta;
    const int sms = ctx.num_sms > 0 ? ctx.num_sms : 1;
    const int slots = sms * ((Cfg::kCtasPerSm == 2 && 2 * (smem + 1024) <= 227 * 1024) ? 2 : 1);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(blocks < slots ? blocks : slots), 1, 1);
    cfg.blockDim = dim3(Cfg::kThreads, 1, 1);
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
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, g.A, g.B, g.C, g.ldc, g.m, g.n, g.k, static_cast<uint16_t *>(g.out_bf16), g.scale_a,
                                       g.scale_b);
    if (e != cudaSuccess) return record_cuda_error(e, "gemm_rmma_kernel launch");
    return QM_OK;
}

// up to eight rows of A take the form with the operands of the MMA exchanged
template <int WARPS, int RG, int MS, int MODE>
static int rmma_launch_cfg(const GemmArgs &g, const DeviceCtx &ctx)
{
    static const bool allow_tok8 = !std::getenv("QM_RMMA_NO_TOK8");
    if (g.m <= 8 && allow_tok8) return rmma_launch_tok<WARPS, RG, MS, MODE, true>(g, ctx);
    return rmma_launch_tok<WARPS, RG, MS, MODE, false>(g, ctx);
}

int rmma_launch(const GemmArgs &g, const DeviceCtx &ctx)
{
    if (!rmma_eligible(g)) return QM_ERR_ARG;
    // whole blocks of rows and whole rounds of K: the variant without bounds checks
    static const int forced_mode = std::getenv("QM_RMMA_MODE") ? std::atoi(std::getenv("QM_RMMA_MODE")) : -1;
    if (g.n % 32 == 0 && g.k % 4096 == 0 && forced_mode != 0) {
        // 256-bit loads need 32-byte-aligned rows
        if ((reinterpret_cast<uintptr_t>(g.B) & 31u) == 0 && forced_mode != 2) return rmma_launch_cfg<16, 4, 2, 3>(g, ctx);
        return rmma_launch_cfg<16, 4, 2, 2>(g, ctx);
    }
    return rmma_launch_cfg<16, 4, 2, 0>(g, ctx);
}

// ---- offline weight pre-layout (optional) --------------------------------------------------------------------------
// Weights are static in inference; the reference left a hook for rearranging them once and never built it (kernel.cu:57
// `#define PRESHUFFLE false`, kernel.cu:450 `reorganize_packed_B`).  Here B' holds, for every 32-row block and every round of
// 4096 K-elements, the chunks in the order the kernel's lanes load them.
namespace {
constexpr int kPreWarps = 16, kPreRG = 4, kPreMS = 2;  // the configuration the library runs
int pre_rounds(int k) { return ((k / 32 + 3) / 4 + kPreWarps * kPreMS - 1) / (kPreWarps * kPreMS); }
}  // namespace

size_t prelayout_bytes(int n, int k)
{
    const size_t blocks = ((size_t)n + 8 * kPreRG - 1) / (8 * kPreRG);
    return blocks * (size_t)pre_rounds(k) * kPreWarps * 32 * kPreMS * kPreRG * 16;
}

int prelayout_launch(const uint8_t *B, uint8_t *Bp, int n, int k, cudaStream_t s)
{
    const int64_t total_chunks = (int64_t)(prelayout_bytes(n, k) / 16);
    if (total_chunks == 0) return QM_OK;
    const int64_t blocks = (total_chunks + 255) / 256;
    prelayout_kernel<kPreWarps, kPreRG, kPreMS><<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, s>>>(
        B, reinterpret_cast<uint4 *>(Bp), n, k, pre_rounds(k), total_chunks);
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? QM_OK : record_cuda_error(e, "prelayout_kernel launch");
}

int rmma_launch_prelaid(const GemmArgs &g, const DeviceCtx &ctx)
{
    if (!rmma_eligible(g)) return QM_ERR_ARG;
    return rmma_launch_cfg<kPreWarps, kPreRG, kPreMS, 1>(g, ctx);
}

}  // namespace qm
