// Packed-int4 GEMM for sm_100a, decode form (few rows of A, many rows of B): weight streaming.
//
// Same contract as gemm_tc_kernel (exact int32 C = A * B^T on nibbles; replaces the reference's
// igemm<Config>, kernel.cu:62-266) for m <= 64.  B (the weights, n x k) is the large operand and every
// byte of it is read exactly once, so the kernel is built to keep as many bytes of B in flight per SM as
// possible and to touch them as few times as possible on the way to the tensor core:
//
//  * 128 rows of B sit on the UMMA M axis, the (padded) rows of A on the UMMA N axis (BN = 16, 32 or 64).
//  * Warp 0, one lane: TMA producer.  A stage is 256 elements of K: two 64-byte-wide boxes of 128 B rows
//    (64-byte TMA swizzle) and two of BN A rows (linear), into a ring of SP packed stages.  Nothing else
//    in the CTA's shared memory is large, so the ring takes ~160 KB: that many bytes are in flight per SM.
//  * Warps 6-13: B converters.  Thread = one B row of one 128-element sub-block: four conflict-free
//    16-byte loads, the s4 -> s8 split in registers, and one tcgen05.st of 32 columns into a ring of SC
//    operand stages in TMEM.  The converted weights never go back to shared memory: tcgen05.mma takes them
//    as its A operand from TMEM.  Per stage the shared-memory pipe carries the 16 KB TMA write and the
//    16 KB of converter loads, against 96 KB when the converted tile is staged in shared memory.
//  * Warps 14-15: A converters, packed rows -> K-major SWIZZLE_128B int8 tile in shared memory (the
//    MMA's B operand; 4 KB per stage at BN = 16).
//  * Warp 1, one lane: eight tcgen05.mma.kind::i8 (M = 128, N = BN, K = 32) per stage into one of two
//    TMEM accumulators; tcgen05.commit frees the operand stage and publishes finished accumulators.
//  * Warps 2-5: epilogue.  tcgen05.ld, arithmetic shift by 8, C[q][p] stores (lanes hold consecutive p:
//    each column is one coalesced 128-byte store).  With K split over CTAs the partial tiles meet in
//    scratch memory and whichever partition arrives last adds them up (no CTA waits for another).
//
// TMEM map (512 / R columns): two accumulators of BN columns, then the operand ring of SC stages, 128 lanes x
// 32 columns per sub-block (128 bytes of K per row: four 32-byte MMA slices, each 16 bytes of even
// elements then 16 bytes of odd elements, the K order the A converters produce as well).
//
// Launches chain through programmatic dependent launch: set-up overlaps the previous kernel's tail and
// global memory is touched only after griddepcontrol.wait.  All waits are bounded as in gemm_tc_kernel.
#include <atomic>
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "qm_epilogue.cuh"
#include "qm_internal.h"
#include "qm_ptx.cuh"
#include "qm_tc_common.cuh"

namespace qm {

namespace {

using namespace ptx;
using namespace tc;

constexpr int kH = 2;             // 128-element sub-blocks per stage
constexpr int kRowsP = 128;       // B rows per tile (UMMA M)
constexpr int kPkRowBytes = 64;   // packed bytes per row per sub-block
constexpr int kPkSubP = kRowsP * kPkRowBytes;  // 8 KB
constexpr int kASubCols = 32;     // TMEM columns per converted sub-block
constexpr int kNumPConvWarps = 8, kNumQConvWarps = 2;
constexpr int kFirstPConvWarp = 6, kFirstQConvWarp = kFirstPConvWarp + kNumPConvWarps;
constexpr int kNumWarps = kFirstQConvWarp + kNumQConvWarps;  // 16
constexpr int kNumThreads = kNumWarps * 32;
constexpr int kQConvThreads = kNumQConvWarps * 32;
constexpr int kArrivals = kNumPConvWarps + kNumQConvWarps;
// R = CTAs of this kernel that fit on one SM at a time.  With R = 2 a CTA takes half of the shared memory, TMEM and
// registers: two CTAs of one launch hide each other's pipeline bubbles, and under programmatic dependent launch the
// next launch's CTAs are resident (set up, first weights requested) while this launch's CTAs are still working.
//
// CL = the K partitions of a tile form a thread-block cluster (one CTA each) and add their partial tiles up through
// the cluster's shared memory instead of global scratch: partition r sends the 32-row quarters it does not own to their
// owners with st.async (data + byte count on the owner's mbarrier) and sums the quarters it owns (quarter q belongs to
// partition q % split_k).
template <int BN, int R, bool CL>
struct DecCfg {
    static_assert(BN == 16 || BN == 32 || BN == 64, "UMMA N of the decode form");
    static_assert(R == 1 || R == 2, "CTAs per SM");
    static_assert(!CL || R == 1, "the cluster form runs one CTA per SM");
    static constexpr int kRxSlotBytes = 32 * BN * 4;              // one quarter of a partial tile, [row][BN] int32
    static constexpr int kRxSlots = 4;                            // owned quarters x senders: at most 2 x 2 (split_k = 3)
    static constexpr int kRxBytes = CL ? kRxSlots * kRxSlotBytes : 0;
    static constexpr int kStageBudget = R == 1 ? 200 * 1024 : 104 * 1024;
    static constexpr int kTmemCols = 512 / R;
    static constexpr int kPkSubQ = BN * kPkRowBytes;
    static constexpr int kCvSubQ = BN * 128;
    static constexpr int kPkStage = kH * (kPkSubP + kPkSubQ);
    static constexpr int kCvStage = kH * kCvSubQ;
    static constexpr int kAccCols = 2 * BN;  // two accumulators
    static constexpr int SC = R == 1 ? (BN <= 32 ? 6 : 4) : (BN <= 32 ? 3 : 2);
    static constexpr int SP_raw = (kStageBudget - SC * kCvStage - kRxBytes) / kPkStage;
    static constexpr int SP = SP_raw > 10 ? 10 : SP_raw;
    static constexpr int kNumBarriers = 2 * SP + 2 * SC + 4 + 2;  // ... + two receive barriers (owned quarters)
    static constexpr int kSmemBytes = 1024 + SC * kCvStage + SP * kPkStage + kRxBytes + kNumBarriers * 8 + 16;
    static constexpr int kQItems = kH * BN * 4;  // 16-byte packed chunks of A per stage
    static constexpr int kQIters = kQItems / kQConvThreads;
    static constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    static_assert(kAccCols + SC * kH * kASubCols <= kTmemCols, "TMEM budget");
    static_assert(R * (kSmemBytes + 1024) <= 232448, "shared memory");
    static_assert(SP >= 2, "packed ring");
    static_assert(kPkStage % 1024 == 0 && kCvSubQ % 1024 == 0, "stage alignment");
    static_assert(kQItems % kQConvThreads == 0, "A items");
};

// 16 bytes into the shared memory of another CTA of the cluster; the bytes are counted on that CTA's mbarrier.
__device__ __forceinline__ void st_async_v4(uint32_t remote_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t remote_bar)
{
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(remote_addr),
                 "r"(a), "r"(b), "r"(c), "r"(d), "r"(remote_bar)
                 : "memory");
}

// L2 prefetch of one TMA box: no shared memory, no barrier, no architectural effect.
__device__ __forceinline__ void tma_prefetch_2d(const void *tmap, int32_t x, int32_t y)
{
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(tmap), "r"(x), "r"(y) : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem desc], int8 -> int32, one CTA.  One thread issues it.
__device__ __forceinline__ void umma_i8_ta1(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
        "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
        "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st_wait()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// One piece of work: stages [kb0, kb1) of output tile `tile`; it is part `part` of the `nparts` pieces of that tile.
struct Work {
    int tile, kb0, kb1, part, nparts;
};

// The list of pieces a CTA runs, the same in every role.  Two ways to cut the (tile, stage) space:
//  * split: every tile is cut into `split_k` near-equal K partitions; pieces are dealt round-robin to the CTAs;
//  * balanced (parts_stride > 0 and split_k == 0): the tiles' stages are laid end to end and CTA c takes the
//    contiguous share [c T / G, (c + 1) T / G) of the T stages, so that every CTA streams the same number of bytes
//    whatever the tile count; a share covers the tail of one tile, whole tiles, and the head of another.
struct WorkList {
    int split_k, nkb, num_items, t, step;  // split form
    long long g, g_end, total;             // balanced form: next stage, end of the share, T
    int cta, num_ctas;

    __device__ __forceinline__ int owner(long long stage) const { return (int)(((stage + 1) * num_ctas - 1) / total); }

    __device__ __forceinline__ void init(int split_k_, int nkb_, int tiles, int cta_, int num_ctas_)
    {
        split_k = split_k_, nkb = nkb_, cta = cta_, num_ctas = num_ctas_;
        num_items = tiles * (split_k > 0 ? split_k : 1);
        t = cta, step = num_ctas;
        total = (long long)tiles * nkb;
        g = (long long)cta * total / num_ctas;
        g_end = (long long)(cta + 1) * total / num_ctas;
    }

    __device__ __forceinline__ bool next(Work &w)
    {
        if (split_k > 0) {
            if (t >= num_items) return false;
            w.tile = t / split_k, w.part = t % split_k, w.nparts = split_k;
            w.kb0 = (int)(((long long)w.part * nkb) / split_k);
            w.kb1 = (int)(((long long)(w.part + 1) * nkb) / split_k);
            t += step;
            return true;
        }
        if (g >= g_end) return false;
        w.tile = (int)(g / nkb);
        const long long base = (long long)w.tile * nkb;
        const long long end = g_end < base + nkb ? g_end : base + nkb;
        w.kb0 = (int)(g - base), w.kb1 = (int)(end - base);
        const int first = owner(base);
        w.nparts = owner(base + nkb - 1) - first + 1;
        w.part = cta - first;
        g = end;
        return true;
    }
};

template <int BN, int R, bool CL>
__global__ void __launch_bounds__(kNumThreads, R)
gemm_dec_kernel(const __grid_constant__ CUtensorMap tmapP, const __grid_constant__ CUtensorMap tmapQ,
                int32_t *__restrict__ C, int64_t ldc, int rowsP, int rowsQ, int K, int *status, int split_k, int parts_stride,
                int32_t *__restrict__ scratch, int *__restrict__ counters, uint16_t *__restrict__ out_bf16,
                const float *__restrict__ scale_a, const float *__restrict__ scale_b)
{
    // out_bf16 != NULL: fused dequantisation, out[q][p] = bf16(float(sum) * scale_a[q] * scale_b[p]) instead of C[q][p] = sum
    // (q = row of A, p = row of B; a NULL scale vector is all ones).
    // split_k >= 1: K partitions per tile (parts_stride = split_k); split_k == 0: balanced shares, at most parts_stride
    // pieces per tile.  Piece `part` of tile `tile` owns scratch slot tile * parts_stride + part.
    using Cfg = DecCfg<BN, R, CL>;
    constexpr int SP = Cfg::SP, SC = Cfg::SC;
    extern __shared__ uint8_t smem_raw[];

    const uint32_t raw_u32 = smem_u32(smem_raw);
    const uint32_t cv0 = (raw_u32 + 1023u) & ~1023u;  // converted A stages: [stage][sub-block][row][128 B]
    const uint32_t pk0 = cv0 + SC * Cfg::kCvStage;    // packed stages: [stage][B sub-blocks (swizzle 64B)][A sub-blocks (linear)]
    const uint32_t rx0 = pk0 + SP * Cfg::kPkStage;    // cluster form: received quarters of partial tiles
    const uint32_t bar0 = rx0 + Cfg::kRxBytes;
    auto pk_full = [&](int s) { return bar0 + 8u * s; };
    auto pk_empty = [&](int s) { return bar0 + 8u * (SP + s); };
    auto cv_full = [&](int s) { return bar0 + 8u * (2 * SP + s); };
    auto cv_empty = [&](int s) { return bar0 + 8u * (2 * SP + SC + s); };
    auto acc_full = [&](int b) { return bar0 + 8u * (2 * SP + 2 * SC + b); };
    auto acc_empty = [&](int b) { return bar0 + 8u * (2 * SP + 2 * SC + 2 + b); };
    auto rx_bar = [&](int qi) { return bar0 + 8u * (2 * SP + 2 * SC + 4 + qi); };
    const uint32_t tmem_slot = bar0 + 8u * Cfg::kNumBarriers;
    uint32_t *tmem_slot_ptr = reinterpret_cast<uint32_t *>(smem_raw + (tmem_slot - raw_u32));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_raw + (tmem_slot + 4 - raw_u32));

    grid_launch_dependents();  // the next launch of the stream may begin its own set-up now

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tilesP = (rowsP + kRowsP - 1) / kRowsP;
    const int tilesQ = (rowsQ + BN - 1) / BN;
    const int num_kb_total = (K + kH * 128 - 1) / (kH * 128);  // stages per tile; TMA zero-fills beyond K
    WorkList work;
    work.init(split_k, num_kb_total, tilesP * tilesQ, (int)blockIdx.x, (int)gridDim.x);
    Work w;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SP; ++s) {
            mbar_init(pk_full(s), 1);
            mbar_init(pk_empty(s), kArrivals);
        }
        for (int s = 0; s < SC; ++s) {
            mbar_init(cv_full(s), kArrivals);
            mbar_init(cv_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 4);
            mbar_init(rx_bar(b), 1);
        }
        *abort_flag = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tmap(&tmapP);
        prefetch_tmap(&tmapQ);
    }
    if (warp == 1) {
        tmem_alloc<1>(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish<1>();
    }
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (CL) {
        // the peers' receive barriers must exist before anything is sent to them
        cluster_arrive();
        cluster_wait();
    }
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;
    const uint32_t tmem_a0 = tmem_base + Cfg::kAccCols;
    if (warp == 0 && lane == 0) {
        // Ask L2 for the first ring-full of B before waiting for the previous kernel: a prefetch changes nothing
        // the program can observe (L2 is the coherence point, so even a B the previous kernel still writes reads
        // correctly afterwards), and the loads issued after the wait then find their lines on the way or in L2.
        WorkList ahead = work;
        Work wa;
        int n = 0;
        while (n < SP && ahead.next(wa)) {
            const int yP = (wa.tile % tilesP) * kRowsP;
            for (int kb = wa.kb0; kb < wa.kb1 && n < SP; ++kb, ++n) {
#pragma unroll
                for (int h = 0; h < kH; ++h) tma_prefetch_2d(&tmapP, (kb * kH + h) * kPkRowBytes, yP);
            }
        }
    }
    grid_dependency_wait();  // nothing before this line read or wrote global memory (the prefetch returns no data)

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            while (ok && work.next(w)) {
                const int yP = (w.tile % tilesP) * kRowsP;
                const int yQ = (w.tile / tilesP) * BN;
                for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
                    const int s = it % SP;
                    const uint32_t ph = (it / SP) & 1u;
                    if (!mbar_wait(pk_empty(s), ph ^ 1u, abort_flag)) {
                        report_timeout(status, kWaitProducerSlot);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    const uint32_t dst = pk0 + s * Cfg::kPkStage;
                    mbar_arrive_expect_tx(pk_full(s), Cfg::kPkStage);
#pragma unroll
                    for (int h = 0; h < kH; ++h) {
                        const int x = (kb * kH + h) * kPkRowBytes;
                        tma_load_2d(dst + h * kPkSubP, &tmapP, x, yP, pk_full(s));
                        tma_load_2d(dst + kH * kPkSubP + h * Cfg::kPkSubQ, &tmapQ, x, yQ, pk_full(s));
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            uint32_t it = 0, lt = 0;
            bool ok = true;
            for (; ok && work.next(w); ++lt) {
                const int buf = lt & 1;
                const uint32_t bph = (lt >> 1) & 1u;
                if (!mbar_wait(acc_empty(buf), bph ^ 1u, abort_flag)) {
                    report_timeout(status, kWaitMmaAcc);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                const int kb0 = w.kb0;
                for (int kb = kb0; kb < w.kb1; ++kb, ++it) {
                    const int s = it % SC;
                    const uint32_t ph = (it / SC) & 1u;
                    if (!mbar_wait(cv_full(s), ph, abort_flag)) {
                        report_timeout(status, kWaitMmaOperands);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
#pragma unroll
                    for (int h = 0; h < kH; ++h) {
                        const uint64_t dQ = make_smem_desc(cv0 + s * Cfg::kCvStage + h * Cfg::kCvSubQ);
                        const uint32_t ta = tmem_a0 + (uint32_t)((s * kH + h) * kASubCols);
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4)
                            umma_i8_ta1(tmem_d, ta + 8u * k4, dQ + 2u * k4, Cfg::kIdesc, (kb != kb0 || (h | k4) != 0) ? 1u : 0u);
                    }
                    umma_commit<1>(cv_empty(s));
                }
                if (ok) umma_commit<1>(acc_full(buf));
            }
        }
        __syncwarp();
    } else if (warp < kFirstPConvWarp) {
        // ------------------------------ epilogue ------------------------------
        const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are the ones this warp may read
        uint32_t lt = 0;
        for (; work.next(w); ++lt) {
            const int tile = w.tile;
            const int buf = lt & 1;
            const uint32_t bph = (lt >> 1) & 1u;
            if (!warp_wait<false>(acc_full(buf), bph, abort_flag, lane)) {
                if (lane == 0) {
                    report_timeout(status, kWaitEpilogueAcc);
                    *abort_flag = 1;
                }
                break;
            }
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN);
            const int row = quarter * 32 + lane;
            const int p = (tile % tilesP) * kRowsP + row;  // row of B = column of C
            const int q0 = (tile / tilesP) * BN;           // first row of A = row of C
            // CNT finished elements of column p, rows q_first .. q_first + CNT - 1 (values >> SHIFT): int32 store, or the
            // dequantised bf16 store.  The choice is made once per call, outside the unrolled loops.
            auto put_cols = [&](auto shift_tag, const auto &vals, int first, int q_first) {
                constexpr int SHIFT = decltype(shift_tag)::value;
                if (p >= rowsP) return;
                if (out_bf16) {
                    const float sbp = scale_b ? __ldg(scale_b + p) : 1.0f;
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (q_first + j < rowsQ)
                            out_bf16[(int64_t)(q_first + j) * ldc + p] = (uint16_t)dequant_bf16_bits(
                                (int32_t)vals[first + j] >> SHIFT, scale_a ? __ldg(scale_a + q_first + j) : 1.0f, sbp);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (q_first + j < rowsQ) C[(int64_t)(q_first + j) * ldc + p] = (int32_t)vals[first + j] >> SHIFT;
                }
            };
            if constexpr (CL) {
                if (w.nparts > 1) {
                    // One piece per CTA, cluster rank = piece.  Row = lane, BN int32 per row, 16-byte chunks XOR-swizzled
                    // so that the owner's 16-byte reads do not collide on banks.
                    constexpr int kChunks = BN / 4;
                    const uint32_t swz = BN == 16 ? (uint32_t)((lane >> 1) & 3) : (uint32_t)(lane & 7);
                    uint32_t v[BN];
#pragma unroll
                    for (int c = 0; c < BN; c += 16) tmem_ld_x16(taddr + c, *reinterpret_cast<uint32_t(*)[16]>(&v[c]));
                    tmem_ld_wait();
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty(buf));
                    const int owner = quarter % w.nparts, qi = quarter / w.nparts;
                    if (owner != w.part) {
                        const int sender = w.part < owner ? w.part : w.part - 1;
                        const uint32_t slot = rx0 + (uint32_t)((qi * (w.nparts - 1) + sender) * Cfg::kRxSlotBytes) + (uint32_t)lane * (BN * 4);
                        const uint32_t rslot = mapa_cluster(slot, (uint32_t)owner);
                        const uint32_t rbar = mapa_cluster(rx_bar(qi), (uint32_t)owner);
#pragma unroll
                        for (int c = 0; c < kChunks; ++c)
                            st_async_v4(rslot + (((uint32_t)c ^ swz) << 4), (uint32_t)((int32_t)v[4 * c] >> 8), (uint32_t)((int32_t)v[4 * c + 1] >> 8),
                                        (uint32_t)((int32_t)v[4 * c + 2] >> 8), (uint32_t)((int32_t)v[4 * c + 3] >> 8), rbar);
                    } else {
                        if (lane == 0) mbar_arrive_expect_tx(rx_bar(qi), (uint32_t)((w.nparts - 1) * Cfg::kRxSlotBytes));
                        __syncwarp();
                        if (!warp_wait<false>(rx_bar(qi), 0u, abort_flag, lane)) {
                            if (lane == 0) {
                                report_timeout(status, kWaitSplitK);
                                *abort_flag = 1;
                            }
                            break;
                        }
#pragma unroll
                        for (int j = 0; j < BN; ++j) v[j] = (uint32_t)((int32_t)v[j] >> 8);
                        for (int sdr = 0; sdr < w.nparts - 1; ++sdr) {
                            const uint32_t slot = rx0 + (uint32_t)((qi * (w.nparts - 1) + sdr) * Cfg::kRxSlotBytes) + (uint32_t)lane * (BN * 4);
#pragma unroll
                            for (int c = 0; c < kChunks; ++c) {
                                const uint4 x = lds128(slot + (((uint32_t)c ^ swz) << 4));
                                v[4 * c] += x.x, v[4 * c + 1] += x.y, v[4 * c + 2] += x.z, v[4 * c + 3] += x.w;
                            }
                        }
#pragma unroll
                        for (int c = 0; c < BN; c += 16) put_cols(std::integral_constant<int, 0>{}, v, c, q0 + c);
                    }
                    continue;
                }
            }
            // Partial tiles go to scratch as [column][row] (coalesced); whichever piece of the tile finishes last
            // sums all of them.  Each warp owns 32 rows of the tile and its own arrival counter: nobody waits.
            int32_t *parts = scratch + (int64_t)tile * parts_stride * (kRowsP * BN);
            int32_t *mine = parts + (int64_t)w.part * (kRowsP * BN);
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                uint32_t v[16];
                tmem_ld_x16(taddr + c, v);
                tmem_ld_wait();
                if (c + 16 == BN) {
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty(buf));  // the last columns are in registers
                }
                if (w.nparts == 1) {
                    put_cols(std::integral_constant<int, 8>{}, v, 0, q0 + c);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) __stcg(mine + (c + j) * kRowsP + row, (int32_t)v[j] >> 8);
                }
            }
            if (w.nparts == 1) continue;
            __threadfence();
            __syncwarp();
            int last = 0;
            if (lane == 0) {
                int *ctr = counters + tile * 4 + quarter;
                last = (atomicAdd(ctr, 1) == w.nparts - 1) ? 1 : 0;
                if (last) *ctr = 0;  // ready for the next launch
            }
            last = __shfl_sync(0xFFFFFFFFu, last, 0);
            if (!last) continue;
            __threadfence();
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                int32_t sum[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) sum[j] = 0;
                for (int sk = 0; sk < w.nparts; ++sk) {
                    const int32_t *src = parts + (int64_t)sk * (kRowsP * BN) + c * kRowsP + row;
#pragma unroll
                    for (int j = 0; j < 16; ++j) sum[j] += __ldcg(src + j * kRowsP);
                }
                put_cols(std::integral_constant<int, 0>{}, sum, 0, q0 + c);
            }
        }
    } else if (warp < kFirstQConvWarp) {
        // ------------------------------ B converters: packed smem -> registers -> TMEM ------------------------------
        const int quarter = warp & 3;                 // TMEM lane quarter this warp may write
        const int h = (warp - kFirstPConvWarp) >> 2;  // sub-block of the stage
        const int r = quarter * 32 + lane;            // row of the tile = TMEM lane
        const uint32_t swz = (uint32_t)((r >> 1) & 3);  // 64-byte TMA swizzle: chunk ^= (row / 2) % 4
        uint32_t it = 0;
        bool ok = true;
        while (ok && work.next(w)) {
            for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
                const int ps = it % SP, cs = it % SC;
                const uint32_t pph = (it / SP) & 1u, cph = (it / SC) & 1u;
                if (!warp_wait<false>(pk_full(ps), pph, abort_flag, lane)) {
                    if (lane == 0) {
                        report_timeout(status, kWaitConvertPacked);
                        *abort_flag = 1;
                    }
                    ok = false;
                    break;
                }
                const uint32_t src = pk0 + ps * Cfg::kPkStage + h * kPkSubP + (uint32_t)r * kPkRowBytes;
                uint4 w[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) w[c] = lds128(src + (((uint32_t)c ^ swz) << 4));
                uint32_t v[32];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint4 lo, hi;
                    split_s4x32(w[c], lo, hi);
                    v[8 * c + 0] = lo.x, v[8 * c + 1] = lo.y, v[8 * c + 2] = lo.z, v[8 * c + 3] = lo.w;
                    v[8 * c + 4] = hi.x, v[8 * c + 5] = hi.y, v[8 * c + 6] = hi.z, v[8 * c + 7] = hi.w;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(pk_empty(ps));  // the packed rows are in registers now
                if (!warp_wait<false>(cv_empty(cs), cph ^ 1u, abort_flag, lane)) {
                    if (lane == 0) {
                        report_timeout(status, kWaitConvertSlot);
                        *abort_flag = 1;
                    }
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                tmem_st_x32(tmem_a0 + ((uint32_t)(quarter * 32) << 16) + (uint32_t)((cs * kH + h) * kASubCols), v);
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(cv_full(cs));
            }
        }
    } else {
        // ------------------------------ A converters: packed smem -> swizzled int8 smem ------------------------------
        const int ctid = threadIdx.x - kFirstQConvWarp * 32;
        uint32_t it = 0;
        bool ok = true;
        while (ok && work.next(w)) {
            for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
                const int ps = it % SP, cs = it % SC;
                const uint32_t pph = (it / SP) & 1u, cph = (it / SC) & 1u;
                if (!warp_wait<false>(pk_full(ps), pph, abort_flag, lane)) {
                    if (lane == 0) {
                        report_timeout(status, kWaitConvertPacked);
                        *abort_flag = 1;
                    }
                    ok = false;
                    break;
                }
                if (!warp_wait<false>(cv_empty(cs), cph ^ 1u, abort_flag, lane)) {
                    if (lane == 0) {
                        report_timeout(status, kWaitConvertSlot);
                        *abort_flag = 1;
                    }
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t src = pk0 + ps * Cfg::kPkStage + kH * kPkSubP;  // both sub-blocks, contiguous
                const uint32_t dst = cv0 + cs * Cfg::kCvStage;
                constexpr int kBatch = Cfg::kQIters < 4 ? Cfg::kQIters : 4;
#pragma unroll 1
                for (int j0 = 0; j0 < Cfg::kQIters; j0 += kBatch) {
                    uint4 wq[kBatch];
#pragma unroll
                    for (int j = 0; j < kBatch; ++j) wq[j] = lds128(src + ((j0 + j) * kQConvThreads + ctid) * 16);
#pragma unroll
                    for (int j = 0; j < kBatch; ++j) {
                        const int i = (j0 + j) * kQConvThreads + ctid;  // chunk index over [sub-block][row][4]
                        const int sub = i / (BN * 4), rem = i % (BN * 4);
                        convert_chunk_to_smem(dst + sub * Cfg::kCvSubQ, rem >> 2, rem & 3, wq[j]);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(pk_empty(ps));
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(cv_full(cs));
            }
        }
    }

    // ------------------------------ teardown ------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (CL) {
        // peers may still be writing into this CTA's receive slots (always, if this CTA gave up on a wait)
        cluster_arrive();
        cluster_wait();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<1>(tmem_base, Cfg::kTmemCols);
    }
}

template <int BN, int R, bool CL>
int prepare_one()
{
    cudaError_t e = cudaFuncSetAttribute(gemm_dec_kernel<BN, R, CL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         DecCfg<BN, R, CL>::kSmemBytes);
    if (e != cudaSuccess) return record_cuda_error(e, "cudaFuncSetAttribute(shared memory)");
    return QM_OK;
}

template <int BN, int R, bool CL>
int launch_one(const GemmArgs &g, const DeviceCtx &ctx, int split_k, bool balanced, int32_t *scratch, size_t scratch_bytes,
               int *counters, int num_counters)
{
    using Cfg = DecCfg<BN, R, CL>;
    const int rowsP = g.n, rowsQ = g.m;
    const int64_t kbytes = g.k / 2;
    CUtensorMap tmP, tmQ;
    int st = make_packed_tmap(&tmP, g.B, rowsP, kbytes, kRowsP, CU_TENSOR_MAP_SWIZZLE_64B);
    if (st != QM_OK) return st;
    st = make_packed_tmap(&tmQ, g.A, rowsQ, kbytes, BN, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st != QM_OK) return st;

    const int tilesP = (rowsP + kRowsP - 1) / kRowsP;
    const int tilesQ = (rowsQ + BN - 1) / BN;
    const int64_t tiles = (int64_t)tilesP * tilesQ;
    const int num_kb = (g.k + kH * 128 - 1) / (kH * 128);
    const int sms = (ctx.num_sms > 0 ? ctx.num_sms : 1) * R;  // CTA slots
    if (tiles > 0x7FFFFFFF / 64) return QM_ERR_SHAPE;
    int units, parts_stride;
    if (balanced) {
        // one contiguous share of the tiles * num_kb stages per CTA; a tile meets at most parts_stride shares
        const int64_t total = tiles * num_kb;
        units = total < sms ? (int)total : sms;
        const int64_t share = total / units;  // shortest share, >= 1
        parts_stride = (int)((num_kb + share - 1) / share) + 1;
        split_k = 0;
    } else {
        if (split_k < 1 || split_k > num_kb) return QM_ERR_ARG;
        const int64_t items = tiles * split_k;
        units = items < sms ? (int)items : sms;
        parts_stride = split_k;
        if (CL) {
            if (split_k < 2 || split_k > 4 || items > 0x7FFFFFFF) return QM_ERR_ARG;
            units = (int)items;  // one piece per CTA, the pieces of a tile are one cluster
        }
    }
    if (parts_stride > 1 && !CL) {
        if ((size_t)tiles * parts_stride * kRowsP * BN * sizeof(int32_t) > scratch_bytes || tiles * 4 > num_counters)
            return QM_ERR_WORKSPACE;
        if (!scratch || !counters) return QM_ERR_NULL;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)units, 1, 1);
    cfg.blockDim = dim3(kNumThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = g.stream;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    static const bool allow_pdl = !std::getenv("QM_NO_PDL");
    if (allow_pdl) {
        // may begin while the previous kernel of the stream drains; the kernel itself waits before global accesses
        attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
        ++cfg.numAttrs;
    }
    if (CL) {
        attr[cfg.numAttrs].id = cudaLaunchAttributeClusterDimension;
        attr[cfg.numAttrs].val.clusterDim.x = (unsigned)split_k;
        attr[cfg.numAttrs].val.clusterDim.y = 1;
        attr[cfg.numAttrs].val.clusterDim.z = 1;
        ++cfg.numAttrs;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_dec_kernel<BN, R, CL>, tmP, tmQ, g.C, g.ldc, rowsP, rowsQ, g.k, ctx.status, split_k,
                                       parts_stride, scratch, counters, static_cast<uint16_t *>(g.out_bf16), g.scale_a, g.scale_b);
    if (e != cudaSuccess) return record_cuda_error(e, "gemm_dec_kernel launch");
    return QM_OK;
}

// g_cluster_cap[device][log2(BN / 16)][size - 2]: clusters of `size` CTAs of the cluster form that the device runs at once
std::atomic<int> g_cluster_cap[64][3][3];

template <int BN>
void query_cluster_capacity(int device)
{
    for (int size = 2; size <= 4; ++size) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(size * 64), 1, 1);
        cfg.blockDim = dim3(kNumThreads, 1, 1);
        cfg.dynamicSmemBytes = DecCfg<BN, 1, true>::kSmemBytes;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)size;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, gemm_dec_kernel<BN, 1, true>, &cfg) != cudaSuccess) {
            cudaGetLastError();  // not fatal: the table's estimate stays in force
            clusters = 0;
        }
        g_cluster_cap[device & 63][BN == 16 ? 0 : (BN == 32 ? 1 : 2)][size - 2].store(clusters, std::memory_order_release);
    }
}

}  // namespace

int dec_cluster_capacity(int device, int tile_n, int size)
{
    if (size < 2 || size > 4 || (tile_n != 16 && tile_n != 32 && tile_n != 64)) return 0;
    return g_cluster_cap[device & 63][tile_n == 16 ? 0 : (tile_n == 32 ? 1 : 2)][size - 2].load(std::memory_order_acquire);
}

int dec_prepare_device()
{
    int device = 0;
    if (cudaGetDevice(&device) == cudaSuccess) {
        query_cluster_capacity<16>(device);
        query_cluster_capacity<32>(device);
        query_cluster_capacity<64>(device);
    }
    int st = prepare_one<16, 1, false>();
    if (st == QM_OK) st = prepare_one<32, 1, false>();
    if (st == QM_OK) st = prepare_one<64, 1, false>();
    if (st == QM_OK) st = prepare_one<16, 2, false>();
    if (st == QM_OK) st = prepare_one<16, 1, true>();
    if (st == QM_OK) st = prepare_one<32, 1, true>();
    if (st == QM_OK) st = prepare_one<64, 1, true>();
    return st;
}

int dec_launch(const GemmArgs &g, const TcPlan &p, const DeviceCtx &ctx)
{
    const bool bal = p.stream_k == 1;
#define QM_DEC_ARGS g, ctx, p.split_k, bal, ctx.scratch, ctx.scratch_bytes, ctx.counters, ctx.num_counters
    if (p.ctas_per_sm == 2) {
        if (p.tile_n != 16 || p.stream_k == 2) return QM_ERR_ARG;
        return launch_one<16, 2, false>(QM_DEC_ARGS);
    }
    if (p.stream_k == 2) {  // K partitions of a tile = one cluster, summed through its shared memory
        switch (p.tile_n) {
        case 16: return launch_one<16, 1, true>(QM_DEC_ARGS);
        case 32: return launch_one<32, 1, true>(QM_DEC_ARGS);
        case 64: return launch_one<64, 1, true>(QM_DEC_ARGS);
        default: return QM_ERR_ARG;
        }
    }
    switch (p.tile_n) {
    case 16: return launch_one<16, 1, false>(QM_DEC_ARGS);
    case 32: return launch_one<32, 1, false>(QM_DEC_ARGS);
    case 64: return launch_one<64, 1, false>(QM_DEC_ARGS);
    default: return QM_ERR_ARG;
    }
#undef QM_DEC_ARGS
}

}  // namespace qm
