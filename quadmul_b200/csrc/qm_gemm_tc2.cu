// Packed-int4 GEMM for sm_100a, large-shape form: 256 x 256 CTA-pair tile with operand A fed to the
// tensor core from TMEM instead of shared memory.
//
// Same contract as gemm_tc_kernel (exact int32 C = A * B^T on nibbles; replaces the reference's
// igemm<Config>, kernel.cu:62-266).  The difference is where the converted A lives.  The pair tile of
// gemm_tc_kernel is bound by the shared-memory data pipe: per 128 elements of K each SM moves 16 KB
// of TMA writes, 16 KB of converter loads, 32 KB of converter stores and 32 KB of MMA operand reads.
// Here the four A-converter warps keep their 128 rows in registers after the s4 -> s8 split and write
// them to TMEM with tcgen05.st; tcgen05.mma takes A as [tmem] and only B as a shared-memory
// descriptor.  That removes A's 16 KB of stores and 16 KB of MMA reads per 128 elements of K.
//
// A pipeline stage holds H sub-blocks of 128 K-elements (H = 2: 256 elements, 8 MMAs per stage), so the
// barrier hand-offs and tcgen05.commit are paid once per 2 x 512 tensor-clocks.
//
// TMEM map (512 columns): [0, 256) one int32 accumulator (128 lanes x 256 columns per CTA);
// [256, 256 + 32*H*S) a ring of S converted A stages, 128 lanes x 32 columns per sub-block (128 bytes
// of K per row: four 32-byte MMA slices, each = 16 bytes of even elements then 16 bytes of odd
// elements, the same K order the B converters produce).  With one accumulator the epilogue does not
// overlap the next tile's MMAs; the loaders and converters do run ahead during it.
//
// Warps: 0 TMA producer, 1 MMA issuer (leader CTA only) and TMEM owner, 2-9 epilogue (two per TMEM lane
// quarter), 10-13 A converters (warp & 3 = TMEM lane quarter = 32-row block), 14-21 B converters.
// Packed A sub-blocks are loaded with the 64-byte TMA swizzle so that one thread can read its whole
// 64-byte row as four conflict-free 16-byte loads; packed B sub-blocks are linear as in gemm_tc_kernel.
// All waits are bounded as in gemm_tc_kernel.
#include <cuda.h>

#include <atomic>

#include <cstdio>
#include <cstdlib>

#include "qm_epilogue.cuh"
#include "qm_internal.h"
#include "qm_ptx.cuh"
#include "qm_tc_common.cuh"
#include "qm_tile_table.h"

namespace qm {

namespace {

using namespace ptx;
using namespace tc;

constexpr int kBN = 256;         // UMMA N of the pair tile
constexpr int kRowsA = 128;      // A rows per CTA
constexpr int kRowsB = kBN / 2;  // B rows per CTA
constexpr int kSubK = 128;       // K elements per sub-block
constexpr int kPkRowBytes = 64;  // packed bytes per row per sub-block
constexpr int kCvRowBytes = 128;
constexpr int kPkSubA = kRowsA * kPkRowBytes;  // 8 KB
constexpr int kPkSubB = kRowsB * kPkRowBytes;  // 8 KB
constexpr int kCvSub = kRowsB * kCvRowBytes;   // 16 KB
constexpr int kASubCols = 32;
constexpr int kAccCols = kBN;
constexpr int kTmemCols = 512;
constexpr int kNumEpiWarps = 8;  // two per TMEM lane quarter, 128 accumulator columns each
constexpr int kNumAConvWarps = 4, kNumBConvWarps = 8;
constexpr int kFirstAConvWarp = 2 + kNumEpiWarps, kFirstBConvWarp = kFirstAConvWarp + kNumAConvWarps;
constexpr int kNumWarps = kFirstBConvWarp + kNumBConvWarps;  // 22
constexpr int kNumThreads = kNumWarps * 32;
constexpr int kBConvThreads = kNumBConvWarps * 32;
constexpr int kBItemsSub = kRowsB * 4;                      // 16-byte packed chunks per sub-block
constexpr int kBItersSub = kBItemsSub / kBConvThreads;      // 2
constexpr int kArrivals = kNumAConvWarps + kNumBConvWarps;  // converter warps per CTA
constexpr int kEpiBufBytes = kTmaStoreBufBytes;  // per epilogue warp: one 4 KB TMA-store buffer (or the 16-column fallback transposer)
constexpr int kEpiBytes = kNumEpiWarps * kEpiBufBytes;
static_assert(kEpiBufBytes >= EpilogueStage<16>::kBytesPerWarp, "epilogue buffer");
constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
static_assert(kBItemsSub % kBConvThreads == 0, "B items");

template <int H>
struct Tc2Cfg {
    static constexpr int S = 6 / H;   // converted stages: B in shared memory, A in TMEM
    static constexpr int SP = 6 / H;  // packed stages
    static constexpr int kPkStage = H * (kPkSubA + kPkSubB);
    static constexpr int kCvStage = H * kCvSub;
    static constexpr int kAStageCols = H * kASubCols;
    static constexpr int kNumBarriers = 2 * SP + 2 * S + 2;
    static constexpr int kSmemBytes = 1024 + S * kCvStage + SP * kPkStage + kEpiBytes + kNumBarriers * 8 + 16;
    static_assert(kAccCols + S * kAStageCols <= kTmemCols, "TMEM budget");
    static_assert(kSmemBytes <= 232448, "shared memory");
};

// D[tmem] (+)= A[tmem] * B[smem desc], CTA pair, int8 -> int32.  One thread of the leader CTA.
__device__ __forceinline__ void umma_i8_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::i8 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// One arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair once every MMA
// issued so far has finished (a barrier signal, not a data transfer).
__device__ __forceinline__ void umma_commit_pair(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"((uint16_t)3)
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

// DQ = fused dequantising epilogue: tmapC describes a bf16 output, every element is the int32 sum times scale_a[row] times
// scale_b[column] rounded to bf16 (qm_epilogue.cuh); stores go through TMA only and K is not split.
template <int H, bool MC, bool DQ>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                const __grid_constant__ CUtensorMap tmapC, int use_tma_store, int32_t *__restrict__ C, int64_t ldc, int M,
                int N, int K, int *status, int split_k, int tail_tiles, int tail_split, const float *__restrict__ scale_a,
                const float *__restrict__ scale_b)
{
    using Cfg = Tc2Cfg<H>;
    constexpr int S = Cfg::S, SP = Cfg::SP;
    extern __shared__ uint8_t smem_raw[];
    // Programmatic dependent launch: the next kernel of the stream may begin its set-up now, and this kernel's own set-up
    // (barriers, TMEM, tensor-map prefetch) runs while the previous kernel drains.  The TMA producer waits for the previous
    // kernel before its first load; every other access to global memory follows data that the producer loaded.
    grid_launch_dependents();
    const uint32_t raw_u32 = smem_u32(smem_raw);
    const uint32_t cv0 = (raw_u32 + 1023u) & ~1023u;   // converted B stages: [stage][sub-block][row][128 B]
    const uint32_t pk0 = cv0 + S * Cfg::kCvStage;      // packed stages: [stage][A sub-blocks (swizzle 64B)][B sub-blocks (linear)]
    const uint32_t epi0 = pk0 + SP * Cfg::kPkStage;    // epilogue transpose buffers
    const uint32_t bar0 = epi0 + kEpiBytes;
    auto pk_full = [&](int s) { return bar0 + 8u * s; };
    auto pk_empty = [&](int s) { return bar0 + 8u * (SP + s); };
    auto cv_full = [&](int s) { return bar0 + 8u * (2 * SP + s); };       // leader's copy is the one waited on
    auto cv_empty = [&](int s) { return bar0 + 8u * (2 * SP + S + s); };  // one per CTA
    const uint32_t acc_full = bar0 + 8u * (2 * SP + 2 * S);
    const uint32_t acc_empty = acc_full + 8u;
    const uint32_t tmem_slot = bar0 + 8u * Cfg::kNumBarriers;
    uint32_t *tmem_slot_ptr = reinterpret_cast<uint32_t *>(smem_raw + (tmem_slot - raw_u32));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_raw + (tmem_slot + 4 - raw_u32));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta_rank = cluster_ctarank();
    const int unit = (int)(blockIdx.x >> 1), num_units = (int)(gridDim.x >> 1);
    const int tilesP = (M + 255) / 256, tilesQ = (N + kBN - 1) / kBN;
    // A work item is one K partition of one tile.  All tiles but the last tail_tiles of the static order are cut into
    // split_k partitions, the last tail_tiles (the ones that would leave most CTA pairs idle in a last round of whole tiles)
    // into tail_split; where a tile has more than one partition they add into a C that the host zeroed.
    const int tiles_all = tilesP * tilesQ;
    const int head_items = (tiles_all - tail_tiles) * split_k;
    const int num_tiles = head_items + tail_tiles * tail_split;  // work items
    const int num_kb_total = (K + H * kSubK - 1) / (H * kSubK);  // stages per tile; TMA zero-fills beyond K
    auto item_tile = [&](int item) { return item < head_items ? item / split_k : tiles_all - tail_tiles + (item - head_items) / tail_split; };
    auto item_parts = [&](int item) { return item < head_items ? split_k : tail_split; };
    auto item_part = [&](int item) { return item < head_items ? item % split_k : (item - head_items) % tail_split; };
    auto kb_begin = [&](int item) { return (int)(((long long)item_part(item) * num_kb_total) / item_parts(item)); };
    auto kb_end = [&](int item) { return (int)(((long long)(item_part(item) + 1) * num_kb_total) / item_parts(item)); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < SP; ++s) {
            mbar_init(pk_full(s), 1);
            mbar_init(pk_empty(s), kArrivals);
        }
        for (int s = 0; s < S; ++s) {
            mbar_init(cv_full(s), 2 * kArrivals);
            mbar_init(cv_empty(s), 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 2 * kNumEpiWarps);
        *abort_flag = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tmap(&tmapA);
        prefetch_tmap(&tmapB);
        if (use_tma_store) prefetch_tmap(&tmapC);
    }
    if (warp == 1) {
        tmem_alloc<2>(tmem_slot, kTmemCols);
        tmem_relinquish<2>();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;
    const uint32_t tmem_a0 = tmem_base + kAccCols;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            grid_dependency_wait();  // nothing before this line read or wrote global memory
            for (int t = unit; t < num_tiles && ok; t += num_units) {
                int tp, tq;
                tile_coords(item_tile(t), tilesP, tilesQ, tp, tq);
                const int yA = tp * 256 + (int)cta_rank * kRowsA;
                const int yB = tq * kBN + (int)cta_rank * kRowsB;
                for (int kb = kb_begin(t), kbe = kb_end(t); kb < kbe; ++kb, ++it) {
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
                    for (int h = 0; h < H; ++h) {
                        const int x = (kb * H + h) * kPkRowBytes;
                        tma_load_2d(dst + h * kPkSubA, &tmapA, x, yA, pk_full(s));
                        tma_load_2d(dst + H * kPkSubA + h * kPkSubB, &tmapB, x, yB, pk_full(s));
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (leader CTA) ------------------------------
        if (lane == 0 && cta_rank == 0) {
            uint32_t it = 0, lt = 0;
            bool ok = true;
            for (int t = unit; t < num_tiles && ok; t += num_units, ++lt) {
                if (!mbar_wait(acc_empty, (lt & 1u) ^ 1u, abort_flag)) {
                    report_timeout(status, kWaitMmaAcc);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after_sync();
                const int kb0 = kb_begin(t);
                for (int kb = kb0, kbe = kb_end(t); kb < kbe; ++kb, ++it) {
                    const int s = it % S;
                    const uint32_t ph = (it / S) & 1u;
                    if (!mbar_wait(cv_full(s), ph, abort_flag)) {
                        report_timeout(status, kWaitMmaOperands);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
#pragma unroll
                    for (int h = 0; h < H; ++h) {
                        const uint64_t dB = make_smem_desc(cv0 + s * Cfg::kCvStage + h * kCvSub);
                        const uint32_t ta = tmem_a0 + (uint32_t)(s * Cfg::kAStageCols + h * kASubCols);
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4)
                            umma_i8_ta(tmem_base, ta + 8u * k4, dB + 2u * k4, kIdesc, (kb != kb0 || (h | k4) != 0) ? 1u : 0u);
                    }
                    if constexpr (MC) {
                        umma_commit_pair(cv_empty(s));
                    } else {
                        umma_commit<2>(cv_empty(s));
                        umma_commit<2>(mapa_cluster(cv_empty(s), 1));
                    }
                }
                if (ok) {
                    if constexpr (MC) {
                        umma_commit_pair(acc_full);
                    } else {
                        umma_commit<2>(acc_full);
                        umma_commit<2>(mapa_cluster(acc_full, 1));
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp < kFirstAConvWarp) {
        // ------------------------------ epilogue ------------------------------
        // Warp = (TMEM lane quarter, column half): four 32 x 32 blocks.  Two blocks are held in registers, so the
        // last TMEM load is issued after only two of the four stores; the accumulator is handed back to the MMA
        // issuer at that point and the remaining stores run under the next tile's main loop.
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        uint32_t lt = 0;
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(C) & 15u) == 0) && ((ldc & 3) == 0);
        const uint32_t buf = epi0 + (uint32_t)((warp - 2) * kEpiBufBytes);
        bool buf_used = false;
        for (int t = unit; t < num_tiles; t += num_units, ++lt) {
            int tp, tq;
            tile_coords(item_tile(t), tilesP, tilesQ, tp, tq);
            const bool ok = warp_wait<false>(acc_full, lt & 1u, abort_flag, lane);
            if (!ok) {
                if (lane == 0) {
                    report_timeout(status, kWaitEpilogueAcc);
                    *abort_flag = 1;
                }
                break;
            }
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * 128);
            const int row0 = tp * 256 + (int)cta_rank * kRowsA + quarter * 32;
            const int q0 = tq * kBN + half * 128;
            const bool reduce_add = item_parts(t) > 1;
            auto store = [&](const uint32_t(&v)[32], int col) {
                if (use_tma_store) {
                    if (buf_used) {
                        if (lane == 0) tma_store_wait_read<0>();  // the previous store has finished reading the buffer
                        __syncwarp();
                    }
                    store_block_tma(v, buf, lane, &tmapC, col, row0, false, reduce_add);
                    buf_used = true;
                } else {
                    store_block_rows_swizzled(v, buf, lane, C, ldc, row0, col, M, N, vec_ok);
                }
            };
            uint32_t va[32], vb[32];
            if constexpr (DQ) {
                // this lane's row scale and, spread over the lanes, the scales of the warp's 128 columns
                const int row = row0 + lane;
                const float sa = (scale_a && row < M) ? __ldg(scale_a + row) : 1.0f;
                float sb[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int col = q0 + 32 * i + lane;
                    sb[i] = (scale_b && col < N) ? __ldg(scale_b + col) : 1.0f;
                }
                tmem_ld_x32(taddr, va);
                tmem_ld_x32(taddr + 32, vb);
                tmem_ld_wait();
                if (buf_used) {
                    if (lane == 0) tma_store_wait_read<0>();
                    __syncwarp();
                }
                store_pair_bf16_tma(va, vb, buf, lane, &tmapC, q0, row0, sa, sb[0], sb[1]);
                buf_used = true;
                tmem_ld_x32(taddr + 64, va);
                tmem_ld_x32(taddr + 96, vb);
                tmem_ld_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(acc_empty, 0);
                if (lane == 0) tma_store_wait_read<0>();
                __syncwarp();
                store_pair_bf16_tma(va, vb, buf, lane, &tmapC, q0 + 64, row0, sa, sb[2], sb[3]);
                continue;
            }
            tmem_ld_x32(taddr, va);
            tmem_ld_x32(taddr + 32, vb);
            tmem_ld_wait();
            store(va, q0);
            tmem_ld_x32(taddr + 64, va);
            store(vb, q0 + 32);
            tmem_ld_x32(taddr + 96, vb);
            tmem_ld_wait();
            // every column of this warp's share is in registers: the accumulator may be overwritten
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty, 0);
            store(va, q0 + 64);
            store(vb, q0 + 96);
        }
        if (use_tma_store && lane == 0) tma_store_wait_all();  // the buffer must outlive the stores that read it
        __syncwarp();
    } else if (warp < kFirstBConvWarp) {
        // ------------------------------ A converters: packed smem -> registers -> TMEM ------------------------------
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;              // row of this CTA's A tile = TMEM lane
        const uint32_t swz = (uint32_t)((r >> 1) & 3);  // 64-byte TMA swizzle: chunk ^= (row / 2) % 4
        uint32_t it = 0;
        bool ok = true;
        for (int t = unit; t < num_tiles && ok; t += num_units) {
            for (int kb = kb_begin(t), kbe = kb_end(t); kb < kbe; ++kb, ++it) {
                const int ps = it % SP, cs = it % S;
                const uint32_t pph = (it / SP) & 1u, cph = (it / S) & 1u;
                if (!warp_wait<false>(pk_full(ps), pph, abort_flag, lane)) {
                    if (lane == 0) {
                        report_timeout(status, kWaitConvertPacked);
                        *abort_flag = 1;
                    }
                    ok = false;
                    break;
                }
                const uint32_t src = pk0 + ps * Cfg::kPkStage + (uint32_t)r * kPkRowBytes;
                uint4 w[H][4];
#pragma unroll
                for (int h = 0; h < H; ++h)
#pragma unroll
                    for (int c = 0; c < 4; ++c) w[h][c] = lds128(src + h * kPkSubA + (((uint32_t)c ^ swz) << 4));
                __syncwarp();
                if (lane == 0) mbar_arrive(pk_empty(ps));  // packed rows are in registers now
                if (!warp_wait<false>(cv_empty(cs), cph ^ 1u, abort_flag, lane)) {
                    if (lane == 0) {
                        report_timeout(status, kWaitConvertSlot);
                        *abort_flag = 1;
                    }
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t ta = tmem_a0 + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(cs * Cfg::kAStageCols);
#pragma unroll
                for (int h = 0; h < H; ++h) {
                    uint32_t v[32];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint4 lo, hi;
                        split_s4x32(w[h][c], lo, hi);
                        v[8 * c + 0] = lo.x, v[8 * c + 1] = lo.y, v[8 * c + 2] = lo.z, v[8 * c + 3] = lo.w;
                        v[8 * c + 4] = hi.x, v[8 * c + 5] = hi.y, v[8 * c + 6] = hi.z, v[8 * c + 7] = hi.w;
                    }
                    tmem_st_x32(ta + h * kASubCols, v);
                }
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(cv_full(cs), 0);
            }
        }
    } else {
        // ------------------------------ B converters: packed smem -> swizzled int8 smem ------------------------------
        const int ctid = threadIdx.x - kFirstBConvWarp * 32;
        uint32_t it = 0;
        bool ok = true;
        for (int t = unit; t < num_tiles && ok; t += num_units) {
            for (int kb = kb_begin(t), kbe = kb_end(t); kb < kbe; ++kb, ++it) {
                const int ps = it % SP, cs = it % S;
                const uint32_t pph = (it / SP) & 1u, cph = (it / S) & 1u;
                if (!warp_wait<false>(pk_full(ps), pph, abort_flag, lane)) {
                    if (lane == 0) {
                        report_timeout(status, kWaitConvertPacked);
                        *abort_flag = 1;
                    }
                    ok = false;
                    break;
                }
                const uint32_t src = pk0 + ps * Cfg::kPkStage + H * kPkSubA;
                uint4 w[H][kBItersSub];
#pragma unroll
                for (int h = 0; h < H; ++h)
#pragma unroll
                    for (int j = 0; j < kBItersSub; ++j) w[h][j] = lds128(src + h * kPkSubB + (j * kBConvThreads + ctid) * 16);
                __syncwarp();
                if (lane == 0) mbar_arrive(pk_empty(ps));
                if (!warp_wait<false>(cv_empty(cs), cph ^ 1u, abort_flag, lane)) {
                    if (lane == 0) {
                        report_timeout(status, kWaitConvertSlot);
                        *abort_flag = 1;
                    }
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t dst = cv0 + cs * Cfg::kCvStage;
#pragma unroll
                for (int h = 0; h < H; ++h)
#pragma unroll
                    for (int j = 0; j < kBItersSub; ++j) {
                        const int i = j * kBConvThreads + ctid;
                        convert_chunk_to_smem(dst + h * kCvSub, i >> 2, i & 3, w[h][j]);
                    }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(cv_full(cs), 0);
            }
        }
    }

    // ------------------------------ teardown ------------------------------
    tc_fence_before_sync();
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<2>(tmem_base, kTmemCols);
    }
}

// Zeroes the last tail_tiles 256 x 256 tiles of the static order in C (eight blocks of 32 rows per tile): the K partitions of
// those tiles add into them with TMA reduce-add.  C is 16-byte aligned with a row pitch of whole 16 bytes.
__global__ void __launch_bounds__(256) zero_tail_tiles_kernel(int32_t *__restrict__ C, int64_t ldc, int M, int N, int tail_tiles)
{
    grid_launch_dependents();  // the GEMM that follows may set itself up meanwhile; it waits for this grid before its first load
    grid_dependency_wait();    // the kernel before this one may still be writing the same C
    const int tilesP = (M + 255) / 256, tilesQ = (N + kBN - 1) / kBN;
    int tp, tq;
    tile_coords(tilesP * tilesQ - tail_tiles + (int)(blockIdx.x >> 3), tilesP, tilesQ, tp, tq);
    const int row = tp * 256 + (int)(blockIdx.x & 7) * 32 + (int)(threadIdx.x >> 3);
    if (row >= M) return;
    int32_t *dst = C + (int64_t)row * ldc;
    for (int col = tq * kBN + (int)(threadIdx.x & 7) * 4; col < (tq + 1) * kBN && col < N; col += 32) {
        if (col + 4 <= N) {
            *reinterpret_cast<int4 *>(dst + col) = make_int4(0, 0, 0, 0);
        } else {
            for (int c = col; c < N; ++c) dst[c] = 0;
        }
    }
}

template <int H, bool MC, bool DQ>
int tc2_launch_variant(const GemmArgs &g, const DeviceCtx &ctx, int split_k, bool split_tail)
{
    auto kernel = gemm_tc2_kernel<H, MC, DQ>;
    const int64_t kbytes = g.k / 2;
    CUtensorMap tmA, tmB;
    int st = make_packed_tmap(&tmA, g.A, g.m, kbytes, kRowsA, CU_TENSOR_MAP_SWIZZLE_64B);
    if (st != QM_OK) return st;
    st = make_packed_tmap(&tmB, g.B, g.n, kbytes, kRowsB, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st != QM_OK) return st;
    const int num_kb = (g.k + H * kSubK - 1) / (H * kSubK);
    if (split_k < 1 || split_k > num_kb) return QM_ERR_ARG;
    const int64_t tiles = (int64_t)((g.m + 255) / 256) * ((g.n + kBN - 1) / kBN) * split_k;
    if (tiles > 0x7FFFFFFF / 4) return QM_ERR_SHAPE;
    // TMA store of C needs a 16-byte-aligned base and row pitch; otherwise the kernel stores with plain vectors
    static const bool allow_tma_store = !std::getenv("QM_NO_TMA_STORE");
    int use_tma_store =
        (allow_tma_store && !g.plain_stores && (reinterpret_cast<uintptr_t>(g.C) & 15u) == 0 && (g.ldc & 3) == 0 && g.ldc < (1ll << 36)) ? 1 : 0;
    CUtensorMap tmC = tmA;  // placeholder when unused
    if (DQ) {
        if (split_k != 1 || !tc2_can_dequant(g)) return QM_ERR_ALIGN;
        use_tma_store = 1;
        st = make_out_bf16_tmap(&tmC, g.out_bf16, g.m, g.n, g.ldc);
        if (st != QM_OK) return st;
    } else if (use_tma_store) {
        st = make_c_tmap(&tmC, g.C, g.m, g.n, g.ldc);
        if (st != QM_OK) return st;
    }
    static const bool allow_pdl = !std::getenv("QM_NO_PDL");
    // zeroes the last `count` tiles of the static order
    auto zero_tiles = [&](int count) -> int {
        cudaLaunchConfig_t zc = {};
        zc.gridDim = dim3((unsigned)(count * 8), 1, 1);
        zc.blockDim = dim3(256, 1, 1);
        zc.stream = g.stream;
        cudaLaunchAttribute za[1];
        za[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        za[0].val.programmaticStreamSerializationAllowed = 1;
        zc.attrs = za;
        zc.numAttrs = allow_pdl ? 1 : 0;
        cudaError_t ze = cudaLaunchKernelEx(&zc, zero_tail_tiles_kernel, g.C, g.ldc, g.m, g.n, count);
        return ze == cudaSuccess ? QM_OK : record_cuda_error(ze, "zero_tail_tiles_kernel launch");
    };
    if (split_k > 1) {
        // the K partitions accumulate with TMA reduce-add: needs the TMA path and a C that starts at zero (a memset node is
        // faster here than the zeroing kernel: 256 x 4096 x 4096 15.6 against 16.9 us)
        if (!use_tma_store) return QM_ERR_ALIGN;
        cudaError_t me = cudaMemset2DAsync(g.C, (size_t)g.ldc * 4, 0, (size_t)g.n * 4, (size_t)g.m, g.stream);
        if (me != cudaSuccess) return record_cuda_error(me, "cudaMemset2DAsync(C)");
    }

    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kNumThreads, 1, 1);
    cfg.dynamicSmemBytes = Tc2Cfg<H>::kSmemBytes;
    cfg.stream = g.stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;  // the occupancy query below takes the cluster shape only
    // static tile list: every pair of the grid must be resident at once
    // per-device cache; the value is the same whichever thread computes it, so an atomic word is enough
    static std::atomic<int> max_pairs[64];
    int cached = max_pairs[ctx.device & 63].load(std::memory_order_relaxed);
    if (cached == 0) {
        cfg.gridDim = dim3((unsigned)(2 * (ctx.num_sms / 2)), 1, 1);
        int n = 0;
        cudaError_t qe = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
        if (qe != cudaSuccess) return record_cuda_error(qe, "cudaOccupancyMaxActiveClusters");
        cached = n > 0 ? n : 1;
        max_pairs[ctx.device & 63].store(cached, std::memory_order_relaxed);
    }
    int units = ctx.num_sms / 2;
    if (cached < units) units = cached;
    if (units < 1) units = 1;
    if (tiles < units) units = (int)tiles;
    // Whole tiles in rounds over the pairs leave a last round of `rest` tiles with most pairs idle.  When at least two K
    // partitions per tile of that round fit the pairs, they run as partitions that add into the zeroed tiles instead: the last
    // round then takes a fraction of a tile's main loop plus one epilogue (1024 x 10240 x 8192, 160 tiles on 74 pairs: 12 tiles
    // as 6 partitions each).
    int tail_tiles = 0, tail_split = 1;
    if (split_tail && !DQ && split_k == 1 && use_tma_store && tc2_tail_plan(tiles, units, num_kb, &tail_tiles, &tail_split)) {
        st = zero_tiles(tail_tiles);
        if (st != QM_OK) return st;
    }
    cfg.numAttrs = allow_pdl ? 2 : 1;
    cfg.gridDim = dim3((unsigned)(units * 2), 1, 1);
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, tmC, use_tma_store, g.C, g.ldc, g.m, g.n, g.k, ctx.status, split_k, tail_tiles,
                                       tail_split, g.scale_a, g.scale_b);
    if (e != cudaSuccess) return record_cuda_error(e, "gemm_tc2_kernel launch");
    return QM_OK;
}

}  // namespace

// Built variants (sub-blocks per stage, pair-wide commit).  Measured at 8192^3 on B200 before the TMA-store epilogue:
// (1, false) 442 us, (1, true) 418 us, (2, false) 337 us, (2, true) 328 us; only the fastest is compiled in.
#define QM_TC2_FOR_EACH(X) X(2, true, false) X(2, true, true)

int tc2_prepare_device()
{
    cudaError_t e;
#define X(H, MC, DQ)                                                                                                          \
    e = cudaFuncSetAttribute(gemm_tc2_kernel<H, MC, DQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, Tc2Cfg<H>::kSmemBytes); \
    if (e != cudaSuccess) return record_cuda_error(e, "cudaFuncSetAttribute(shared memory)");
    QM_TC2_FOR_EACH(X)
#undef X
    return QM_OK;
}

bool tc2_can_split(const GemmArgs &g)
{
    return !g.plain_stores && (reinterpret_cast<uintptr_t>(g.C) & 15u) == 0 && (g.ldc & 3) == 0 && !std::getenv("QM_NO_TMA_STORE");
}

int tc2_launch(const GemmArgs &g, const DeviceCtx &ctx, int split_k, bool split_tail)
{
    return tc2_launch_variant<2, true, false>(g, ctx, split_k, split_tail);
}

bool tc2_can_dequant(const GemmArgs &g)
{
    return g.out_bf16 && (reinterpret_cast<uintptr_t>(g.out_bf16) & 15u) == 0 && (g.ldc & 7) == 0 && g.ldc < (1ll << 37);
}

int tc2_launch_dequant(const GemmArgs &g, const DeviceCtx &ctx)
{
    return tc2_launch_variant<2, true, true>(g, ctx, 1, false);
}

}  // namespace qm
