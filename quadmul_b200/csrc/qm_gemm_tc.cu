// Packed-int4 GEMM for sm_100a:  TMA -> packed ring -> s4->s8 converters -> tcgen05.mma kind::i8 -> TMEM -> C.
//
// Replaces the reference's WMMA s4 kernel `igemm<Config>` (kernel.cu:62-266) and its launcher
// (kernel.cu:268-289).  The arithmetic contract is the same, exact int32 C = A * B^T on nibbles;
// the structure is not a port:
//
//  * One persistent CTA per SM (or one CTA pair per two SMs) walks a static list of output tiles.
//  * Warp 0, one lane: TMA producer.  cp.async.bulk.tensor.2d copies PACKED rows (64 bytes = 128
//    nibbles of K per row) of both operands into a ring of `SP` packed stages; completion is
//    counted in bytes on an mbarrier.  Rows or K bytes outside the matrix are zero-filled by TMA,
//    so ragged M, N and a K tail need no padding (nibble 0 is the value 0).
//  * Warps 6..13: converters.  tcgen05 has no 4-bit integer MMA, so every 16-byte packed chunk
//    w (32 nibbles) becomes two 16-byte int8 chunks, (w << 4) & 0xF0F0F0F0 (the even elements
//    times 16) and w & 0xF0F0F0F0 (the odd elements times 16), written into a ring of `SC`
//    converted stages in the K-major SWIZZLE_128B layout the MMA reads.  Both operands are
//    permuted along K in the same way, which leaves every dot product unchanged.
//  * Warp 1, one lane: issues tcgen05.mma.kind::i8 (M = 128 or 256, N = BN, K = 32 per
//    instruction) from shared-memory descriptors into one of two TMEM accumulators, and
//    tcgen05.commit hands converted stages back and publishes finished accumulators.
//  * Warps 2..5: epilogue.  tcgen05.ld 32 lanes x 32 columns, arithmetic shift by 8 (the two
//    factors of 16), vectorised global stores; runs under the next tile's main loop.
//
// The accumulator holds 256 x the true sum: |sum| <= 64 K, so K < 131072 keeps it inside int32.
//
// Every mbarrier wait is bounded; on expiry the CTA records QM_ERR_TIMEOUT and the wait site in
// the device status word, raises a CTA-wide abort flag, and all roles fall through to the common
// teardown (TMEM is always freed).
#include <cuda.h>

#include <atomic>

#include <cstdio>
#include <cstdlib>

#include "qm_epilogue.cuh"
#include "qm_internal.h"
#include "qm_ptx.cuh"
#include "qm_tc_common.cuh"

namespace qm {

namespace {

using namespace ptx;
using namespace tc;

constexpr int kNumConvWarps = 8;
constexpr int kFirstEpiWarp = 2;
constexpr int kFirstConvWarp = 6;
constexpr int kNumWarps = kFirstConvWarp + kNumConvWarps;
constexpr int kNumThreads = kNumWarps * 32;
constexpr int kConvThreads = kNumConvWarps * 32;
constexpr int kKBlock = 128;            // K elements per stage
constexpr int kPkRowBytes = kKBlock / 2;  // 64
constexpr int kCvRowBytes = kKBlock;      // 128
constexpr int kStageBudget = 200 * 1024;

constexpr int next_pow2(int x)
{
    int p = 32;
    while (p < x) p *= 2;
    return p;
}

template <int BN, bool SWAP, int G>
struct TcCfg {
    static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N");
    static_assert(G == 1 || (G == 2 && BN % 32 == 0), "pair MMA needs N % 32 == 0");
    static constexpr int kRowsP = 128;     // rows of the UMMA-M operand held by this CTA
    static constexpr int kRowsQ = BN / G;  // rows of the UMMA-N operand held by this CTA
    static constexpr int kRows = kRowsP + kRowsQ;
    // A pipeline stage holds H sub-blocks of 128 K-elements.  The decode form pays a fixed hand-off chain per stage
    // (converter arrive, one thread issuing the MMAs and the commit), so it takes two sub-blocks per stage; the
    // wide tiles keep one (their stages already fill the shared memory).
    static constexpr int H = SWAP ? 2 : 1;
    static constexpr int kPkSub = kRows * kPkRowBytes;
    static constexpr int kCvSub = kRows * kCvRowBytes;
    static constexpr int kPkStage = H * kPkSub;
    static constexpr int kCvStage = H * kCvSub;
    static constexpr int SC = (3 * kCvStage + 4 * kPkStage <= kStageBudget) ? 3 : 2;
    static constexpr int SP_raw = (kStageBudget - SC * kCvStage) / kPkStage;
    static constexpr int SP = SP_raw > 8 ? 8 : SP_raw;
    static constexpr int kTmemCols = next_pow2(2 * BN);
    static constexpr int kNumBarriers = 2 * SP + 2 * SC + 4;
    static constexpr int kEpiChunk = BN >= 32 ? 32 : 16;  // columns per TMEM load in the row-major epilogue
    static constexpr int kEpiBytes = SWAP ? 0 : 4 * EpilogueStage<kEpiChunk>::kBytesPerWarp;
    static constexpr int kSmemBytes = 1024 + SC * kCvStage + SP * kPkStage + kEpiBytes + kNumBarriers * 8 + 16;
    static constexpr int kItems = kRows * 4;  // 16-byte packed chunks per stage
    static constexpr int kItemIters = (kItems + kConvThreads - 1) / kConvThreads;
    static constexpr uint32_t kIdesc = (2u << 4)                      // D format: s32
                                       | (1u << 7)                    // A format: signed 8-bit
                                       | (1u << 10)                   // B format: signed 8-bit
                                       | ((uint32_t)(BN >> 3) << 17)  // N
                                       | ((uint32_t)((128 * G) >> 4) << 24);  // M
    static_assert(kSmemBytes <= 232448, "shared memory");
    static_assert(kPkStage % 1024 == 0 && kCvStage % 1024 == 0, "stage alignment");
};

template <int BN, bool SWAP, int G>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmapP, const __grid_constant__ CUtensorMap tmapQ,
               int32_t *__restrict__ C, int64_t ldc, int rowsP, int rowsQ, int K, int *status, int split_k,
               int32_t *__restrict__ scratch, int *__restrict__ counters)
{
    using Cfg = TcCfg<BN, SWAP, G>;
    constexpr int SP = Cfg::SP, SC = Cfg::SC;
    extern __shared__ uint8_t smem_raw[];

    const uint32_t raw_u32 = smem_u32(smem_raw);
    const uint32_t cv0 = (raw_u32 + 1023u) & ~1023u;
    const uint32_t pk0 = cv0 + SC * Cfg::kCvStage;
    const uint32_t epi0 = pk0 + SP * Cfg::kPkStage;  // per-warp transpose buffers of the row-major epilogue
    const uint32_t bar0 = epi0 + Cfg::kEpiBytes;
    auto pk_full = [&](int s) { return bar0 + 8u * s; };
    auto pk_empty = [&](int s) { return bar0 + 8u * (SP + s); };
    auto cv_full = [&](int s) { return bar0 + 8u * (2 * SP + s); };
    auto cv_empty = [&](int s) { return bar0 + 8u * (2 * SP + SC + s); };
    auto acc_full = [&](int b) { return bar0 + 8u * (2 * SP + 2 * SC + b); };
    auto acc_empty = [&](int b) { return bar0 + 8u * (2 * SP + 2 * SC + 2 + b); };
    const uint32_t tmem_slot = bar0 + 8u * Cfg::kNumBarriers;
    uint32_t *tmem_slot_ptr = reinterpret_cast<uint32_t *>(smem_raw + (tmem_slot - raw_u32));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_raw + (tmem_slot + 4 - raw_u32));

    // Decode-sized launches are dominated by fixed costs, so they chain: the next launch in the stream may start
    // its own set-up (barriers, TMEM, tensor-map fetch) while this one still runs, and touches global memory only
    // after grid_dependency_wait() below.
    if constexpr (SWAP) grid_launch_dependents();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta_rank = (G == 2) ? cluster_ctarank() : 0u;
    const int unit = (G == 2) ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;      // CTA or CTA pair
    const int num_units = (G == 2) ? (int)(gridDim.x >> 1) : (int)gridDim.x;

    const int tilesP = (rowsP + 128 * G - 1) / (128 * G);
    const int tilesQ = (rowsQ + BN - 1) / BN;
    const int num_kb_total = (K + Cfg::H * kKBlock - 1) / (Cfg::H * kKBlock);  // stages; TMA zero-fills beyond K
    // A work item is one K partition of one output tile; partitions of a tile are adjacent items.
    const int num_tiles = tilesP * tilesQ * split_k;
    auto kb_begin = [&](int item) { return (int)(((long long)(item % split_k) * num_kb_total) / split_k); };
    auto kb_end = [&](int item) { return (int)(((long long)(item % split_k + 1) * num_kb_total) / split_k); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < SP; ++s) {
            mbar_init(pk_full(s), 1);
            mbar_init(pk_empty(s), kNumConvWarps);
        }
        for (int s = 0; s < SC; ++s) {
            mbar_init(cv_full(s), kNumConvWarps * G);
            mbar_init(cv_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 4 * G);
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
        tmem_alloc<G>(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish<G>();
    }
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (G == 2) {
        cluster_arrive();
        cluster_wait();
    }
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;
    if constexpr (SWAP) grid_dependency_wait();  // everything before this line touched no global memory

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = unit; t < num_tiles && ok; t += num_units) {
                int tp, tq;
                tile_coords(t / split_k, tilesP, tilesQ, tp, tq);
                const int yP = tp * 128 * G + (int)cta_rank * 128;
                const int yQ = tq * BN + (int)cta_rank * Cfg::kRowsQ;
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
                    for (int h = 0; h < Cfg::H; ++h) {
                        const int x = (kb * Cfg::H + h) * kPkRowBytes;
                        tma_load_2d(dst + h * Cfg::kPkSub, &tmapP, x, yP, pk_full(s));
                        tma_load_2d(dst + h * Cfg::kPkSub + Cfg::kRowsP * kPkRowBytes, &tmapQ, x, yQ, pk_full(s));
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0 && cta_rank == 0) {
            uint32_t it = 0, lt = 0;
            bool ok = true;
            for (int t = unit; t < num_tiles && ok; t += num_units, ++lt) {
                const int buf = lt & 1;
                const uint32_t bph = (lt >> 1) & 1u;
                if (!(G == 2 ? mbar_spin_wait(acc_empty(buf), bph ^ 1u, abort_flag)
                             : mbar_wait(acc_empty(buf), bph ^ 1u, abort_flag))) {
                    report_timeout(status, kWaitMmaAcc);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                const int kb0 = kb_begin(t);
                for (int kb = kb0, kbe = kb_end(t); kb < kbe; ++kb, ++it) {
                    const int s = it % SC;
                    const uint32_t ph = (it / SC) & 1u;
                    if (!(G == 2 ? mbar_spin_wait(cv_full(s), ph, abort_flag) : mbar_wait(cv_full(s), ph, abort_flag))) {
                        report_timeout(status, kWaitMmaOperands);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
#pragma unroll
                    for (int h = 0; h < Cfg::H; ++h) {
                        const uint32_t sub = cv0 + s * Cfg::kCvStage + h * Cfg::kCvSub;
                        const uint64_t dP = make_smem_desc(sub);
                        const uint64_t dQ = make_smem_desc(sub + Cfg::kRowsP * kCvRowBytes);
#pragma unroll
                        for (int k4 = 0; k4 < kKBlock / 32; ++k4) {
                            // +32 bytes of K inside the 128-byte swizzled row = +2 in the address field
                            umma_i8<G>(tmem_d, dP + 2u * k4, dQ + 2u * k4, Cfg::kIdesc,
                                       (kb != kb0 || (h | k4) != 0) ? 1u : 0u);
                        }
                    }
                    umma_commit<G>(cv_empty(s));
                    if constexpr (G == 2) umma_commit<G>(mapa_cluster(cv_empty(s), 1));
                }
                if (ok) {
                    umma_commit<G>(acc_full(buf));
                    if constexpr (G == 2) umma_commit<G>(mapa_cluster(acc_full(buf), 1));
                }
            }
        }
        __syncwarp();
    } else if (warp < kFirstConvWarp) {
        // ------------------------------ epilogue ------------------------------
        const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are the ones this warp may read
        uint32_t lt = 0;
        for (int t = unit; t < num_tiles; t += num_units, ++lt) {
            int tp, tq;
            tile_coords(t / split_k, tilesP, tilesQ, tp, tq);
            const int buf = lt & 1;
            const uint32_t bph = (lt >> 1) & 1u;
            const bool ok = warp_wait<G == 2>(acc_full(buf), bph, abort_flag, lane);
            if (!ok) {
                if (lane == 0) {
                    report_timeout(status, kWaitEpilogueAcc);
                    *abort_flag = 1;
                }
                break;
            }
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN);
            const int p = tp * 128 * G + (int)cta_rank * 128 + quarter * 32 + lane;  // index along the UMMA-M operand
            const int q0 = tq * BN;
            if (split_k > 1) {
                // Partial tile -> scratch as [column][row] (coalesced), then whichever K partition of the
                // tile finishes last sums all of them.  Nobody waits: an arrival counter decides who reduces.
                const int tile = t / split_k;
                const int row = quarter * 32 + lane;
                int32_t *mine = scratch + (int64_t)t * (128 * BN);
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    uint32_t v[16];
                    tmem_ld_x16(taddr + c, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) __stcg(mine + (c + j) * 128 + row, (int32_t)v[j] >> 8);
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty(buf));  // the accumulator is drained; split-K runs single-CTA
                // Each warp owns 32 rows of the tile and its own counter, so no warp waits for another.
                __threadfence();
                __syncwarp();
                int last = 0;
                if (lane == 0) {
                    int *ctr = counters + tile * 4 + quarter;
                    last = (atomicAdd(ctr, 1) == split_k - 1) ? 1 : 0;
                    if (last) *ctr = 0;  // ready for the next launch
                }
                last = __shfl_sync(0xFFFFFFFFu, last, 0);
                if (last) {
                    __threadfence();
                    const int32_t *parts = scratch + (int64_t)tile * split_k * (128 * BN);
#pragma unroll 1
                    for (int c = 0; c < BN; c += 16) {
                        int32_t sum[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) sum[j] = 0;
                        for (int sk = 0; sk < split_k; ++sk) {
                            const int32_t *src = parts + (int64_t)sk * (128 * BN) + c * 128 + row;
#pragma unroll
                            for (int j = 0; j < 16; ++j) sum[j] += __ldcg(src + j * 128);
                        }
                        if (p < rowsP) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int q = q0 + c + j;
                                if (q < rowsQ) {
                                    if constexpr (SWAP) C[(int64_t)q * ldc + p] = sum[j];
                                    else C[(int64_t)p * ldc + q] = sum[j];
                                }
                            }
                        }
                    }
                }
                continue;
            }
            if constexpr (!SWAP) {
                // C[p][q0 + j]: the block arrives one row per lane and leaves as whole row segments.
                const bool vec_ok = ((reinterpret_cast<uintptr_t>(C) & 15u) == 0) && ((ldc & 3) == 0);
                constexpr int CH = Cfg::kEpiChunk;
                const uint32_t stage = epi0 + (uint32_t)((warp - kFirstEpiWarp) * EpilogueStage<CH>::kBytesPerWarp);
                const int row0 = p - lane;
#pragma unroll 1
                for (int c = 0; c < BN; c += CH) {
                    uint32_t v[CH];
                    if constexpr (CH == 32) tmem_ld_x32(taddr + c, v);
                    else tmem_ld_x16(taddr + c, v);
                    tmem_ld_wait();
                    store_block_rows<CH>(v, stage, lane, C, ldc, row0, q0 + c, rowsP, rowsQ, vec_ok);
                }
            } else {
                // C[q0 + j][p]: lanes hold consecutive p, so each column is one coalesced 128-byte store.
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    uint32_t v[16];
                    tmem_ld_x16(taddr + c, v);
                    tmem_ld_wait();
                    if (p < rowsP) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int q = q0 + c + j;
                            if (q < rowsQ) C[(int64_t)q * ldc + p] = (int32_t)v[j] >> 8;
                        }
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if constexpr (G == 2) mbar_arrive_cluster(acc_empty(buf), 0);
                else mbar_arrive(acc_empty(buf));
            }
        }
    } else {
        // ------------------------------ converters ------------------------------
        const int ctid = threadIdx.x - kFirstConvWarp * 32;
        uint32_t it = 0;
        bool ok = true;
        for (int t = unit; t < num_tiles && ok; t += num_units) {
            for (int kb = kb_begin(t), kbe = kb_end(t); kb < kbe; ++kb, ++it) {
                const int ps = it % SP, cs = it % SC;
                const uint32_t pph = (it / SP) & 1u, cph = (it / SC) & 1u;
                const bool w1 = warp_wait<false>(pk_full(ps), pph, abort_flag, lane);
                if (!w1) {
                    if (lane == 0) {
                        report_timeout(status, kWaitConvertPacked);
                        *abort_flag = 1;
                    }
                    ok = false;
                    break;
                }
                const bool w2 = warp_wait<G == 2>(cv_empty(cs), cph ^ 1u, abort_flag, lane);
                if (!w2) {
                    if (lane == 0) {
                        report_timeout(status, kWaitConvertSlot);
                        *abort_flag = 1;
                    }
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
#pragma unroll
                for (int h = 0; h < Cfg::H; ++h) {
                    const uint32_t src = pk0 + ps * Cfg::kPkStage + h * Cfg::kPkSub;
                    const uint32_t dst = cv0 + cs * Cfg::kCvStage + h * Cfg::kCvSub;
                    uint4 w[Cfg::kItemIters];
#pragma unroll
                    for (int j = 0; j < Cfg::kItemIters; ++j) {
                        const int i = j * kConvThreads + ctid;
                        if (Cfg::kItems % kConvThreads == 0 || i < Cfg::kItems) w[j] = lds128(src + i * 16);
                    }
#pragma unroll
                    for (int j = 0; j < Cfg::kItemIters; ++j) {
                        const int i = j * kConvThreads + ctid;
                        if (Cfg::kItems % kConvThreads == 0 || i < Cfg::kItems) convert_chunk_to_smem(dst, i >> 2, i & 3, w[j]);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(pk_empty(ps));
                    if constexpr (G == 2) mbar_arrive_cluster(cv_full(cs), 0);
                    else mbar_arrive(cv_full(cs));
                }
            }
        }
    }

    // ------------------------------ teardown ------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (G == 2) {
        // the peer may still be signalling this CTA's barriers or reading its shared memory
        cluster_arrive();
        cluster_wait();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<G>(tmem_base, Cfg::kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
template <int BN, bool SWAP, int G>
int prepare_one()
{
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, SWAP, G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         TcCfg<BN, SWAP, G>::kSmemBytes);
    if (e != cudaSuccess) return record_cuda_error(e, "cudaFuncSetAttribute(shared memory)");
    return QM_OK;
}

template <int BN, bool SWAP, int G>
int launch_one(const GemmArgs &g, const DeviceCtx &ctx, int split_k, int32_t *scratch, size_t scratch_bytes, int *counters,
               int num_counters)
{
    using Cfg = TcCfg<BN, SWAP, G>;
    const uint8_t *P = SWAP ? g.B : g.A;
    const uint8_t *Q = SWAP ? g.A : g.B;
    const int rowsP = SWAP ? g.n : g.m;
    const int rowsQ = SWAP ? g.m : g.n;
    const int64_t kbytes = g.k / 2;
    CUtensorMap tmP, tmQ;
    int st = make_packed_tmap(&tmP, P, rowsP, kbytes, Cfg::kRowsP, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st != QM_OK) return st;
    st = make_packed_tmap(&tmQ, Q, rowsQ, kbytes, Cfg::kRowsQ, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st != QM_OK) return st;

    const int tilesP = (rowsP + 128 * G - 1) / (128 * G);
    const int tilesQ = (rowsQ + BN - 1) / BN;
    const int num_kb = (g.k + Cfg::H * kKBlock - 1) / (Cfg::H * kKBlock);  // stages
    if (split_k < 1 || split_k > num_kb || (split_k > 1 && G != 1)) return QM_ERR_ARG;
    const int64_t tiles = (int64_t)tilesP * tilesQ * split_k;
    if (tiles > 0x7FFFFFFF / 4) return QM_ERR_SHAPE;
    if (split_k > 1) {
        if ((size_t)tiles * 128 * BN * sizeof(int32_t) > scratch_bytes || (int64_t)tilesP * tilesQ * 4 > num_counters)
            return QM_ERR_WORKSPACE;
        if (!scratch || !counters) return QM_ERR_NULL;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kNumThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = g.stream;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    if (G == 2) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.numAttrs = 1;
    }
    static const bool allow_pdl = !std::getenv("QM_NO_PDL");
    if (SWAP && allow_pdl) {
        // may begin while the previous kernel of the stream drains; the kernel itself waits before global accesses
        attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
        ++cfg.numAttrs;
    }
    // The tile list is static, so every CTA (pair) of the grid must be resident at once: a pair that
    // only starts when another has finished would run its whole share of tiles alone.
    int units = ctx.num_sms / G;
    if (G == 2) {
        // per-device cache; the value is the same whichever thread computes it, so an atomic word is enough
        static std::atomic<int> max_pairs[64];
        int cached = max_pairs[ctx.device & 63].load(std::memory_order_relaxed);
        if (cached == 0) {
            cfg.gridDim = dim3((unsigned)(2 * (ctx.num_sms / 2)), 1, 1);
            int n = 0;
            cudaError_t qe = cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel<BN, SWAP, G>, &cfg);
            if (qe != cudaSuccess) return record_cuda_error(qe, "cudaOccupancyMaxActiveClusters");
            cached = n > 0 ? n : 1;
            max_pairs[ctx.device & 63].store(cached, std::memory_order_relaxed);
            if (std::getenv("QM_LOG"))
                std::fprintf(stderr, "quadmul_b200: tile_n=%d pair kernel: %d CTA pairs resident at once (%d SMs)\n", BN,
                             cached, ctx.num_sms);
        }
        if (cached < units) units = cached;
    }
    if (units < 1) units = 1;
    if (tiles < units) units = (int)tiles;
    cfg.gridDim = dim3((unsigned)(units * G), 1, 1);
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, SWAP, G>, tmP, tmQ, g.C, g.ldc, rowsP, rowsQ, g.k,
                                       ctx.status, split_k, scratch, counters);
    if (e != cudaSuccess) return record_cuda_error(e, "gemm_tc_kernel launch");
    return QM_OK;
}

}  // namespace

#define QM_TC_FOR_EACH(X) \
    X(16, false, 1)       \
    X(32, false, 1)       \
    X(64, false, 1)       \
    X(128, false, 1)      \
    X(256, false, 1)      \
    X(16, true, 1)        \
    X(32, true, 1)        \
    X(64, true, 1)        \
    X(128, true, 1)       \
    X(128, false, 2)      \
    X(256, false, 2)

int tc_prepare_device()
{
    int st;
#define X(BN, SW, G)                \
    st = prepare_one<BN, SW, G>(); \
    if (st != QM_OK) return st;
    QM_TC_FOR_EACH(X)
#undef X
    return QM_OK;
}

int tc_launch(const GemmArgs &g, const TcPlan &p, const DeviceCtx &ctx)
{
    return tc_launch_with_scratch(g, p, ctx, ctx.scratch, ctx.scratch_bytes, ctx.counters, ctx.num_counters);
}

int tc_launch_with_scratch(const GemmArgs &g, const TcPlan &p, const DeviceCtx &ctx, int32_t *scratch, size_t scratch_bytes,
                           int *counters, int num_counters)
{
#define X(BN, SW, G)                                                               \
    if (p.tile_n == BN && (p.swap_ab != 0) == SW && p.cta_pair == G)               \
        return launch_one<BN, SW, G>(g, ctx, p.split_k, scratch, scratch_bytes, counters, num_counters);
    QM_TC_FOR_EACH(X)
#undef X
    return QM_ERR_ARG;
}

// Scratch a split-K launch needs: one 128 x tile_n int32 partial per (tile, K partition), one counter per tile.
size_t tc_scratch_bytes_needed(int m, int n, const TcPlan &p)
{
    if (p.split_k <= 1) return 0;
    const int rowsP = p.swap_ab ? n : m, rowsQ = p.swap_ab ? m : n;
    const int64_t tiles = (int64_t)((rowsP + 127) / 128) * ((rowsQ + p.tile_n - 1) / p.tile_n);
    return (size_t)tiles * p.split_k * 128 * p.tile_n * sizeof(int32_t);
}

int tc_counters_needed(int m, int n, const TcPlan &p)
{
    if (p.split_k <= 1) return 0;
    const int rowsP = p.swap_ab ? n : m, rowsQ = p.swap_ab ? m : n;
    return 4 * ((rowsP + 127) / 128) * ((rowsQ + p.tile_n - 1) / p.tile_n);  // one per 32-row quarter of a tile
}

}  // namespace qm
