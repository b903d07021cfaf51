// Packed-int4 GEMM for sm_100a, large-shape form: 256 x 256 CTA-pair tile with operand A fed to the
// tensor core from TMEM instead of shared memory.
//
// Same contract as gemm_tc_kernel (exact int32 C = A * B^T on nibbles; replaces the reference's
// igemm<Config>, kernel.cu:62-266).  The difference is where the converted A lives.  The pair tile of
// gemm_tc_kernel is bound by the shared-memory data pipe: per 128-element K block each SM moves 16 KB
// of TMA writes, 16 KB of converter loads, 32 KB of converter stores and 32 KB of MMA operand reads.
// Here the four A-converter warps keep their 128 rows in registers after the s4 -> s8 split and write
// them to TMEM with tcgen05.st; tcgen05.mma takes A as [tmem] and only B as a shared-memory
// descriptor.  That removes A's 16 KB of stores and 16 KB of MMA reads per K block.
//
// TMEM map (512 columns): [0, 256) one int32 accumulator (128 lanes x 256 columns per CTA);
// [256, 256 + 32*S) a ring of S converted A stages, 128 lanes x 32 columns each (128 bytes of K per
// row: four 32-byte MMA slices, each = 16 bytes of even elements then 16 bytes of odd elements, the
// same K order the B converters produce).  With one accumulator the epilogue does not overlap the
// next tile's MMAs; the loaders and converters do run ahead during it.
//
// Warps: 0 TMA producer, 1 MMA issuer (leader CTA only) and TMEM owner, 2-5 epilogue, 6-9 A
// converters (warp & 3 = TMEM lane quarter = 32-row block), 10-17 B converters.
// Packed A tiles are loaded with the 64-byte TMA swizzle so that one thread can read its whole
// 64-byte row as four conflict-free 16-byte loads; packed B tiles are linear as in gemm_tc_kernel.
// All waits are bounded as in gemm_tc_kernel.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>

#include "qm_internal.h"
#include "qm_ptx.cuh"

namespace qm {

namespace {

using namespace ptx;

constexpr int kBN = 256;            // UMMA N of the pair tile
constexpr int kRowsA = 128;         // A rows per CTA
constexpr int kRowsB = kBN / 2;     // B rows per CTA
constexpr int kKBlock = 128;
constexpr int kPkRowBytes = 64;
constexpr int kCvRowBytes = 128;
constexpr int kS = 6;               // converted stages: B in shared memory, A in TMEM
constexpr int kSP = 6;              // packed stages
constexpr int kPkStage = (kRowsA + kRowsB) * kPkRowBytes;  // 16 KB
constexpr int kCvStage = kRowsB * kCvRowBytes;             // 16 KB
constexpr int kAccCols = kBN;
constexpr int kAStageCols = 32;
constexpr int kTmemCols = 512;
constexpr int kNumAConvWarps = 4, kNumBConvWarps = 8;
constexpr int kFirstAConvWarp = 6, kFirstBConvWarp = 10;
constexpr int kNumWarps = kFirstBConvWarp + kNumBConvWarps;  // 18
constexpr int kNumThreads = kNumWarps * 32;
constexpr int kBConvThreads = kNumBConvWarps * 32;
constexpr int kBItems = kRowsB * 4;
constexpr int kBItemIters = kBItems / kBConvThreads;  // 2
constexpr int kNumBarriers = 2 * kSP + 2 * kS + 2;
constexpr int kSmemBytes = 1024 + kS * kCvStage + kSP * kPkStage + kNumBarriers * 8 + 16;
constexpr int kRasterGroup = 8;
constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
static_assert(kAccCols + kS * kAStageCols <= kTmemCols, "TMEM budget");
static_assert(kBItems % kBConvThreads == 0, "B items");
static_assert(kSmemBytes <= 232448, "shared memory");

__device__ __forceinline__ void tile_coords2(int t, int tilesP, int tilesQ, int &tp, int &tq)
{
    const int per_group = kRasterGroup * tilesQ;
    const int g = t / per_group, rem = t - g * per_group;
    const int p0 = g * kRasterGroup;
    const int gsz = min(kRasterGroup, tilesP - p0);
    tq = rem / gsz;
    tp = p0 + (rem - tq * gsz);
}

__device__ __forceinline__ void report_timeout2(int *status, int site)
{
    if (atomicCAS(status, 0, (int)QM_ERR_TIMEOUT) == 0) status[1] = site | ((int)blockIdx.x << 8);
}

__device__ __forceinline__ uint64_t make_smem_desc2(uint32_t addr)
{
    const uint32_t lo = ((addr & 0x3FFFFu) >> 4) | (1u << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}

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

__global__ void __launch_bounds__(kNumThreads, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                int32_t *__restrict__ C, int64_t ldc, int M, int N, int K, int *status)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_u32 = smem_u32(smem_raw);
    const uint32_t cv0 = (raw_u32 + 1023u) & ~1023u;  // converted B stages
    const uint32_t pk0 = cv0 + kS * kCvStage;         // packed stages: A (swizzle 64B) then B (linear)
    const uint32_t bar0 = pk0 + kSP * kPkStage;
    auto pk_full = [&](int s) { return bar0 + 8u * s; };
    auto pk_empty = [&](int s) { return bar0 + 8u * (kSP + s); };
    auto cv_full = [&](int s) { return bar0 + 8u * (2 * kSP + s); };        // leader's copy is the one waited on
    auto cv_empty = [&](int s) { return bar0 + 8u * (2 * kSP + kS + s); };  // one per CTA
    const uint32_t acc_full = bar0 + 8u * (2 * kSP + 2 * kS);
    const uint32_t acc_empty = acc_full + 8u;
    const uint32_t tmem_slot = bar0 + 8u * kNumBarriers;
    uint32_t *tmem_slot_ptr = reinterpret_cast<uint32_t *>(smem_raw + (tmem_slot - raw_u32));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_raw + (tmem_slot + 4 - raw_u32));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta_rank = cluster_ctarank();
    const int unit = (int)(blockIdx.x >> 1), num_units = (int)(gridDim.x >> 1);
    const int tilesP = (M + 255) / 256, tilesQ = (N + kBN - 1) / kBN;
    const int num_tiles = tilesP * tilesQ;
    const int num_kb = (K + kKBlock - 1) / kKBlock;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kSP; ++s) {
            mbar_init(pk_full(s), 1);
            mbar_init(pk_empty(s), kNumAConvWarps + kNumBConvWarps);
        }
        for (int s = 0; s < kS; ++s) {
            mbar_init(cv_full(s), 2 * (kNumAConvWarps + kNumBConvWarps));
            mbar_init(cv_empty(s), 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 8);
        *abort_flag = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tmap(&tmapA);
        prefetch_tmap(&tmapB);
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
            for (int t = unit; t < num_tiles && ok; t += num_units) {
                int tp, tq;
                tile_coords2(t, tilesP, tilesQ, tp, tq);
                const int yA = tp * 256 + (int)cta_rank * kRowsA;
                const int yB = tq * kBN + (int)cta_rank * kRowsB;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kSP;
                    const uint32_t ph = (it / kSP) & 1u;
                    if (!mbar_wait(pk_empty(s), ph ^ 1u, abort_flag)) {
                        report_timeout2(status, kWaitProducerSlot);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    const uint32_t dst = pk0 + s * kPkStage;
                    mbar_arrive_expect_tx(pk_full(s), kPkStage);
                    tma_load_2d(dst, &tmapA, kb * kPkRowBytes, yA, pk_full(s));
                    tma_load_2d(dst + kRowsA * kPkRowBytes, &tmapB, kb * kPkRowBytes, yB, pk_full(s));
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
                    report_timeout2(status, kWaitMmaAcc);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after_sync();
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kS;
                    const uint32_t ph = (it / kS) & 1u;
                    if (!mbar_wait(cv_full(s), ph, abort_flag)) {
                        report_timeout2(status, kWaitMmaOperands);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint64_t dB = make_smem_desc2(cv0 + s * kCvStage);
                    const uint32_t ta = tmem_a0 + (uint32_t)(s * kAStageCols);
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4)
                        umma_i8_ta(tmem_base, ta + 8u * k4, dB + 2u * k4, kIdesc, (kb | k4) != 0 ? 1u : 0u);
                    umma_commit<2>(cv_empty(s));
                    umma_commit<2>(mapa_cluster(cv_empty(s), 1));
                }
                if (ok) {
                    umma_commit<2>(acc_full);
                    umma_commit<2>(mapa_cluster(acc_full, 1));
                }
            }
        }
        __syncwarp();
    } else if (warp < kFirstAConvWarp) {
        // ------------------------------ epilogue ------------------------------
        const int quarter = warp & 3;
        uint32_t lt = 0;
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(C) & 15u) == 0) && ((ldc & 3) == 0);
        for (int t = unit; t < num_tiles; t += num_units, ++lt) {
            int tp, tq;
            tile_coords2(t, tilesP, tilesQ, tp, tq);
            const bool ok = warp_wait<false>(acc_full, lt & 1u, abort_flag, lane);
            if (!ok) {
                if (lane == 0) {
                    report_timeout2(status, kWaitEpilogueAcc);
                    *abort_flag = 1;
                }
                break;
            }
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
            const int p = tp * 256 + (int)cta_rank * kRowsA + quarter * 32 + lane;
            const int q0 = tq * kBN;
            int32_t *crow = C + (int64_t)p * ldc + q0;
#pragma unroll 1
            for (int c = 0; c < kBN; c += 32) {
                uint32_t v[32];
                tmem_ld_x32(taddr + c, v);
                tmem_ld_wait();
                if (p < M) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const int q = q0 + c + j;
                        int4 o;
                        o.x = (int32_t)v[j] >> 8;
                        o.y = (int32_t)v[j + 1] >> 8;
                        o.z = (int32_t)v[j + 2] >> 8;
                        o.w = (int32_t)v[j + 3] >> 8;
                        if (vec_ok && q + 3 < N) {
                            *reinterpret_cast<int4 *>(crow + c + j) = o;
                        } else {
                            if (q < N) crow[c + j] = o.x;
                            if (q + 1 < N) crow[c + j + 1] = o.y;
                            if (q + 2 < N) crow[c + j + 2] = o.z;
                            if (q + 3 < N) crow[c + j + 3] = o.w;
                        }
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty, 0);
        }
    } else if (warp < kFirstBConvWarp) {
        // ------------------------------ A converters: packed smem -> registers -> TMEM ------------------------------
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;           // row of this CTA's A tile = TMEM lane
        const uint32_t swz = (uint32_t)((r >> 1) & 3);  // 64-byte TMA swizzle: chunk ^= (row / 2) % 4
        uint32_t it = 0;
        bool ok = true;
        for (int t = unit; t < num_tiles && ok; t += num_units) {
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const int ps = it % kSP, cs = it % kS;
                const uint32_t pph = (it / kSP) & 1u, cph = (it / kS) & 1u;
                if (!warp_wait<false>(pk_full(ps), pph, abort_flag, lane)) {
                    if (lane == 0) {
                        report_timeout2(status, kWaitConvertPacked);
                        *abort_flag = 1;
                    }
                    ok = false;
                    break;
                }
                const uint32_t src = pk0 + ps * kPkStage + (uint32_t)r * kPkRowBytes;
                uint4 w[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) w[c] = lds128(src + (((uint32_t)c ^ swz) << 4));
                uint32_t v[32];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    v[8 * c + 0] = (w[c].x << 4) & 0xF0F0F0F0u;
                    v[8 * c + 1] = (w[c].y << 4) & 0xF0F0F0F0u;
                    v[8 * c + 2] = (w[c].z << 4) & 0xF0F0F0F0u;
                    v[8 * c + 3] = (w[c].w << 4) & 0xF0F0F0F0u;
                    v[8 * c + 4] = w[c].x & 0xF0F0F0F0u;
                    v[8 * c + 5] = w[c].y & 0xF0F0F0F0u;
                    v[8 * c + 6] = w[c].z & 0xF0F0F0F0u;
                    v[8 * c + 7] = w[c].w & 0xF0F0F0F0u;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(pk_empty(ps));  // packed rows are in registers now
                if (!warp_wait<false>(cv_empty(cs), cph ^ 1u, abort_flag, lane)) {
                    if (lane == 0) {
                        report_timeout2(status, kWaitConvertSlot);
                        *abort_flag = 1;
                    }
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                tmem_st_x32(tmem_a0 + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(cs * kAStageCols), v);
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
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const int ps = it % kSP, cs = it % kS;
                const uint32_t pph = (it / kSP) & 1u, cph = (it / kS) & 1u;
                if (!warp_wait<false>(pk_full(ps), pph, abort_flag, lane)) {
                    if (lane == 0) {
                        report_timeout2(status, kWaitConvertPacked);
                        *abort_flag = 1;
                    }
                    ok = false;
                    break;
                }
                const uint32_t src = pk0 + ps * kPkStage + kRowsA * kPkRowBytes;
                uint4 w[kBItemIters];
#pragma unroll
                for (int j = 0; j < kBItemIters; ++j) w[j] = lds128(src + (j * kBConvThreads + ctid) * 16);
                __syncwarp();
                if (lane == 0) mbar_arrive(pk_empty(ps));
                if (!warp_wait<false>(cv_empty(cs), cph ^ 1u, abort_flag, lane)) {
                    if (lane == 0) {
                        report_timeout2(status, kWaitConvertSlot);
                        *abort_flag = 1;
                    }
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t dst = cv0 + cs * kCvStage;
#pragma unroll
                for (int j = 0; j < kBItemIters; ++j) {
                    const int i = j * kBConvThreads + ctid;
                    const int rr = i >> 2, c = i & 3;
                    const uint32_t d = dst + rr * kCvRowBytes + (((2 * c) ^ (rr & 7)) << 4);
                    uint4 lo, hi;
                    lo.x = (w[j].x << 4) & 0xF0F0F0F0u;
                    lo.y = (w[j].y << 4) & 0xF0F0F0F0u;
                    lo.z = (w[j].z << 4) & 0xF0F0F0F0u;
                    lo.w = (w[j].w << 4) & 0xF0F0F0F0u;
                    hi.x = w[j].x & 0xF0F0F0F0u;
                    hi.y = w[j].y & 0xF0F0F0F0u;
                    hi.z = w[j].z & 0xF0F0F0F0u;
                    hi.w = w[j].w & 0xF0F0F0F0u;
                    sts128(d, lo);
                    sts128(d ^ 16u, hi);
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

typedef CUresult (*EncodeTiledFn2)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn2 encode_fn2()
{
    static EncodeTiledFn2 fn = []() -> EncodeTiledFn2 {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn2>(p);
    }();
    return fn;
}

int make_tmap2(CUtensorMap *map, const void *base, int rows, int64_t kbytes, int box_rows, CUtensorMapSwizzle swizzle)
{
    EncodeTiledFn2 fn = encode_fn2();
    if (!fn) return record_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point");
    cuuint64_t dims[2] = {(cuuint64_t)kbytes, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)kbytes};
    cuuint32_t box[2] = {(cuuint32_t)kPkRowBytes, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return record_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return QM_OK;
}

}  // namespace

int tc2_prepare_device()
{
    cudaError_t e = cudaFuncSetAttribute(gemm_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    return e == cudaSuccess ? QM_OK : record_cuda_error(e, "cudaFuncSetAttribute(shared memory)");
}

int tc2_launch(const GemmArgs &g, const DeviceCtx &ctx)
{
    const int64_t kbytes = g.k / 2;
    CUtensorMap tmA, tmB;
    int st = make_tmap2(&tmA, g.A, g.m, kbytes, kRowsA, CU_TENSOR_MAP_SWIZZLE_64B);
    if (st != QM_OK) return st;
    st = make_tmap2(&tmB, g.B, g.n, kbytes, kRowsB, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st != QM_OK) return st;
    const int64_t tiles = (int64_t)((g.m + 255) / 256) * ((g.n + kBN - 1) / kBN);
    if (tiles > 0x7FFFFFFF / 4) return QM_ERR_SHAPE;

    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kNumThreads, 1, 1);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = g.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // static tile list: every pair of the grid must be resident at once
    static int max_pairs[64] = {0};
    int &cached = max_pairs[ctx.device & 63];
    if (cached == 0) {
        cfg.gridDim = dim3((unsigned)(2 * (ctx.num_sms / 2)), 1, 1);
        int n = 0;
        cudaError_t qe = cudaOccupancyMaxActiveClusters(&n, gemm_tc2_kernel, &cfg);
        if (qe != cudaSuccess) return record_cuda_error(qe, "cudaOccupancyMaxActiveClusters");
        cached = n > 0 ? n : 1;
    }
    int units = ctx.num_sms / 2;
    if (cached < units) units = cached;
    if (units < 1) units = 1;
    if (tiles < units) units = (int)tiles;
    cfg.gridDim = dim3((unsigned)(units * 2), 1, 1);
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc2_kernel, tmA, tmB, g.C, g.ldc, g.m, g.n, g.k, ctx.status);
    if (e != cudaSuccess) return record_cuda_error(e, "gemm_tc2_kernel launch");
    return QM_OK;
}

}  // namespace qm
