// Coalesced store of an accumulator block that sits one row per lane (as tcgen05.ld 32x32b delivers it).
//
// A direct store from that register layout makes every warp store touch 32 different rows (32 separate
// 16-byte pieces), which the L1 store path serialises.  Here the warp first writes its 32 x CH block to a
// private shared-memory buffer (row pitch CH*4 + 16 bytes: conflict-free for 16-byte accesses both ways),
// then reads it back with consecutive lanes on consecutive 16-byte pieces of a row, so each global store
// instruction writes whole contiguous row segments (128 bytes per row for CH = 32).
#pragma once
#include <cuda_bf16.h>

#include "qm_ptx.cuh"

namespace qm {

template <int CH>
struct EpilogueStage {
    static constexpr int kPitch = CH * 4 + 16;         // bytes
    static constexpr int kBytesPerWarp = 32 * kPitch;  // 4608 for CH = 32
};

// v[j] = 256 * block[lane][j].  Writes block[r][c] >> 8 to C[(row0 + r) * ldc + col0 + c] for rows < M, cols < N.
template <int CH>
__device__ __forceinline__ void store_block_rows(const uint32_t (&v)[CH], uint32_t stage, int lane, int32_t *__restrict__ C,
                                                 int64_t ldc, int row0, int col0, int M, int N, bool vec_ok)
{
    constexpr int kPitch = EpilogueStage<CH>::kPitch;
    constexpr int kLanesPerRow = CH / 4;            // 16-byte pieces per row
    constexpr int kRowsPerInst = 32 / kLanesPerRow;  // rows covered by one warp-wide store
#pragma unroll
    for (int j = 0; j < CH; j += 4) {
        uint4 o;
        o.x = (uint32_t)((int32_t)v[j] >> 8);
        o.y = (uint32_t)((int32_t)v[j + 1] >> 8);
        o.z = (uint32_t)((int32_t)v[j + 2] >> 8);
        o.w = (uint32_t)((int32_t)v[j + 3] >> 8);
        ptx::sts128(stage + lane * kPitch + j * 4, o);
    }
    __syncwarp();
    const int sub = lane / kLanesPerRow, piece = lane % kLanesPerRow;
    const int q = col0 + piece * 4;
#pragma unroll
    for (int i = 0; i < 32 / kRowsPerInst; ++i) {
        const int r = i * kRowsPerInst + sub;
        const uint4 o = ptx::lds128(stage + r * kPitch + piece * 16);
        const int row = row0 + r;
        if (row < M) {
            int32_t *dst = C + (int64_t)row * ldc + q;
            if (vec_ok && q + 3 < N) {
                *reinterpret_cast<uint4 *>(dst) = o;
            } else {
                if (q < N) dst[0] = (int32_t)o.x;
                if (q + 1 < N) dst[1] = (int32_t)o.y;
                if (q + 2 < N) dst[2] = (int32_t)o.z;
                if (q + 3 < N) dst[3] = (int32_t)o.w;
            }
        }
    }
    __syncwarp();  // the buffer is rewritten by the next block
}

// The same for a whole 32 x 32 block through a 4 KB buffer without padding: 16-byte piece j of row r sits at piece j ^ (r & 7)
// (conflict-free both ways), and a warp-wide store writes four whole 128-byte row segments.  Full segments matter when C is
// in another GPU's memory: they make better NVLink packets than the 64-byte pieces of two half blocks.
__device__ __forceinline__ void store_block_rows_swizzled(const uint32_t (&v)[32], uint32_t stage, int lane, int32_t *__restrict__ C,
                                                          int64_t ldc, int row0, int col0, int M, int N, bool vec_ok)
{
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        uint4 o;
        o.x = (uint32_t)((int32_t)v[4 * j] >> 8);
        o.y = (uint32_t)((int32_t)v[4 * j + 1] >> 8);
        o.z = (uint32_t)((int32_t)v[4 * j + 2] >> 8);
        o.w = (uint32_t)((int32_t)v[4 * j + 3] >> 8);
        ptx::sts128(stage + lane * 128 + (((uint32_t)j ^ ((uint32_t)lane & 7u)) << 4), o);
    }
    __syncwarp();
    const int sub = lane >> 3, piece = lane & 7;
    const int q = col0 + piece * 4;
    int32_t *dst = C + (int64_t)(row0 + sub) * ldc + q;
    // (not unrolled: this path is not the common one, and eight row pointers in flight would cost the kernel registers)
#pragma unroll 1
    for (int i = 0; i < 8; ++i, dst += 4 * ldc) {
        const int r = i * 4 + sub;
        const uint4 o = ptx::lds128(stage + r * 128 + (((uint32_t)piece ^ ((uint32_t)r & 7u)) << 4));
        const int row = row0 + r;
        if (row < M) {
            if (vec_ok && q + 3 < N) {
                *reinterpret_cast<uint4 *>(dst) = o;
            } else {
                if (q < N) dst[0] = (int32_t)o.x;
                if (q + 1 < N) dst[1] = (int32_t)o.y;
                if (q + 2 < N) dst[2] = (int32_t)o.z;
                if (q + 3 < N) dst[3] = (int32_t)o.w;
            }
        }
    }
    __syncwarp();  // the buffer is rewritten by the next block
}

// ---- TMA-store form ---------------------------------------------------------------------------
// The warp writes its 32 x 32 int32 block into a 4 KB shared-memory buffer in the 128-byte-swizzled
// layout of the C tensor map (16-byte piece j of row r at piece j ^ (r & 7): conflict-free), and one lane
// hands the buffer to the TMA engine, which writes whole 128-byte row segments and clips at M and N.
// Two buffers per warp alternate; a buffer is reused once the store issued from it two blocks earlier has
// finished reading it.  Needs a 16-byte-aligned C and ldc % 4 == 0 (checked by the host).
constexpr int kTmaStoreBufBytes = 32 * 128;

__device__ __forceinline__ void tma_store_2d(const void *tmap, uint32_t smem_src, int32_t x, int32_t y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(x), "r"(y), "r"(smem_src)
                 : "memory");
}

// Same transfer, but the 32-bit integers are ADDED to what global memory holds (exact and order-independent for
// int32, so K partitions of a tile can accumulate into one C that starts at zero).
__device__ __forceinline__ void tma_reduce_add_2d(const void *tmap, uint32_t smem_src, int32_t x, int32_t y)
{
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(x), "r"(y), "r"(smem_src)
                 : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

template <int kPending>
__device__ __forceinline__ void tma_store_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}

__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// v[j] = 256 * block[lane][j]; `buf` is this warp's buffer for this block (1024-byte aligned);
// `first_use` is false once the buffer has been handed to the TMA engine before.
__device__ __forceinline__ void store_block_tma(const uint32_t (&v)[32], uint32_t buf, int lane, const void *tmapC, int col0,
                                                int row0, bool reuse, bool accumulate = false)
{
    if (reuse) {
        if (lane == 0) tma_store_wait_read<1>();  // at most the other buffer's store may still be reading
        __syncwarp();
    }
    const uint32_t row = buf + lane * 128;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        uint4 o;
        o.x = (uint32_t)((int32_t)v[4 * j] >> 8);
        o.y = (uint32_t)((int32_t)v[4 * j + 1] >> 8);
        o.z = (uint32_t)((int32_t)v[4 * j + 2] >> 8);
        o.w = (uint32_t)((int32_t)v[4 * j + 3] >> 8);
        ptx::sts128(row + (((uint32_t)j ^ ((uint32_t)lane & 7u)) << 4), o);
    }
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
        if (accumulate) tma_reduce_add_2d(tmapC, buf, col0, row0);
        else tma_store_2d(tmapC, buf, col0, row0);
        tma_store_commit();
    }
}

// ---- fused dequantisation --------------------------------------------------------------------
// One output element: the exact int32 sum as float (round to nearest even), times the row scale, times the column
// scale (two separate fp32 multiplications, in this order), rounded to nearest even bf16.  The CPU oracle does the same
// four steps, so the results agree bit for bit.
__device__ __forceinline__ uint32_t dequant_bf16_bits(int32_t sum, float sa, float sb)
{
    const float f = __fmul_rn(__fmul_rn(__int2float_rn(sum), sa), sb);
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}

// va / vb = 256 x two neighbouring 32 x 32 accumulator blocks (columns col0 .. col0 + 31 and col0 + 32 .. col0 + 63), one
// row per lane; `sa` = this lane's row scale; lane j of sb0 / sb1 holds the scale of column col0 + j / col0 + 32 + j.
// Writes the 32 x 64 bf16 block (128-byte rows, 128-byte-swizzled like the tensor map) and hands it to the TMA engine.
__device__ __forceinline__ void store_pair_bf16_tma(const uint32_t (&va)[32], const uint32_t (&vb)[32], uint32_t buf, int lane,
                                                    const void *tmapOut, int col0, int row0, float sa, float sb0, float sb1)
{
    const uint32_t row = buf + lane * 128;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j = (c & 3) * 8 + 2 * i;  // column inside the 32-column block
            const float s0 = __shfl_sync(0xFFFFFFFFu, c < 4 ? sb0 : sb1, j);
            const float s1 = __shfl_sync(0xFFFFFFFFu, c < 4 ? sb0 : sb1, j + 1);
            const int32_t x0 = (int32_t)(c < 4 ? va[j] : vb[j]) >> 8, x1 = (int32_t)(c < 4 ? va[j + 1] : vb[j + 1]) >> 8;
            o[i] = dequant_bf16_bits(x0, sa, s0) | (dequant_bf16_bits(x1, sa, s1) << 16);
        }
        ptx::sts128(row + (((uint32_t)c ^ ((uint32_t)lane & 7u)) << 4), make_uint4(o[0], o[1], o[2], o[3]));
    }
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
        tma_store_2d(tmapOut, buf, col0, row0);
        tma_store_commit();
    }
}

}  // namespace qm
