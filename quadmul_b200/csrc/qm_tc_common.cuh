// Pieces shared by the two tensor-core GEMM kernels (qm_gemm_tc.cu, qm_gemm_tc2.cu): the static tile order,
// the time-out report, the UMMA shared-memory descriptor, the s4 -> s8 split and the TMA tensor maps.
#pragma once
#include <cuda.h>

#include "qm_internal.h"
#include "qm_ptx.cuh"

namespace qm {
namespace tc {

constexpr int kRasterGroup = 8;

// Static tile order: groups of kRasterGroup P-tiles, P fastest inside a group, so the tiles in flight at one
// time share operand rows in L2.
__device__ __forceinline__ void tile_coords(int t, int tilesP, int tilesQ, int &tp, int &tq)
{
    const int per_group = kRasterGroup * tilesQ;
    const int g = t / per_group, rem = t - g * per_group;
    const int p0 = g * kRasterGroup;
    const int gsz = min(kRasterGroup, tilesP - p0);
    tq = rem / gsz;
    tp = p0 + (rem - tq * gsz);
}

// First expiry wins: status[0] = QM_ERR_TIMEOUT, status[1] = wait site | block index << 8.
__device__ __forceinline__ void report_timeout(int *status, int site)
{
    if (atomicCAS(status, 0, (int)QM_ERR_TIMEOUT) == 0) status[1] = site | ((int)blockIdx.x << 8);
}

// K-major operand tile: 128-byte rows, 8-row groups 1024 bytes apart, SWIZZLE_128B, descriptor version 1.
// Advancing by 32 bytes of K inside the swizzled row is +2 in the address field.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr)
{
    const uint32_t lo = ((addr & 0x3FFFFu) >> 4) | (1u << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}

// 32 nibbles -> the 16 even elements times 16 (lo) and the 16 odd elements times 16 (hi), each as int8.
__device__ __forceinline__ void split_s4x32(const uint4 &w, uint4 &lo, uint4 &hi)
{
    lo.x = (w.x << 4) & 0xF0F0F0F0u;
    lo.y = (w.y << 4) & 0xF0F0F0F0u;
    lo.z = (w.z << 4) & 0xF0F0F0F0u;
    lo.w = (w.w << 4) & 0xF0F0F0F0u;
    hi.x = w.x & 0xF0F0F0F0u;
    hi.y = w.y & 0xF0F0F0F0u;
    hi.z = w.z & 0xF0F0F0F0u;
    hi.w = w.w & 0xF0F0F0F0u;
}

// One packed 16-byte chunk (row r, chunk c of a 64-byte packed row) into a converted K-major SWIZZLE_128B tile:
// 16-byte pieces 2c (even elements) and 2c + 1 (odd elements) of row r, piece index XOR (r & 7).
__device__ __forceinline__ void convert_chunk_to_smem(uint32_t tile, int r, int c, const uint4 &w)
{
    uint4 lo, hi;
    split_s4x32(w, lo, hi);
    const uint32_t d = tile + r * 128 + (((2 * c) ^ (r & 7)) << 4);
    ptx::sts128(d, lo);
    ptx::sts128(d ^ 16u, hi);
}

// ---- host: tensor maps ---------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Packed matrix [rows][kbytes] of bytes; box = 64 bytes x box_rows; zero fill outside the matrix.
inline int make_packed_tmap(CUtensorMap *map, const void *base, int rows, int64_t kbytes, int box_rows, CUtensorMapSwizzle swizzle)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return record_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point");
    cuuint64_t dims[2] = {(cuuint64_t)kbytes, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)kbytes};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return record_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return QM_OK;
}

// C as a 2-D int32 tensor [m][n] with row pitch ldc; 32 x 32 boxes, 128-byte swizzle (for TMA stores).
inline int make_c_tmap(CUtensorMap *map, const int32_t *C, int m, int n, int64_t ldc)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return record_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point");
    cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)m};
    cuuint64_t strides[1] = {(cuuint64_t)ldc * 4};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<int32_t *>(C), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return record_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(C)");
    return QM_OK;
}

// The bf16 output of the fused dequantising epilogue as a 2-D tensor [m][n] with row pitch ldc; 64 x 32 boxes (128-byte
// rows), 128-byte swizzle.
inline int make_out_bf16_tmap(CUtensorMap *map, const void *out, int m, int n, int64_t ldc)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return record_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point");
    cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)m};
    cuuint64_t strides[1] = {(cuuint64_t)ldc * 2};
    cuuint32_t box[2] = {64, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(out), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return record_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled(bf16 out)");
    return QM_OK;
}

}  // namespace tc
}  // namespace qm
