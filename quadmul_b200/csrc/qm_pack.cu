// HBM-bound byte kernels around the GEMM: pack (int8 -> nibbles), unpack (nibbles -> int8),
// the counter-based fill used by the benchmark, and the un-interleave of gathered C slabs.
//
// pack   follows the reference's Python packer  (test.py:6-15): byte j = (x[2j] & 15) | (x[2j+1] << 4).
// unpack follows the reference's host function  (kernel.cu:387-408): low nibble first, x > 7 -> x - 16.
//
// Every warp access is a whole contiguous run (pack: 512 B in, 256 B out per instruction; unpack: 256 B in,
// 512 B out), several loads are in flight per thread, grids are a multiple of the SM count and grid-stride
// over the rest.  Algorithmic traffic is 1.5 bytes per element.
#include "qm_internal.h"

namespace qm {

namespace {

constexpr int kThreads = 256;
// Measured on B200 (16384 x 16384 elements): unroll 2 with 32 CTAs per SM gave 5.7 TB/s for both directions,
// within 4 % of a device-to-device copy of the same size; unroll 4 / 8 CTAs per SM was 2-5 % slower.
#ifndef QM_PACK_UNROLL
#define QM_PACK_UNROLL 2
#endif
#ifndef QM_PACK_CTAS_PER_SM
#define QM_PACK_CTAS_PER_SM 32
#endif
constexpr int kUnroll = QM_PACK_UNROLL;
constexpr int kMaxWorld = 16;

__device__ __forceinline__ uint32_t pack8(uint32_t w0, uint32_t w1)
{
    // w holds 4 int8 values e0 o0 e1 o1 (little endian). Keep the low nibble of each byte, fold
    // each odd byte onto the even byte below it, then gather the even bytes of both words.
    uint32_t n0 = w0 & 0x0F0F0F0Fu, n1 = w1 & 0x0F0F0F0Fu;
    n0 |= n0 >> 4;
    n1 |= n1 >> 4;
    return __byte_perm(n0, n1, 0x6420);
}

__device__ __forceinline__ uint32_t sext_nibbles(uint32_t n)
{
    // n: one 4-bit value in the low half of each byte. Adding 30x the sign bit (8 -> 0xF0) sets
    // the upper four bits of negative values; bytes do not interact because 0xF0 + 0x0F < 256.
    return (n & 0x08080808u) * 30u + n;
}

__device__ __forceinline__ void unpack8(uint32_t w, uint32_t &o0, uint32_t &o1)
{
    uint32_t e = sext_nibbles(w & 0x0F0F0F0Fu);         // elements 0,2,4,6
    uint32_t o = sext_nibbles((w >> 4) & 0x0F0F0F0Fu);  // elements 1,3,5,7
    o0 = __byte_perm(e, o, 0x5140);                     // e0 o0 e1 o1
    o1 = __byte_perm(e, o, 0x7362);                     // e2 o2 e3 o3
}

// in: total_in bytes (int8), out: total_in / 2 bytes.  Vector body, scalar tail.
__global__ void __launch_bounds__(kThreads) pack_kernel(const int8_t *__restrict__ in, uint8_t *__restrict__ out,
                                                        int64_t total_in, int vec_ok)
{
    const int64_t nvec = vec_ok ? total_in / 16 : 0;  // 16 input bytes -> 8 output bytes
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const uint4 *vin = reinterpret_cast<const uint4 *>(in);
    uint2 *vout = reinterpret_cast<uint2 *>(out);
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < nvec; i += stride * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
            if (i + u * stride < nvec) v[u] = __ldcs(vin + i + u * stride);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
            if (i + u * stride < nvec) {
                uint2 r;
                r.x = pack8(v[u].x, v[u].y);
                r.y = pack8(v[u].z, v[u].w);
                __stcs(vout + i + u * stride, r);
            }
    }
    // tail (or everything, when the pointers are not vector-aligned): one output byte per thread
    for (int64_t j = nvec * 8 + (int64_t)blockIdx.x * kThreads + threadIdx.x; j < total_in / 2; j += stride) {
        unsigned e = (unsigned)in[2 * j] & 15u, o = (unsigned)in[2 * j + 1] & 15u;
        out[j] = (uint8_t)(e | (o << 4));
    }
}

// in: total_packed bytes, out: 2 * total_packed bytes (int8).  A thread turns 8 packed bytes into 16 output bytes,
// so consecutive lanes read consecutive 8-byte pieces and write consecutive 16-byte pieces: both sides of every
// warp access are whole contiguous runs (256 B in, 512 B out).
__global__ void __launch_bounds__(kThreads) unpack_kernel(const uint8_t *__restrict__ in, int8_t *__restrict__ out,
                                                          int64_t total_packed, int vec_ok)
{
    constexpr int kU = 2 * kUnroll;
    const int64_t nvec = vec_ok ? total_packed / 8 : 0;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const uint2 *vin = reinterpret_cast<const uint2 *>(in);
    uint4 *vout = reinterpret_cast<uint4 *>(out);
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < nvec; i += stride * kU) {
        uint2 v[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u)
            if (i + u * stride < nvec) v[u] = __ldcs(vin + i + u * stride);
#pragma unroll
        for (int u = 0; u < kU; ++u)
            if (i + u * stride < nvec) {
                uint4 a;
                unpack8(v[u].x, a.x, a.y);
                unpack8(v[u].y, a.z, a.w);
                __stcs(vout + i + u * stride, a);
            }
    }
    for (int64_t j = nvec * 8 + (int64_t)blockIdx.x * kThreads + threadIdx.x; j < total_packed; j += stride) {
        int lo = in[j] & 15, hi = in[j] >> 4;
        out[2 * j] = (int8_t)(lo > 7 ? lo - 16 : lo);
        out[2 * j + 1] = (int8_t)(hi > 7 ? hi - 16 : hi);
    }
}

__device__ __forceinline__ uint64_t mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Element e (flat index row * k + col) has value ((mix64(seed + e) >> 33) & 15) - 8; its nibble is
// that value modulo 16.  One thread writes 4 packed bytes (8 elements).
__global__ void __launch_bounds__(kThreads) fill_kernel(uint8_t *__restrict__ out, int64_t total_packed, uint64_t seed)
{
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const int64_t nwords = total_packed / 4;
    for (int64_t w = (int64_t)blockIdx.x * kThreads + threadIdx.x; w < nwords; w += stride) {
        uint32_t word = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            uint32_t u = (uint32_t)(mix64(seed + (uint64_t)(w * 8 + e)) >> 33) & 15u;
            word |= ((u + 8u) & 15u) << (4 * e);
        }
        reinterpret_cast<uint32_t *>(out)[w] = word;
    }
    for (int64_t j = nwords * 4 + (int64_t)blockIdx.x * kThreads + threadIdx.x; j < total_packed; j += stride) {
        uint32_t e = (uint32_t)(mix64(seed + (uint64_t)(2 * j)) >> 33) & 15u;
        uint32_t o = (uint32_t)(mix64(seed + (uint64_t)(2 * j + 1)) >> 33) & 15u;
        out[j] = (uint8_t)(((e + 8u) & 15u) | (((o + 8u) & 15u) << 4));
    }
}

// slabs[g][row][slab_stride] holds rank g's columns; C[row][begin_g + c] = slabs[g][row][c].
struct ShardTable {
    int begin[kMaxWorld + 1];  // begin[g] .. begin[g + 1] are rank g's columns
};

__global__ void __launch_bounds__(kThreads) unshard_kernel(const int32_t *__restrict__ slabs, int32_t *__restrict__ C,
                                                           int m, int n, int world, int64_t slab_stride, ShardTable t)
{
    const int64_t total = (int64_t)m * n;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride) {
        const int row = (int)(i / n), col = (int)(i % n);
        int g = 0;
        while (g + 1 < world && col >= t.begin[g + 1]) ++g;
        C[i] = slabs[((int64_t)g * m + row) * slab_stride + (col - t.begin[g])];
    }
}

int grid_for(int64_t work_items, int num_sms_hint)
{
    int64_t blocks = (work_items + kThreads - 1) / kThreads;
    int64_t cap = (int64_t)num_sms_hint * QM_PACK_CTAS_PER_SM;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

int sm_count()
{
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms > 0 ? sms : 148;
}

}  // namespace

int pack_launch(const int8_t *in, uint8_t *out, int64_t rows, int64_t k, cudaStream_t s)
{
    const int64_t total_in = rows * k;
    if (total_in == 0) return QM_OK;
    const int vec_ok = ((reinterpret_cast<uintptr_t>(in) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 7u) == 0);
    pack_kernel<<<grid_for(total_in / 16 / kUnroll + 1, sm_count()), kThreads, 0, s>>>(in, out, total_in, vec_ok);
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? QM_OK : record_cuda_error(e, "pack_kernel launch");
}

int unpack_launch(const uint8_t *in, int8_t *out, int64_t rows, int64_t k, cudaStream_t s)
{
    const int64_t total_packed = rows * (k / 2);
    if (total_packed == 0) return QM_OK;
    const int vec_ok = ((reinterpret_cast<uintptr_t>(in) & 7u) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0);
    unpack_kernel<<<grid_for(total_packed / 8 / (2 * kUnroll) + 1, sm_count()), kThreads, 0, s>>>(in, out, total_packed, vec_ok);
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? QM_OK : record_cuda_error(e, "unpack_kernel launch");
}

int fill_launch(uint8_t *out, int64_t rows, int64_t k, uint64_t seed, cudaStream_t s)
{
    const int64_t total_packed = rows * (k / 2);
    if (total_packed == 0) return QM_OK;
    if (reinterpret_cast<uintptr_t>(out) & 3u) return QM_ERR_ALIGN;
    fill_kernel<<<grid_for(total_packed / 4 + 1, sm_count()), kThreads, 0, s>>>(out, total_packed, seed);
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? QM_OK : record_cuda_error(e, "fill_kernel launch");
}

int unshard_launch(const int32_t *slabs, int32_t *C, int m, int n, int world, int64_t slab_stride, cudaStream_t s)
{
    const int64_t total = (int64_t)m * n;
    if (total == 0) return QM_OK;
    if (world < 1 || world > kMaxWorld) return QM_ERR_ARG;
    ShardTable t;
    for (int g = 0; g < world; ++g) {
        int count = 0;
        nshard_range(n, world, g, &t.begin[g], &count);
        t.begin[g + 1] = t.begin[g] + count;
    }
    unshard_kernel<<<grid_for(total, sm_count()), kThreads, 0, s>>>(slabs, C, m, n, world, slab_stride, t);
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? QM_OK : record_cuda_error(e, "unshard_kernel launch");
}

}  // namespace qm
