// Internal interfaces between the C-ABI layer (qm_api.cu) and the kernel files.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

#include "../../include/quadmul_b200.h"

namespace qm {

// Where an in-kernel bounded wait gave up (second word of the device status).
enum WaitSite : int {
    kWaitNone = 0,
    kWaitProducerSlot = 1,   // TMA producer waiting for a free packed stage
    kWaitConvertPacked = 2,  // converters waiting for TMA data
    kWaitConvertSlot = 3,    // converters waiting for a free converted stage
    kWaitMmaAcc = 4,         // MMA issuer waiting for a drained accumulator
    kWaitMmaOperands = 5,    // MMA issuer waiting for converted operands
    kWaitEpilogueAcc = 6,    // epilogue waiting for a finished accumulator
    kWaitSplitK = 7,         // split-K reducer waiting for partial tiles
    kWaitPeer = 8,           // waiting for the peer CTA of a pair
    kWaitSelfTest = 9        // qm_selftest_wait_timeout: a barrier that nothing completes
};

// Per-device state created by qm_init.
struct DeviceCtx {
    bool ready = false;
    int device = -1;
    int num_sms = 0;
    int cc_major = 0;
    int *status = nullptr;         // [2] device words: code, site
    int32_t *scratch = nullptr;    // split-K partial tiles
    size_t scratch_bytes = 0;
    int *counters = nullptr;       // split-K arrival counters (self-resetting, start at zero)
    int num_counters = 0;
};

struct GemmArgs {
    const uint8_t *A;  // M x K/2
    const uint8_t *B;  // N x K/2
    int32_t *C;        // M x ldc
    int m, n, k;
    int64_t ldc;
    cudaStream_t stream;
    bool plain_stores = false;  // write C with ordinary vector stores only (destination in another GPU's memory)
    // fused dequantisation (qm_gemm_s4_dequant_bf16): out[r][c] = bf16(float(sum) * scale_a[r] * scale_b[c]); C is unused,
    // ldc counts bf16 elements; a NULL scale vector means all ones
    void *out_bf16 = nullptr;
    const float *scale_a = nullptr;
    const float *scale_b = nullptr;
};

// Resolved tensor-path plan (see qm_tile_table.h for how it is chosen).
struct TcPlan {
    int tile_n;    // UMMA N extent: 16, 32, 64, 128, 256
    int swap_ab;   // 0: C rows on UMMA-M; 1: C columns (B rows) on UMMA-M
    int split_k;   // >= 1
    int cta_pair;  // 1 or 2
    int a_tmem;    // 1: the UMMA-M operand goes through TMEM: gemm_tc2_kernel (256 x 256 pair tile) or, with swap_ab,
                   //    gemm_dec_kernel (decode form)
    int stream_k;  // gemm_dec_kernel only: 0 = split_k partitions through scratch, 1 = one equal contiguous share of the
                   // (tile, K) work per CTA, 2 = split_k partitions as one cluster, summed through its shared memory
    int ctas_per_sm;  // gemm_dec_kernel only: 1 or 2 resident CTAs per SM (2: tile_n 16 only)
};

// qm_gemm_tc.cu
int tc_prepare_device();  // opt-in shared memory sizes for every instantiation; returns qm_status
int tc_launch(const GemmArgs &g, const TcPlan &p, const DeviceCtx &ctx);
int tc_launch_with_scratch(const GemmArgs &g, const TcPlan &p, const DeviceCtx &ctx, int32_t *scratch, size_t scratch_bytes,
                           int *counters, int num_counters);
size_t tc_scratch_bytes_needed(int m, int n, const TcPlan &p);
int tc_counters_needed(int m, int n, const TcPlan &p);

// qm_gemm_tc2.cu: 256 x 256 pair tile, A through TMEM
int tc2_prepare_device();
// split_tail: a short last round of whole tiles may run as K partitions of its tiles (tc2_tail_plan); needs tc2_can_split
int tc2_launch(const GemmArgs &g, const DeviceCtx &ctx, int split_k, bool split_tail);
bool tc2_can_split(const GemmArgs &g);  // K partitions accumulate through TMA reduce-add: needs an aligned local C
bool tc2_can_dequant(const GemmArgs &g);  // the fused bf16 epilogue stores with TMA only: aligned out, ldc % 8 == 0
int tc2_launch_dequant(const GemmArgs &g, const DeviceCtx &ctx);

// qm_dequant.cu: out[r][c] = bf16(float(acc[r][c]) * scale_a[r] * scale_b[c]) for an int32 matrix already in memory
int dequant_launch(const int32_t *acc, int64_t ld_acc, const float *scale_a, const float *scale_b, void *out_bf16, int64_t ldc,
                   int m, int n, cudaStream_t s);

// qm_gemm_dec.cu: decode form (swap_ab, tile_n 16/32/64), B rows through TMEM; split-K through the context's scratch
int dec_prepare_device();
// clusters of `size` (2..4) CTAs of the decode kernel's cluster form that `device` runs at once; 0 = the driver did not say
int dec_cluster_capacity(int device, int tile_n, int size);
int dec_launch(const GemmArgs &g, const TcPlan &p, const DeviceCtx &ctx);

// qm_gemv.cu: one to four rows of A, weight streaming with dp4a (no tensor cores); int32 or fused bf16 output
constexpr int kGemvMaxRows = 4;
constexpr size_t kGemvMaxSmemBytes = 200 * 1024;  // converted rows of A held by a CTA
// Shape limits of the row kernel (the table decides among the eligible kernel families in qm_tile_table.h).
inline bool gemv_shape_limits(int m, int k)
{
    if (m < 1 || m > kGemvMaxRows || k % 32 != 0 || k >= 131072) return false;
    return (size_t)(m <= 1 ? 1 : (m <= 2 ? 2 : 4)) * (size_t)k <= kGemvMaxSmemBytes;
}
bool gemv_eligible(const GemmArgs &g);  // shape limits of the kernel itself (any n) and 16-byte-aligned A and B
int gemv_launch(const GemmArgs &g, const DeviceCtx &ctx);

// qm_gemm_rmma.cu: up to 16 rows of A on small weight matrices; weights straight into registers, mma.sync s8
constexpr int kRmmaMaxK = 8192;  // 16 converted rows of A (16 * K bytes) + 32 KB of partial tiles fit in shared memory
constexpr int kRmmaMaxRows = 64;       // rows of A, in tiles of 16 that pass through shared memory one after the other
constexpr int kRmmaMaxKTiled = 4096;   // ... which needs a block's weights resident in registers (16 warps x 2 steps x 128 elements)
// Shape limits of the kernel (the table decides among the eligible kernel families in qm_tile_table.h).
inline bool rmma_shape_limits(int m, int k)
{
    return m >= 1 && m <= kRmmaMaxRows && k % 32 == 0 && k <= (m <= 16 ? kRmmaMaxK : kRmmaMaxKTiled);
}
// offline weight layout for this kernel (optional): every warp-wide load reads 512 consecutive bytes, a warp's 4 KB and a
// CTA's 64 KB per round contiguous; rows padded to 32, K to 4096 elements
size_t prelayout_bytes(int n, int k);
int prelayout_launch(const uint8_t *B, uint8_t *Bp, int n, int k, cudaStream_t s);
int rmma_launch_prelaid(const GemmArgs &g, const DeviceCtx &ctx);  // g.B = the pre-laid-out form
bool rmma_eligible(const GemmArgs &g);  // limits of the kernel itself (m <= 16, k <= kRmmaMaxK, any n) and 16-byte-aligned A and B
int rmma_launch(const GemmArgs &g, const DeviceCtx &ctx);

// qm_gemm_simt.cu
int simt_launch(const GemmArgs &g);

// qm_pack.cu
int pack_launch(const int8_t *in, uint8_t *out, int64_t rows, int64_t k, cudaStream_t s);
int unpack_launch(const uint8_t *in, int8_t *out, int64_t rows, int64_t k, cudaStream_t s);
int fill_launch(uint8_t *out, int64_t rows, int64_t k, uint64_t seed, cudaStream_t s);
int unshard_launch(const int32_t *slabs, int32_t *C, int m, int n, int world, int64_t slab_stride, cudaStream_t s);

// qm_peer_flags.cu: completion flags between GPUs (fused gather)
int flag_signal_launch(int *flag, int value, cudaStream_t s);
int flags_wait_launch(const int *flags, int count, int value, int timeout_ms, int *status, cudaStream_t s);

// qm_api.cu
// Column split of n over `world` ranks: whole units of 128 columns where n allows, the last ranks
// take the remainder units.
void nshard_range(int n, int world, int rank, int *begin, int *count);
int record_cuda_error(cudaError_t e, const char *what);  // returns QM_ERR_CUDA, stores the text

}  // namespace qm
