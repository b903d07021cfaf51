// C ABI of the library (include/quadmul_b200.h): argument checks, per-device set-up, dispatch.
// This layer stands where the reference has `wrapper` (kernel.cu:334-385) and the pybind
// function `gemm` (extension.cpp:8-24).
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include "qm_internal.h"
#include "qm_tc_common.cuh"
#include "qm_tile_table.h"

namespace qm {

namespace {

constexpr int kMaxDevices = 64;
// Split-K scratch of a device: kNumSlices independent slices of partial-tile memory and arrival counters.  Every stream
// that launches a kernel with scratch gets a slice of its own (first come, first served), so launches that overlap on
// the GPU from different streams never share partial tiles or counters; launches in one stream are ordered anyway.
constexpr int kNumSlices = 6;
constexpr size_t kSliceBytes = 32u << 20;  // partial tiles per slice
constexpr int kSliceCounters = 8192;       // arrival counters / share flags per slice
DeviceCtx g_ctx[kMaxDevices];
std::atomic<bool> g_ctx_ready[kMaxDevices];  // release-stored after g_ctx[dev] is complete, acquire-loaded on the fast path
std::atomic<uintptr_t> g_slice_key[kMaxDevices][kNumSlices];  // which stream owns a slice (0 = free)
std::mutex g_mutex;
thread_local std::string t_last_error;

constexpr int kHostSlabs = 8;   // row slabs whose result copy overlaps the next slab's upload and GEMM
constexpr int kHostBParts = 4;  // blocks of B rows the first slab takes one by one, so that the first download starts early
struct HostStage {             // grow-only device buffers, copy stream and events of qm_gemm_s4_host
    void *a = nullptr, *b = nullptr, *c = nullptr;
    size_t a_bytes = 0, b_bytes = 0, c_bytes = 0;
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t slab_done[kHostSlabs + kHostBParts] = {};
    bool streams_ready = false;
};
HostStage g_stage[kMaxDevices];

int ensure_ctx(DeviceCtx **out)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e, "cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return QM_ERR_ARG;
    DeviceCtx &c = g_ctx[dev];
    if (!g_ctx_ready[dev].load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!g_ctx_ready[dev].load(std::memory_order_relaxed)) {
            int major = 0, sms = 0;
            if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess)
                return record_cuda_error(e, "cudaDeviceGetAttribute");
            if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess)
                return record_cuda_error(e, "cudaDeviceGetAttribute");
            if (major != 10) return QM_ERR_ARCH;
            int *status = nullptr;
            if ((e = cudaMalloc(&status, 2 * sizeof(int))) != cudaSuccess) return record_cuda_error(e, "cudaMalloc(status)");
            if ((e = cudaMemset(status, 0, 2 * sizeof(int))) != cudaSuccess) return record_cuda_error(e, "cudaMemset(status)");
            int st = tc_prepare_device();
            if (st == QM_OK) st = tc2_prepare_device();
            if (st == QM_OK) st = dec_prepare_device();
            if (st != QM_OK) {
                cudaFree(status);
                return st;
            }
            // split-K scratch: partial tiles and self-resetting arrival counters (zero between launches)
            void *scratch = nullptr, *counters = nullptr;
            if ((e = cudaMalloc(&scratch, kNumSlices * kSliceBytes)) == cudaSuccess &&
                (e = cudaMalloc(&counters, (size_t)kNumSlices * kSliceCounters * sizeof(int))) == cudaSuccess)
                e = cudaMemset(counters, 0, (size_t)kNumSlices * kSliceCounters * sizeof(int));
            if (e != cudaSuccess) {
                cudaFree(status);
                cudaFree(scratch);
                cudaFree(counters);
                return record_cuda_error(e, "cudaMalloc/cudaMemset(split-K scratch)");
            }
            c.scratch = static_cast<int32_t *>(scratch);
            c.scratch_bytes = kSliceBytes;
            c.counters = static_cast<int *>(counters);
            c.num_counters = kSliceCounters;
            c.device = dev;
            c.cc_major = major;
            c.num_sms = sms;
            c.status = status;
            c.ready = true;
            g_ctx_ready[dev].store(true, std::memory_order_release);
        }
    }
    *out = &c;
    return QM_OK;
}

// The scratch slice of `stream` on this device: -1 when every slice already belongs to another stream (the caller then
// runs a form that needs no scratch).  The legacy default stream is one key whether it is passed as NULL or by its handle;
// the per-thread default stream is a different stream in every host thread, so its key is the thread.
uintptr_t stream_key(cudaStream_t stream)
{
    static thread_local char t_thread_tag;
    if (stream == nullptr) return reinterpret_cast<uintptr_t>(cudaStreamLegacy);
    if (stream == cudaStreamPerThread) return reinterpret_cast<uintptr_t>(&t_thread_tag);
    return reinterpret_cast<uintptr_t>(stream);
}

int slice_of_stream(int dev, cudaStream_t stream)
{
    const uintptr_t key = stream_key(stream);
    std::atomic<uintptr_t> *keys = g_slice_key[dev];
    for (int i = 0; i < kNumSlices; ++i) {
        uintptr_t cur = keys[i].load(std::memory_order_acquire);
        if (cur == key) return i;
        if (cur == 0) {
            if (keys[i].compare_exchange_strong(cur, key, std::memory_order_acq_rel)) return i;
            if (cur == key) return i;
        }
    }
    return -1;
}

// A copy of the device context whose scratch and counters are the slice of `stream` (none: empty scratch).
DeviceCtx ctx_for_stream(const DeviceCtx &c, cudaStream_t stream)
{
    DeviceCtx lc = c;
    const int slice = slice_of_stream(c.device, stream);
    if (slice < 0) {
        lc.scratch = nullptr, lc.scratch_bytes = 0, lc.counters = nullptr, lc.num_counters = 0;
    } else {
        lc.scratch = c.scratch + (size_t)slice * (kSliceBytes / sizeof(int32_t));
        lc.counters = c.counters + (size_t)slice * kSliceCounters;
    }
    return lc;
}

int check_gemm_args(const void *A, const void *B, void *C, int m, int n, int k, int64_t ldc)
{
    if (m < 0 || n < 0 || k < 0 || (k & 1)) return QM_ERR_SHAPE;
    if (m == 0 || n == 0) return QM_OK;
    if (!C) return QM_ERR_NULL;
    if (ldc < n) return QM_ERR_SHAPE;
    if (k > 0 && (!A || !B)) return QM_ERR_NULL;
    return QM_OK;
}

int gemm_dispatch(const void *A, const void *B, void *C, int m, int n, int k, int64_t ldc, void *stream,
                  const qm_gemm_opts_t *opts)
{
    int st = check_gemm_args(A, B, C, m, n, k, ldc);
    if (st != QM_OK) return st;
    if (m == 0 || n == 0) return QM_OK;
    DeviceCtx *ctx = nullptr;
    st = ensure_ctx(&ctx);
    if (st != QM_OK) return st;
    GemmArgs g{static_cast<const uint8_t *>(A), static_cast<const uint8_t *>(B), static_cast<int32_t *>(C), m, n, k, ldc,
               static_cast<cudaStream_t>(stream)};
    g.plain_stores = opts && opts->plain_stores != 0;
    if (k == 0) {  // empty sum: C = 0
        cudaError_t e = cudaMemset2DAsync(C, (size_t)ldc * 4, 0, (size_t)n * 4, (size_t)m, g.stream);
        return e == cudaSuccess ? QM_OK : record_cuda_error(e, "cudaMemset2DAsync");
    }
    int kernel = opts ? opts->kernel : QM_KERNEL_AUTO;
    if (kernel < QM_KERNEL_AUTO || kernel > QM_KERNEL_RMMA) return QM_ERR_ARG;
    if (kernel == QM_KERNEL_RMMA) return rmma_eligible(g) ? rmma_launch(g, *ctx) : ((m > kRmmaMaxRows || k > (m <= 16 ? kRmmaMaxK : kRmmaMaxKTiled)) ? QM_ERR_ARG : QM_ERR_ALIGN);
    const bool eligible = tc_eligible(g);
    if (kernel == QM_KERNEL_TC && !eligible) return QM_ERR_ALIGN;
    if (kernel == QM_KERNEL_GEMV && !gemv_eligible(g)) return m > kGemvMaxRows ? QM_ERR_ARG : QM_ERR_ALIGN;
    // decode shapes: the generated table (swept shapes, else the cost model) picks among the families that can take the call
    if (kernel == QM_KERNEL_AUTO && m <= kRmmaMaxRows) {
        const bool ok[3] = {rmma_eligible(g), gemv_eligible(g), eligible};
        const int fam = choose_decode_family(m, n, k, ctx->num_sms, ok);
        if (fam == kFamRmma) return rmma_launch(g, *ctx);
        if (fam == kFamGemv) kernel = QM_KERNEL_GEMV;
    }
    if (kernel == QM_KERNEL_AUTO) kernel = eligible ? QM_KERNEL_TC : QM_KERNEL_SIMT;
    if (kernel == QM_KERNEL_SIMT) return simt_launch(g);
    if (kernel == QM_KERNEL_GEMV) return gemv_launch(g, *ctx);

    TcPlan p = plan_tc(m, n, k, ctx->num_sms);
    if (opts) {
        if (opts->swap_ab < 0 || opts->swap_ab > 2 || opts->split_k < 0 || opts->cta_pair < 0 || opts->cta_pair > 2 ||
            opts->tile_n < 0)
            return QM_ERR_ARG;
        // the table's K split belongs to the table's tile form: an explicit form starts unsplit
        if (opts->swap_ab || opts->tile_n || opts->cta_pair || opts->a_tmem) p.split_k = 1;
        if (opts->swap_ab) p.swap_ab = opts->swap_ab - 1;
        if (opts->tile_n) p.tile_n = opts->tile_n;
        if (opts->split_k) p.split_k = opts->split_k;
        if (opts->cta_pair) p.cta_pair = opts->cta_pair;
        if (opts->a_tmem < 0 || opts->a_tmem > 2) return QM_ERR_ARG;
        if (opts->a_tmem) p.a_tmem = opts->a_tmem - 1;
        else if (opts->swap_ab || opts->tile_n || opts->cta_pair) p.a_tmem = 0;
        if (opts->stream_k < 0 || opts->stream_k > 3) return QM_ERR_ARG;
        if (opts->stream_k) p.stream_k = opts->stream_k - 1;
        else if (opts->swap_ab || opts->tile_n || opts->cta_pair || opts->a_tmem || opts->split_k) p.stream_k = 0;
        // the decode kernel has all three forms; the large-shape kernel takes 2 as "cut a short last round of tiles into K partitions"
        if (p.stream_k && !(p.a_tmem && p.swap_ab) && !(p.a_tmem && !p.swap_ab && p.stream_k == 1)) return QM_ERR_ARG;
        if (opts->ctas_per_sm < 0 || opts->ctas_per_sm > 2) return QM_ERR_ARG;
        if (opts->ctas_per_sm) p.ctas_per_sm = opts->ctas_per_sm;
        else if (opts->swap_ab || opts->tile_n || opts->cta_pair || opts->a_tmem || opts->split_k || opts->stream_k) p.ctas_per_sm = 1;
        if (p.ctas_per_sm == 2 && !(p.a_tmem && p.swap_ab && p.tile_n == 16)) return QM_ERR_ARG;
    }
    // Scratch (partial tiles, arrival counters, share flags) comes from the slice of this call's stream; a form that
    // needs none does not claim a slice.  With every slice taken by other streams the scratch is empty and the table's
    // choice falls back to a form without it, below.
    const bool is_dec = p.a_tmem && p.swap_ab;
    const bool wants_scratch = is_dec ? ((p.split_k > 1 && p.stream_k != 2) || p.stream_k == 1) : (!p.a_tmem && p.split_k > 1);
    DeviceCtx lc = *ctx;
    if (wants_scratch) lc = ctx_for_stream(*ctx, g.stream);
    else lc.scratch = nullptr, lc.scratch_bytes = 0, lc.counters = nullptr, lc.num_counters = 0;
    const bool through_scratch = (p.swap_ab || !p.a_tmem) && !(p.swap_ab && p.a_tmem && p.stream_k == 2);
    if (p.split_k > 1 && !(opts && opts->split_k) && through_scratch &&
        (tc_scratch_bytes_needed(m, n, p) > lc.scratch_bytes || tc_counters_needed(m, n, p) > lc.num_counters))
        p.split_k = 1;  // the table's choice does not fit the scratch: run unsplit rather than fail
    if (is_dec && p.stream_k == 2 && !(opts && (opts->split_k || opts->stream_k))) {
        // the table sized the cluster for a typical device; this device may hold fewer clusters of that size at once
        const int tiles = ((n + 127) / 128) * ((m + p.tile_n - 1) / p.tile_n);
        for (int cap; p.split_k >= 2 && (cap = dec_cluster_capacity(ctx->device, p.tile_n, p.split_k)) > 0 && tiles > cap;) --p.split_k;
    }
    if (p.stream_k == 2 && p.split_k < 2) p.stream_k = 0, p.split_k = 1;  // a cluster of one partition is the plain form
    if (is_dec) {
        if ((p.tile_n != 16 && p.tile_n != 32 && p.tile_n != 64) || p.cta_pair != 1) return QM_ERR_ARG;
        st = dec_launch(g, p, lc);
        if (st == QM_ERR_WORKSPACE && p.stream_k && !(opts && opts->stream_k)) {
            p.stream_k = 0, p.split_k = 1;  // the table's choice does not fit the scratch: run unsplit rather than fail
            st = dec_launch(g, p, lc);
        }
        return st;
    }
    if (p.a_tmem) {
        if (p.tile_n != 256 || p.cta_pair != 2) return QM_ERR_ARG;
        if (p.split_k > 1 && !tc2_can_split(g)) {
            if (opts && opts->split_k) return QM_ERR_ALIGN;
            p.split_k = 1;
        }
        static const bool allow_tail = !std::getenv("QM_TC2_NO_TAIL");
        return tc2_launch(g, lc, p.split_k, allow_tail && p.stream_k == 1 && p.split_k == 1 && tc2_can_split(g));
    }
    return tc_launch(g, p, lc);
}

}  // namespace

int record_cuda_error(cudaError_t e, const char *what)
{
    t_last_error = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
    return QM_ERR_CUDA;
}

void nshard_range(int n, int world, int rank, int *begin, int *count)
{
    const int unit = (n % 128 == 0 && n / 128 >= world) ? 128 : 1;
    const int units = n / unit, base = units / world, extra = units % world;
    const int first_big = world - extra;  // ranks >= first_big carry one more unit
    const int my_units = base + (rank >= first_big ? 1 : 0);
    const int my_begin_units = rank * base + (rank > first_big ? rank - first_big : 0);
    *begin = my_begin_units * unit;
    *count = my_units * unit;
}

}  // namespace qm

using namespace qm;

// The time-out path of the GEMM kernels in isolation: one warp waits, with the same bounded whole-warp wait the kernels use,
// on an mbarrier that nothing ever completes; the wait gives up after its limit and records QM_ERR_TIMEOUT / kWaitSelfTest.
static __global__ void wait_timeout_kernel(int *status)
{
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        abort_flag = 0;
        ptx::fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const bool ok = ptx::warp_wait<false>(ptx::smem_u32(&bar), 0u, &abort_flag, (int)threadIdx.x);
        if (!ok && threadIdx.x == 0) tc::report_timeout(status, kWaitSelfTest);
    }
}

extern "C" {

const char *qm_status_string(int status)
{
    switch (status) {
        case QM_OK: return "QM_OK";
        case QM_ERR_NULL: return "QM_ERR_NULL: a required pointer is NULL";
        case QM_ERR_SHAPE: return "QM_ERR_SHAPE: m, n, k must be non-negative, k even, ldc >= n";
        case QM_ERR_ALIGN: return "QM_ERR_ALIGN: operand alignment not supported by the requested kernel";
        case QM_ERR_CUDA: return "QM_ERR_CUDA: a CUDA call failed (see qm_last_cuda_error)";
        case QM_ERR_TIMEOUT: return "QM_ERR_TIMEOUT: a bounded in-kernel wait expired";
        case QM_ERR_ARCH: return "QM_ERR_ARCH: the current device is not compute capability 10.x";
        case QM_ERR_WORKSPACE: return "QM_ERR_WORKSPACE: scratch memory too small";
        case QM_ERR_ARG: return "QM_ERR_ARG: option out of range";
        default: return "QM_ERR_UNKNOWN";
    }
}

int qm_version(void) { return 101; }

const char *qm_last_cuda_error(void) { return t_last_error.c_str(); }

int qm_init(int device)
{
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return record_cuda_error(e, "cudaGetDevice");
    if (device != prev && (e = cudaSetDevice(device)) != cudaSuccess) return record_cuda_error(e, "cudaSetDevice");
    DeviceCtx *ctx = nullptr;
    int st = ensure_ctx(&ctx);
    if (device != prev) cudaSetDevice(prev);
    return st;
}

int qm_gemm_s4(const void *A, const void *B, void *C, int m, int n, int k, void *stream)
{
    return gemm_dispatch(A, B, C, m, n, k, n, stream, nullptr);
}

int qm_gemm_s4_ex(const void *A, const void *B, void *C, int m, int n, int k, void *stream, const qm_gemm_opts_t *opts)
{
    return gemm_dispatch(A, B, C, m, n, k, n, stream, opts);
}

int qm_gemm_s4_ldc(const void *A, const void *B, void *C, int m, int n, int k, int64_t ldc, void *stream)
{
    return gemm_dispatch(A, B, C, m, n, k, ldc, stream, nullptr);
}

int qm_gemm_s4_ldc_ex(const void *A, const void *B, void *C, int m, int n, int k, int64_t ldc, void *stream,
                      const qm_gemm_opts_t *opts)
{
    return gemm_dispatch(A, B, C, m, n, k, ldc, stream, opts);
}

int qm_gemm_s4_dequant_bf16(const void *A, const void *B, const float *scale_a, const float *scale_b, void *out_bf16, int m, int n,
                            int k, int64_t ldc, void *workspace, size_t workspace_bytes, void *stream)
{
    int st = check_gemm_args(A, B, out_bf16, m, n, k, ldc);
    if (st != QM_OK) return st;
    if (m == 0 || n == 0) return QM_OK;
    DeviceCtx *ctx = nullptr;
    st = ensure_ctx(&ctx);
    if (st != QM_OK) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (k > 0) {
        GemmArgs g{static_cast<const uint8_t *>(A), static_cast<const uint8_t *>(B), nullptr, m, n, k, ldc, s};
        g.out_bf16 = out_bf16, g.scale_a = scale_a, g.scale_b = scale_b;
        const TcPlan p = plan_tc(m, n, k, ctx->num_sms);
        // fused: the large-shape, the decode and the dp4a row kernel convert inside their epilogues and never write the int32 matrix
        if (m <= kRmmaMaxRows) {
            const bool ok[3] = {rmma_eligible(g), gemv_eligible(g), tc_eligible(g)};
            const int fam = choose_decode_family(m, n, k, ctx->num_sms, ok);
            if (fam == kFamRmma) return rmma_launch(g, *ctx);
            if (fam == kFamGemv) return gemv_launch(g, *ctx);
        }
        if (tc_eligible(g) && p.a_tmem && !p.swap_ab && tc2_can_dequant(g)) return tc2_launch_dequant(g, *ctx);
        if (tc_eligible(g) && p.a_tmem && p.swap_ab) {
            TcPlan q = p;
            const DeviceCtx lc = ctx_for_stream(*ctx, s);  // scratch slice of this call's stream
            if (q.split_k > 1 && q.stream_k != 2 &&
                (tc_scratch_bytes_needed(m, n, q) > lc.scratch_bytes || tc_counters_needed(m, n, q) > lc.num_counters))
                q.split_k = 1;
            st = dec_launch(g, q, lc);
            if (st == QM_ERR_WORKSPACE && q.stream_k == 1) {
                q.stream_k = 0, q.split_k = 1;
                st = dec_launch(g, q, lc);
            }
            return st;
        }
    }
    // composed: int32 product into the caller's workspace, then one element-wise pass
    const size_t need = (size_t)m * (size_t)n * sizeof(int32_t);
    if (!workspace || workspace_bytes < need) return QM_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 3u) != 0) return QM_ERR_ALIGN;
    st = gemm_dispatch(A, B, workspace, m, n, k, n, stream, nullptr);
    if (st != QM_OK) return st;
    return dequant_launch(static_cast<const int32_t *>(workspace), n, scale_a, scale_b, out_bf16, ldc, m, n, s);
}

size_t qm_gemm_s4_dequant_workspace_bytes(int m, int n, int k, int64_t ldc, const void *out_bf16)
{
    if (m <= 0 || n <= 0 || k < 0) return 0;
    if (k > 0 && k % 32 == 0 && k < 131072) {
        GemmArgs g{nullptr, nullptr, nullptr, m, n, k, ldc, nullptr};
        g.out_bf16 = out_bf16 ? const_cast<void *>(out_bf16) : reinterpret_cast<void *>(uintptr_t(16));  // NULL: assume aligned
        const TcPlan p = plan_tc(m, n, k, 148);
        // the operands are assumed 16-byte aligned here; an unaligned A or B takes the composed path and needs the workspace
        if (p.a_tmem && !p.swap_ab && tc2_can_dequant(g)) return 0;
        if (p.a_tmem && p.swap_ab) return 0;  // decode kernel (and the dp4a row kernel below it): any alignment of out
    }
    return (size_t)m * (size_t)n * sizeof(int32_t);
}

int qm_selftest_wait_timeout(void *stream)
{
    DeviceCtx *ctx = nullptr;
    int st = ensure_ctx(&ctx);
    if (st != QM_OK) return st;
    wait_timeout_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(ctx->status);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? QM_OK : record_cuda_error(e, "wait_timeout_kernel launch");
}

int qm_gemm_s4_host(const void *hA, const void *hB, void *hC, int m, int n, int k)
{
    int st = check_gemm_args(hA, hB, hC, m, n, k, n);
    if (st != QM_OK) return st;
    if (m == 0 || n == 0) return QM_OK;
    DeviceCtx *ctx = nullptr;
    st = ensure_ctx(&ctx);
    if (st != QM_OK) return st;
    const size_t a_bytes = (size_t)m * (k / 2), b_bytes = (size_t)n * (k / 2), c_bytes = (size_t)m * n * 4;
    std::lock_guard<std::mutex> lock(g_mutex);
    HostStage &s = g_stage[ctx->device];
    auto grow = [](void *&p, size_t &have, size_t need) -> cudaError_t {
        if (need <= have) return cudaSuccess;
        if (p) cudaFree(p);
        p = nullptr;
        have = 0;
        cudaError_t e = cudaMalloc(&p, need);
        if (e == cudaSuccess) have = need;
        return e;
    };
    cudaError_t e;
    if ((e = grow(s.a, s.a_bytes, a_bytes ? a_bytes : 16)) != cudaSuccess) return record_cuda_error(e, "cudaMalloc(A)");
    if ((e = grow(s.b, s.b_bytes, b_bytes ? b_bytes : 16)) != cudaSuccess) return record_cuda_error(e, "cudaMalloc(B)");
    if ((e = grow(s.c, s.c_bytes, c_bytes)) != cudaSuccess) return record_cuda_error(e, "cudaMalloc(C)");
    cudaStream_t stream = cudaStreamPerThread;
    // Large results: cut C into row slabs and copy slab i back on a second stream while slab i+1 is uploaded and
    // computed, so the two PCIe directions and the GEMM overlap.  Small ones: one upload, one GEMM, one download.
    const int slabs = (c_bytes >= (32u << 20) && m >= 256 * kHostSlabs) ? kHostSlabs : 1;
    if (slabs > 1 && !s.streams_ready) {
        if ((e = cudaStreamCreateWithFlags(&s.copy_stream, cudaStreamNonBlocking)) != cudaSuccess)
            return record_cuda_error(e, "cudaStreamCreate");
        for (int i = 0; i < kHostSlabs + kHostBParts; ++i)
            if ((e = cudaEventCreateWithFlags(&s.slab_done[i], cudaEventDisableTiming)) != cudaSuccess)
                return record_cuda_error(e, "cudaEventCreate");
        s.streams_ready = true;
    }
    const int rows_per_slab = slabs > 1 ? ((m / slabs + 255) / 256) * 256 : m;
    const size_t row_a = (size_t)(k / 2), row_c = (size_t)n * 4;
    // The result (4 bytes per output) is what the bus spends its time on, so the first download should start as early as
    // possible: the first row slab does not wait for all of B but takes it in kHostBParts blocks of rows, each followed by
    // the product for those columns of C and their download, while the next block of B is still on its way up.
    const int b_parts = (slabs > 1 && n >= 256 * kHostBParts) ? kHostBParts : 1;
    const int cols_per_part = b_parts > 1 ? ((n / b_parts + 255) / 256) * 256 : n;
    if (b_parts == 1 && b_bytes && (e = cudaMemcpyAsync(s.b, hB, b_bytes, cudaMemcpyHostToDevice, stream)) != cudaSuccess)
        return record_cuda_error(e, "cudaMemcpyAsync(B)");
    for (int i = 0, r0 = 0; r0 < m; ++i, r0 += rows_per_slab) {
        const int rows = (m - r0 < rows_per_slab) ? m - r0 : rows_per_slab;
        char *dA = static_cast<char *>(s.a) + (size_t)r0 * row_a;
        char *dC = static_cast<char *>(s.c) + (size_t)r0 * row_c;
        if (row_a && (e = cudaMemcpyAsync(dA, static_cast<const char *>(hA) + (size_t)r0 * row_a, (size_t)rows * row_a,
                                          cudaMemcpyHostToDevice, stream)) != cudaSuccess)
            return record_cuda_error(e, "cudaMemcpyAsync(A)");
        if (i == 0 && b_parts > 1) {
            for (int j = 0, c0 = 0; c0 < n; ++j, c0 += cols_per_part) {
                const int cols = (n - c0 < cols_per_part) ? n - c0 : cols_per_part;
                char *dB = static_cast<char *>(s.b) + (size_t)c0 * row_a;
                if (row_a && (e = cudaMemcpyAsync(dB, static_cast<const char *>(hB) + (size_t)c0 * row_a, (size_t)cols * row_a,
                                                  cudaMemcpyHostToDevice, stream)) != cudaSuccess)
                    return record_cuda_error(e, "cudaMemcpyAsync(B)");
                st = gemm_dispatch(dA, dB, dC + (size_t)c0 * 4, rows, cols, k, n, stream, nullptr);
                if (st != QM_OK) return st;
                cudaEvent_t ev = s.slab_done[kHostSlabs + j % kHostBParts];
                if ((e = cudaEventRecord(ev, stream)) != cudaSuccess) return record_cuda_error(e, "cudaEventRecord");
                if ((e = cudaStreamWaitEvent(s.copy_stream, ev, 0)) != cudaSuccess) return record_cuda_error(e, "cudaStreamWaitEvent");
                if ((e = cudaMemcpy2DAsync(static_cast<char *>(hC) + (size_t)c0 * 4, row_c, dC + (size_t)c0 * 4, row_c, (size_t)cols * 4,
                                           (size_t)rows, cudaMemcpyDeviceToHost, s.copy_stream)) != cudaSuccess)
                    return record_cuda_error(e, "cudaMemcpy2DAsync(C)");
            }
            continue;
        }
        st = gemm_dispatch(dA, s.b, dC, rows, n, k, n, stream, nullptr);
        if (st != QM_OK) return st;
        cudaStream_t out_stream = stream;
        if (slabs > 1) {
            if ((e = cudaEventRecord(s.slab_done[i % kHostSlabs], stream)) != cudaSuccess) return record_cuda_error(e, "cudaEventRecord");
            if ((e = cudaStreamWaitEvent(s.copy_stream, s.slab_done[i % kHostSlabs], 0)) != cudaSuccess)
                return record_cuda_error(e, "cudaStreamWaitEvent");
            out_stream = s.copy_stream;
        }
        if ((e = cudaMemcpyAsync(static_cast<char *>(hC) + (size_t)r0 * row_c, dC, (size_t)rows * row_c, cudaMemcpyDeviceToHost,
                                 out_stream)) != cudaSuccess)
            return record_cuda_error(e, "cudaMemcpyAsync(C)");
    }
    if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) return record_cuda_error(e, "cudaStreamSynchronize");
    if (slabs > 1 && (e = cudaStreamSynchronize(s.copy_stream)) != cudaSuccess)
        return record_cuda_error(e, "cudaStreamSynchronize(copy)");
    int code = 0;
    if ((e = cudaMemcpy(&code, ctx->status, sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess)
        return record_cuda_error(e, "cudaMemcpy(status)");
    return code;
}

int qm_pack_s4(const void *in_s8, void *out_packed, int64_t rows, int64_t k, void *stream)
{
    if (rows < 0 || k < 0 || (k & 1)) return QM_ERR_SHAPE;
    if (rows == 0 || k == 0) return QM_OK;
    if (!in_s8 || !out_packed) return QM_ERR_NULL;
    return pack_launch(static_cast<const int8_t *>(in_s8), static_cast<uint8_t *>(out_packed), rows, k,
                       static_cast<cudaStream_t>(stream));
}

int qm_unpack_s4(const void *in_packed, void *out_s8, int64_t rows, int64_t k, void *stream)
{
    if (rows < 0 || k < 0 || (k & 1)) return QM_ERR_SHAPE;
    if (rows == 0 || k == 0) return QM_OK;
    if (!in_packed || !out_s8) return QM_ERR_NULL;
    return unpack_launch(static_cast<const uint8_t *>(in_packed), static_cast<int8_t *>(out_s8), rows, k,
                         static_cast<cudaStream_t>(stream));
}

int qm_fill_s4(void *out_packed, int64_t rows, int64_t k, uint64_t seed, void *stream)
{
    if (rows < 0 || k < 0 || (k & 1)) return QM_ERR_SHAPE;
    if (rows == 0 || k == 0) return QM_OK;
    if (!out_packed) return QM_ERR_NULL;
    return fill_launch(static_cast<uint8_t *>(out_packed), rows, k, seed, static_cast<cudaStream_t>(stream));
}

int qm_nshard_range(int n, int world, int rank, int *begin, int *count)
{
    if (!begin || !count) return QM_ERR_NULL;
    if (n < 0 || world < 1 || rank < 0 || rank >= world) return QM_ERR_ARG;
    nshard_range(n, world, rank, begin, count);
    return QM_OK;
}

int qm_unshard_c(const void *slabs, void *C, int m, int n, int world, int64_t slab_stride, void *stream)
{
    if (m < 0 || n < 0 || world < 1) return QM_ERR_SHAPE;
    if (m == 0 || n == 0) return QM_OK;
    if (!slabs || !C) return QM_ERR_NULL;
    return unshard_launch(static_cast<const int32_t *>(slabs), static_cast<int32_t *>(C), m, n, world, slab_stride,
                          static_cast<cudaStream_t>(stream));
}

size_t qm_prelayout_b_bytes(int n, int k)
{
    if (n <= 0 || k <= 0) return 0;
    return prelayout_bytes(n, k);
}

int qm_prelayout_b(const void *B, void *B_pre, int n, int k, void *stream)
{
    if (n < 0 || k < 0 || (k % 32) != 0) return QM_ERR_SHAPE;
    if (n == 0 || k == 0) return QM_OK;
    if (!B || !B_pre) return QM_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(B) & 15u) || (reinterpret_cast<uintptr_t>(B_pre) & 15u)) return QM_ERR_ALIGN;
    return prelayout_launch(static_cast<const uint8_t *>(B), static_cast<uint8_t *>(B_pre), n, k, static_cast<cudaStream_t>(stream));
}

int qm_gemm_s4_prelaid(const void *A, const void *B_pre, void *C, int m, int n, int k, void *stream)
{
    int st = check_gemm_args(A, B_pre, C, m, n, k, n);
    if (st != QM_OK) return st;
    if (m == 0 || n == 0) return QM_OK;
    if (k == 0 || (k % 32) != 0) return QM_ERR_SHAPE;
    DeviceCtx *ctx = nullptr;
    st = ensure_ctx(&ctx);
    if (st != QM_OK) return st;
    GemmArgs g{static_cast<const uint8_t *>(A), static_cast<const uint8_t *>(B_pre), static_cast<int32_t *>(C), m, n, k, n,
               static_cast<cudaStream_t>(stream)};
    if (m > kRmmaMaxRows || k > (m <= 16 ? kRmmaMaxK : kRmmaMaxKTiled)) return QM_ERR_ARG;
    if (!rmma_eligible(g)) return QM_ERR_ALIGN;
    return rmma_launch_prelaid(g, *ctx);
}

int qm_flag_signal(int *flag, int value, void *stream)
{
    if (!flag) return QM_ERR_NULL;
    return flag_signal_launch(flag, value, static_cast<cudaStream_t>(stream));
}

int qm_flags_wait(const int *flags, int count, int value, int timeout_ms, void *stream)
{
    if (!flags) return QM_ERR_NULL;
    if (count < 1 || count > 64 || timeout_ms < 1 || timeout_ms > 60000) return QM_ERR_ARG;
    DeviceCtx *ctx = nullptr;
    int st = ensure_ctx(&ctx);
    if (st != QM_OK) return st;
    return flags_wait_launch(flags, count, value, timeout_ms, ctx->status, static_cast<cudaStream_t>(stream));
}

int qm_device_status(int *code, int *where, int clear)
{
    DeviceCtx *ctx = nullptr;
    int st = ensure_ctx(&ctx);
    if (st != QM_OK) return st;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return record_cuda_error(e, "cudaDeviceSynchronize");
    int words[2] = {0, 0};
    if ((e = cudaMemcpy(words, ctx->status, sizeof(words), cudaMemcpyDeviceToHost)) != cudaSuccess)
        return record_cuda_error(e, "cudaMemcpy(status)");
    if (code) *code = words[0];
    if (where) *where = words[1];
    if (clear) {
        if ((e = cudaMemset(ctx->status, 0, sizeof(words))) != cudaSuccess) return record_cuda_error(e, "cudaMemset(status)");
        // A launch whose wait expired leaves arrival counters and share flags of its K partitions non-zero (the partitions
        // that gave up never arrive); they are self-resetting only in launches that complete.  Start the next launch clean.
        if ((e = cudaMemset(ctx->counters, 0, (size_t)kNumSlices * kSliceCounters * sizeof(int))) != cudaSuccess)
            return record_cuda_error(e, "cudaMemset(counters)");
    }
    return QM_OK;
}

int qm_stream_release(void *stream)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e, "cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return QM_ERR_ARG;
    const uintptr_t key = stream_key(static_cast<cudaStream_t>(stream));
    for (int i = 0; i < kNumSlices; ++i) {
        uintptr_t cur = key;
        if (g_slice_key[dev][i].compare_exchange_strong(cur, 0, std::memory_order_acq_rel)) break;
    }
    return QM_OK;
}

int qm_selftest_stale_counters(void *stream)
{
    DeviceCtx *ctx = nullptr;
    int st = ensure_ctx(&ctx);
    if (st != QM_OK) return st;
    const DeviceCtx lc = ctx_for_stream(*ctx, static_cast<cudaStream_t>(stream));
    if (!lc.counters) return QM_ERR_WORKSPACE;
    cudaError_t e = cudaMemsetAsync(lc.counters, 1, 256 * sizeof(int), static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? QM_OK : record_cuda_error(e, "cudaMemsetAsync(counters)");
}

int qm_plan(int m, int n, int k, qm_gemm_opts_t *opts)
{
    if (!opts) return QM_ERR_NULL;
    if (m < 0 || n < 0 || k < 0 || (k & 1)) return QM_ERR_SHAPE;
    std::memset(opts, 0, sizeof(*opts));
    if (k % 32 != 0 || k >= 131072) {
        opts->kernel = QM_KERNEL_SIMT;
        return QM_OK;
    }
    TcPlan p = plan_tc(m, n, k, 148);
    opts->kernel = QM_KERNEL_TC;
    if (m >= 1 && m <= kRmmaMaxRows) {  // aligned operands assumed
        const bool ok[3] = {rmma_shape_limits(m, k), gemv_shape_limits(m, k), true};
        const int fam = choose_decode_family(m, n, k, 148, ok);
        opts->kernel = fam == kFamRmma ? QM_KERNEL_RMMA : (fam == kFamGemv ? QM_KERNEL_GEMV : QM_KERNEL_TC);
    }
    opts->tile_n = p.tile_n;
    opts->swap_ab = p.swap_ab + 1;
    opts->split_k = p.split_k;
    opts->cta_pair = p.cta_pair;
    opts->a_tmem = p.a_tmem + 1;
    opts->stream_k = p.stream_k + 1;
    opts->ctas_per_sm = p.ctas_per_sm;
    return QM_OK;
}

}  // extern "C"

// The reference's C++ entry point (extension.cpp:6, kernel.cu:334), same signature and linkage.
void wrapper(void *A, void *B, void *C, const int m, const int n, const int k, CUstream_st *stream)
{
    int st = qm_gemm_s4(A, B, C, m, n, k, stream);
    if (st != QM_OK) {
        static int reported_mask = 0;
        if (!(reported_mask & (1 << st))) {
            reported_mask |= 1 << st;
            std::fprintf(stderr, "quadmul_b200: wrapper(m=%d, n=%d, k=%d) failed: %s %s\n", m, n, k, qm_status_string(st),
                         qm_last_cuda_error());
        }
    }
}
