// qm_gemm_s4_static_scratch: the split-K GEMM for callers that are not allowed to allocate.
//
// Who needs it: code that runs inside another system's memory regime and must not call cudaMalloc
// (or anything that does) -- a plug-in executing under a host framework's memory pool or a fixed
// device-memory budget, or a real-time loop where an allocation is an unbounded stall.  The ordinary entry
// points take their split-K scratch from buffers that qm_init (or the first call on a device)
// obtains with cudaMalloc; this one owns its scratch as file-scope __device__ arrays that are part
// of the loaded module, so nothing is allocated, ever.  The price is a fixed, modest capacity
// (below) that every GPU loading the library carries until the process exits.
//
// In host code `g_scratch` etc. are only handles for the symbol, not device addresses.  The real
// addresses are looked up with cudaGetSymbolAddress once per device, with that device current, on
// the first call made for that device; that first call should therefore be made outside any stream
// capture.  Later calls do no look-ups.
//
// All calls on one device share the arrays.  The arrays keep whatever the previous call left: the
// arrival counters, which must start at zero, are cleared on the stream before every launch, and
// the partial tiles are fully rewritten before they are read.  Two calls that overlap on the GPU
// (different streams, no ordering) race on the scratch and give wrong results; order them.
#include <atomic>
#include <mutex>

#include "qm_internal.h"
#include "qm_tile_table.h"

namespace {

constexpr size_t kStaticScratchInts = (8u << 20) / sizeof(int32_t);  // 8 MiB of partial tiles
constexpr int kStaticCounters = 4096;                               // 4 per output tile

static __device__ __align__(256) int32_t g_scratch[kStaticScratchInts];
static __device__ __align__(256) int g_counters[kStaticCounters];
static __device__ __align__(256) int g_status[2];  // in-kernel wait status of launches made through this entry point

struct StaticCtx {
    int32_t *scratch = nullptr;
    int *counters = nullptr;
    qm::DeviceCtx dev;
};

constexpr int kMaxDevices = 64;
StaticCtx g_static[kMaxDevices];
std::atomic<bool> g_static_ready[kMaxDevices];  // release-stored after g_static[dev] is complete
std::mutex g_static_mutex;

// First call on a device: resolve the device addresses of the arrays for THAT device.
int setup_current_device(StaticCtx **out)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return qm::record_cuda_error(e, "cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return QM_ERR_ARG;
    StaticCtx &s = g_static[dev];
    if (!g_static_ready[dev].load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!g_static_ready[dev].load(std::memory_order_relaxed)) {
            int major = 0, sms = 0;
            if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess)
                return qm::record_cuda_error(e, "cudaDeviceGetAttribute");
            if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess)
                return qm::record_cuda_error(e, "cudaDeviceGetAttribute");
            if (major != 10) return QM_ERR_ARCH;
            void *p_scratch = nullptr, *p_counters = nullptr, *p_status = nullptr;
            if ((e = cudaGetSymbolAddress(&p_scratch, g_scratch)) != cudaSuccess)
                return qm::record_cuda_error(e, "cudaGetSymbolAddress(scratch)");
            if ((e = cudaGetSymbolAddress(&p_counters, g_counters)) != cudaSuccess)
                return qm::record_cuda_error(e, "cudaGetSymbolAddress(counters)");
            if ((e = cudaGetSymbolAddress(&p_status, g_status)) != cudaSuccess)
                return qm::record_cuda_error(e, "cudaGetSymbolAddress(status)");
            int st = qm::tc_prepare_device();  // kernel attributes only; allocates nothing
            if (st != QM_OK) return st;
            s.scratch = static_cast<int32_t *>(p_scratch);
            s.counters = static_cast<int *>(p_counters);
            s.dev.device = dev;
            s.dev.cc_major = major;
            s.dev.num_sms = sms;
            s.dev.status = static_cast<int *>(p_status);
            s.dev.ready = true;
            g_static_ready[dev].store(true, std::memory_order_release);
        }
    }
    *out = &s;
    return QM_OK;
}

}  // namespace

extern "C" int qm_gemm_s4_static_scratch(const void *A, const void *B, void *C, int m, int n, int k, int split_k,
                                         void *stream)
{
    if (m < 0 || n < 0 || k <= 0 || (k & 1) || split_k < 1) return QM_ERR_SHAPE;
    if (m == 0 || n == 0) return QM_OK;
    if (!A || !B || !C) return QM_ERR_NULL;
    qm::GemmArgs g{static_cast<const uint8_t *>(A), static_cast<const uint8_t *>(B), static_cast<int32_t *>(C), m, n, k, n,
                   static_cast<cudaStream_t>(stream)};
    if (!qm::tc_eligible(g)) return QM_ERR_ALIGN;  // this entry point is the tensor-core split-K kernel only
    StaticCtx *s = nullptr;
    int st = setup_current_device(&s);
    if (st != QM_OK) return st;
    qm::TcPlan p = qm::plan_tc(m, n, k, s->dev.num_sms);
    p.cta_pair = 1;  // split-K runs on single-CTA tiles
    if (p.tile_n > 128 && !p.swap_ab) p.tile_n = 128;
    p.split_k = split_k;
    if (split_k > (k + 127) / 128) return QM_ERR_ARG;
    if (qm::tc_scratch_bytes_needed(m, n, p) > kStaticScratchInts * sizeof(int32_t) ||
        qm::tc_counters_needed(m, n, p) > kStaticCounters)
        return QM_ERR_WORKSPACE;  // beyond the built-in capacity: use qm_gemm_s4 or fewer partitions
    if (split_k > 1) {
        // the counters must start at zero whatever an earlier (possibly failed) launch left behind
        cudaError_t e = cudaMemsetAsync(s->counters, 0, sizeof(int) * (size_t)qm::tc_counters_needed(m, n, p), g.stream);
        if (e != cudaSuccess) return qm::record_cuda_error(e, "cudaMemsetAsync(counters)");
    }
    return qm::tc_launch_with_scratch(g, p, s->dev, s->scratch, kStaticScratchInts * sizeof(int32_t), s->counters,
                                      kStaticCounters);
}

// The status word of this entry point's launches.  Reads the file-scope word through the address resolved at set-up; a
// device on which the entry point was never used has nothing to report.
extern "C" int qm_static_scratch_status(int *code, int *where, int clear)
{
    if (code) *code = 0;
    if (where) *where = 0;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return qm::record_cuda_error(e, "cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return QM_ERR_ARG;
    if (!g_static_ready[dev].load(std::memory_order_acquire)) return QM_OK;
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return qm::record_cuda_error(e, "cudaDeviceSynchronize");
    int words[2] = {0, 0};
    int *status = g_static[dev].dev.status;
    if ((e = cudaMemcpy(words, status, sizeof(words), cudaMemcpyDeviceToHost)) != cudaSuccess)
        return qm::record_cuda_error(e, "cudaMemcpy(status)");
    if (code) *code = words[0];
    if (where) *where = words[1];
    if (clear && (e = cudaMemset(status, 0, sizeof(words))) != cudaSuccess) return qm::record_cuda_error(e, "cudaMemset(status)");
    return QM_OK;
}
