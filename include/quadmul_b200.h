/*
 * quadmul_b200 -- C ABI of the B200 (sm_100a) packed signed-int4 GEMM.
 *
 *   C[M,N] (int32, row-major) = A[M,K] (s4) * B[N,K]^T (s4)
 *
 * Operand layout (identical to carsonpo/quadmul, so the library is a drop-in for its
 * GEMM path): two two's-complement nibbles per byte, element 2j in the LOW nibble and element
 * 2j+1 in the HIGH nibble of byte j (reference: test.py:14, kernel.cu:395-396, kernel.cu:387);
 * A is row-major M x K/2 bytes, B is N x K/2 bytes (K contiguous: "B is transposed",
 * reference kernel.cu:77-78); C is M x N int32 and is fully overwritten.
 *
 * All pointers are DEVICE pointers on the current CUDA device unless a function says "host".
 * `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).  Calls are
 * asynchronous on that stream; nothing here synchronises unless stated.  Every function returns
 * a qm_status_t and never fails silently; there is no CPU fallback.
 */
#ifndef QUADMUL_B200_H
#define QUADMUL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum qm_status {
    QM_OK = 0,
    QM_ERR_NULL = 1,      /* a required pointer is NULL                                   */
    QM_ERR_SHAPE = 2,     /* m, n, k not positive, k odd, or sizes overflow the kernel     */
    QM_ERR_ALIGN = 3,     /* reserved: operands the selected kernel cannot address         */
    QM_ERR_CUDA = 4,      /* a CUDA runtime/driver call failed (see qm_last_cuda_error)    */
    QM_ERR_TIMEOUT = 5,   /* a bounded in-kernel wait expired (see qm_device_status)       */
    QM_ERR_ARCH = 6,      /* the current device is not compute capability 10.x             */
    QM_ERR_WORKSPACE = 7, /* caller-provided or built-in scratch is too small              */
    QM_ERR_ARG = 8        /* an option value is out of range                               */
} qm_status_t;

/* Kernel families the dispatcher chooses from.  QM_KERNEL_AUTO lets the tile table decide. */
typedef enum qm_kernel {
    QM_KERNEL_AUTO = 0,
    QM_KERNEL_TC = 1,  /* TMA + mbarrier ring + in-smem s4->s8 + tcgen05.mma kind::i8 + TMEM   */
    QM_KERNEL_SIMT = 2, /* dp4a kernel for shapes/alignments the tensor path does not take      */
    QM_KERNEL_GEMV = 3, /* m <= 4: weight-streaming dp4a kernel (same shape limits as QM_KERNEL_TC) */
    QM_KERNEL_RMMA = 4  /* m <= 64 (k <= 8192 for m <= 16, k <= 4096 beyond): weights straight into registers, warp-level mma.sync s8 */
} qm_kernel_t;

/* Options for qm_gemm_s4_ex.  Zero-initialise for defaults. */
typedef struct qm_gemm_opts {
    int kernel;     /* qm_kernel_t                                                              */
    int tile_n;     /* 0 = table; UMMA N extent of the CTA tile: 16..256 (multiple of 16)       */
    int swap_ab;    /* 0 = table, 1 = C rows on UMMA-M (prefill form), 2 = C columns on UMMA-M  */
    int split_k;    /* 0 = table; >= 1 number of K partitions reduced through scratch memory    */
    int cta_pair;   /* 0 = table, 1 = single-CTA MMA, 2 = two-CTA (cta_group::2) MMA            */
    int a_tmem;     /* 0 = table, 1 = the UMMA-M operand from shared memory, 2 = from TMEM: with tile_n 256,
                       cta_pair 2 and no swap the large-shape kernel; with swap_ab 2 and tile_n 16/32/64
                       the decode kernel                                                          */
    int plain_stores; /* 1 = write C with ordinary vector stores only (no TMA store); for a C that lives in
                         another GPU's memory (peer mapping), as the fused gather of the sharded driver uses */
    int stream_k;   /* how K is cut and the partial tiles meet.  Decode kernel: 0 = table, 1 = split_k partitions
                       per tile summed through scratch memory, 2 = one equal contiguous share of the (tile, K) work
                       per CTA summed through scratch memory, 3 = split_k (2..4) partitions per tile, one CTA each in
                       one thread-block cluster, summed through the cluster's shared memory.  Large-shape kernel
                       (256 x 256 pair tile): 0 = table, 1 = whole tiles only, 2 = when the last round of whole tiles
                       over the CTA pairs is short, its tiles run as K partitions that add into zeroed tiles */
    int ctas_per_sm; /* decode kernel only: 0 = table, 1 = one CTA per SM with the whole shared memory as its ring,
                        2 = two smaller CTAs per SM (tile_n 16 only)                                  */
} qm_gemm_opts_t;

const char *qm_status_string(int status);
int qm_version(void);

/* Text of the last CUDA error this thread saw inside the library ("" if none). */
const char *qm_last_cuda_error(void);

/*
 * One-time per-device set-up (status word, split-K scratch, kernel attributes).  Optional: the
 * first qm_gemm_s4 on a device does it implicitly, but that first call then allocates, so call
 * qm_init before capturing a CUDA graph.  Replaces nothing in the reference (it has no set-up;
 * reference kernel.cu:268-289 launches unconditionally).
 */
int qm_init(int device);

/*
 * The GEMM.  Replaces `wrapper(void*A, void*B, void*C, int m, int n, int k, cudaStream_t)`
 * (reference kernel.cu:334-385) behind `quadmul.gemm` (reference extension.cpp:8-24).  Unlike the
 * reference, every (m, n, k) with k even is accepted; shapes the tensor path cannot take
 * (k % 32 != 0, pointers not 16-byte aligned, k >= 131072) run on the dp4a kernel instead.
 *
 * Calls may overlap on the GPU (different streams, several host threads).  Forms that cut K keep their partial tiles and
 * arrival counters in per-device scratch memory that qm_init allocates; every stream gets a slice of its own the first time
 * it needs one (6 slices per device; the per-thread default stream counts once per host thread), and a call on a seventh stream
 * runs a form without scratch instead, so results never depend on what else is running.  A launch captured into a CUDA graph
 * keeps the slice of the stream it was captured on: graphs that are replayed at the same time must have been captured on
 * different streams.
 */
int qm_gemm_s4(const void *A, const void *B, void *C, int m, int n, int k, void *stream);

/*
 * Gives back the scratch slice that `stream` holds on the current device (see qm_gemm_s4), for programs that create and
 * destroy many streams.  Call it when no work of this library is pending on the stream, e.g. before cudaStreamDestroy.
 * A stream without a slice is not an error.  No counterpart in the reference (its kernel keeps no state).
 */
int qm_stream_release(void *stream);

/* Same, with explicit kernel/tile choices (used by the tuner and the tests). */
int qm_gemm_s4_ex(const void *A, const void *B, void *C, int m, int n, int k, void *stream,
                  const qm_gemm_opts_t *opts);

/*
 * Same product with a leading dimension for C (elements): writes C[r * ldc + c].  Lets a rank that
 * owns a block of B's rows write its column slab straight into a full-width C.
 */
int qm_gemm_s4_ldc(const void *A, const void *B, void *C, int m, int n, int k, int64_t ldc,
                   void *stream);

/* qm_gemm_s4_ldc with options (see qm_gemm_opts_t). */
int qm_gemm_s4_ldc_ex(const void *A, const void *B, void *C, int m, int n, int k, int64_t ldc,
                      void *stream, const qm_gemm_opts_t *opts);

/*
 * HOST-buffer form for FFI callers that hold plain memory: copies A and B to the device, runs
 * the GEMM, copies C back and synchronises.  hA: m*k/2 bytes, hB: n*k/2 bytes, hC: m*n int32.
 * Replaces the sequence cudaMalloc/cudaMemcpy/launch/cudaMemcpy of the reference's stand-alone
 * harness (reference kernel.cu:457-508).
 */
int qm_gemm_s4_host(const void *hA, const void *hB, void *hC, int m, int n, int k);

/*
 * Pack int8 values in [-8, 7] (rows x k, k even) into nibbles (rows x k/2 bytes).
 * Replaces the Python `pack_b` (reference test.py:6-15).
 */
int qm_pack_s4(const void *in_s8, void *out_packed, int64_t rows, int64_t k, void *stream);

/*
 * Unpack nibbles (rows x k/2 bytes) into sign-extended int8 (rows x k).
 * Replaces the host function `unpack_int4_matrix` (reference kernel.cu:389-408).
 */
int qm_unpack_s4(const void *in_packed, void *out_s8, int64_t rows, int64_t k, void *stream);

/*
 * Fill a packed matrix with the counter-based generator value(seed,row,col) in [-8, 7]
 * (splitmix64 of seed + row*k + col, bits 33..36, minus 8).  Stands in for
 * `torch.randint` + `pack_b` of the reference's test (reference test.py:22-27).
 */
int qm_fill_s4(void *out_packed, int64_t rows, int64_t k, uint64_t seed, void *stream);

/*
 * Column-sharded multi-GPU helpers.  Rank `rank` of `world` owns B rows
 * [*begin, *begin + *count), i.e. the columns of C with those indices.  The split is contiguous,
 * in units of 128 columns where n allows, remainder to the last ranks.  No counterpart in the
 * reference (it is single-GPU).
 */
int qm_nshard_range(int n, int world, int rank, int *begin, int *count);

/*
 * Rank-major gathered slabs [world][m][*] (as an all-gather of per-rank column slabs produces,
 * each rank's slab padded to `slab_stride` elements) -> row-major C[m][n].
 */
int qm_unshard_c(const void *slabs, void *C, int m, int n, int world, int64_t slab_stride,
                 void *stream);

/*
 * Completion flags for the fused gather of the column-sharded product, where every rank's GEMM stores its slab straight
 * into the destination rank's C (qm_gemm_s4_ldc_ex with plain_stores on a peer mapping).
 *   qm_flag_signal: in stream order (after the GEMM), a system-scope fence and a release store of `value` to *flag;
 *     `flag` is normally a peer-mapped pointer to word `rank` of a flag array in the DESTINATION's memory.
 *   qm_flags_wait: a kernel on the current device that polls flags[0 .. count) (count <= 64) until each has reached
 *     `value` (values are step numbers that only grow), for at most `timeout_ms` (1 .. 60000).  If the limit expires
 *     the kernel records QM_ERR_TIMEOUT, wait site 8, in the device status word (qm_device_status) and returns: a rank
 *     that never signals costs the limit, it does not hang the GPU.
 * No counterpart in the reference (it is single-GPU).
 */
int qm_flag_signal(int *flag, int value, void *stream);
int qm_flags_wait(const int *flags, int count, int value, int timeout_ms, void *stream);

/*
 * In-kernel wait status of the current device: *code is 0 or QM_ERR_TIMEOUT, *where identifies
 * the wait that gave up.  Synchronises the device.  `clear` != 0 resets the word and zeroes the arrival
 * counters of the split-K scratch, which a launch that gave up leaves non-zero; the C of such a launch
 * is undefined.  Launches made through qm_gemm_s4_static_scratch report to a word of their own, see
 * qm_static_scratch_status.  No counterpart in the reference (its kernel has no waits).
 */
int qm_device_status(int *code, int *where, int clear);

/*
 * Test hook for the recovery path above: writes non-zero values into the first arrival counters of `stream`'s scratch
 * slice, as a launch whose wait expired would leave them (asynchronous on `stream`; nothing waits, nothing faults).
 * Until qm_device_status(clear = 1) has run, split-K launches on that stream sum the wrong partial tiles.  No
 * counterpart in the reference.
 */
int qm_selftest_stale_counters(void *stream);

/*
 * Exercises the time-out path of the kernels without a GEMM: launches one warp that waits, with the same bounded wait the
 * GEMM kernels use, on a barrier that nothing ever completes.  The wait gives up after its limit (0.2 s), the kernel
 * returns normally, and qm_device_status then reports QM_ERR_TIMEOUT with wait site 9.  Nothing faults or hangs; the
 * context stays usable.  No counterpart in the reference (its kernel has no waits that could fail).
 */
int qm_selftest_wait_timeout(void *stream);

/*
 * The split-K tensor-core GEMM for callers that must not allocate device memory (a plug-in under a
 * host framework's memory pool or a fixed device-memory budget, a real-time loop that cannot absorb
 * an allocation's stall).  It has no counterpart in the reference.  Same product and layouts as qm_gemm_s4
 * (ldc = n), computed in `split_k` >= 1 partitions of K whose partial tiles are summed through
 * scratch that lives in file-scope __device__ arrays of the library: no cudaMalloc, no cudaFree,
 * no allocating library call, on any call.
 *   Capacity: 8 MiB of partial tiles and 4096 arrival counters, i.e.
 *   tiles * split_k * 128 * tile_n * 4 bytes <= 8 MiB with tiles = ceil(n/128) * ceil(m/tile_n) for
 *   m <= 128 (tile_n = 16, 32, 64, 128 >= m), and 4 * tiles <= 4096; QM_ERR_WORKSPACE beyond it.
 *   Needs k % 32 == 0, k < 131072 and 16-byte-aligned A and B (QM_ERR_ALIGN otherwise).
 *   The first call on a device looks up the arrays' device addresses (cudaGetSymbolAddress) with
 *   that device current; make that first call outside any stream capture.  The arrays are part of the
 *   library's device code: the driver reserves their memory when it loads that code, which with lazy
 *   module loading happens during this first call -- so a process whose device memory is already
 *   exhausted sees the out-of-memory error here, as QM_ERR_CUDA, and nowhere later.
 *   Every call on a device shares the arrays: calls that overlap on the GPU race; order them.
 *   A bounded in-kernel wait that expires is recorded in a status word that also lives in the
 *   library's device code; read it with qm_static_scratch_status (qm_device_status allocates).
 */
int qm_gemm_s4_static_scratch(const void *A, const void *B, void *C, int m, int n, int k, int split_k,
                              void *stream);

/*
 * In-kernel wait status of the launches made through qm_gemm_s4_static_scratch on the current device:
 * same meaning as qm_device_status, and like that entry point it allocates nothing.  Synchronises the
 * device.  QM_OK with *code = 0 when that entry point has not been used on this device yet.  It has no
 * counterpart in the reference.
 */
int qm_static_scratch_status(int *code, int *where, int clear);

/*
 * The GEMM with a fused dequantising epilogue, for W4A4 inference: out[r][c] (bfloat16, row pitch ldc elements) =
 * bf16( float(sum) * scale_a[r] * scale_b[c] ), where sum is the exact int32 dot product, float() and bf16() round to
 * nearest even and the two multiplications are separate fp32 operations in that order (the CPU oracle repeats exactly
 * these steps, so results are compared bit for bit).  scale_a (m floats, per row of A / token) and scale_b (n floats, per
 * row of B / output channel) are device pointers; NULL means all ones.  It has no counterpart in the reference, whose
 * only epilogue is the int32 store (reference kernel.cu:155-184; README.md:7 names fusing as the intended use).
 *   Shapes that run the 256 x 256 large-shape kernel (m > 64, n > 128, k % 32 == 0, A, B and out 16-byte aligned,
 *   ldc % 8 == 0) or the decode kernel (m <= 64, k % 32 == 0, A and B 16-byte aligned) convert inside the GEMM
 *   epilogue and never write the int32 matrix: C traffic drops from 4 to 2 bytes per element and `workspace` is not
 *   touched.  Every other shape computes the int32 product into `workspace`
 *   (m * n * 4 bytes, device memory, 4-byte aligned; QM_ERR_WORKSPACE if smaller) and converts in a second pass.
 *   qm_gemm_s4_dequant_workspace_bytes tells which: 0 = fused (for 16-byte-aligned A and B).
 */
int qm_gemm_s4_dequant_bf16(const void *A, const void *B, const float *scale_a, const float *scale_b, void *out_bf16, int m, int n,
                            int k, int64_t ldc, void *workspace, size_t workspace_bytes, void *stream);
size_t qm_gemm_s4_dequant_workspace_bytes(int m, int n, int k, int64_t ldc, const void *out_bf16);

/*
 * Offline weight pre-layout for decode (optional; the plain layout stays the default everywhere).  Weights are static in
 * inference, so B can be rearranged once: qm_prelayout_b writes B' (qm_prelayout_b_bytes(n, k) bytes: rows padded to 32,
 * K to 4096 elements, still 4 bits per element) in the order in which the lanes of the register-resident decode kernel
 * load it: every load instruction of a warp reads 512 consecutive bytes, a warp's 4 KB and a CTA's 64 KB per round are
 * consecutive addresses.  qm_gemm_s4_prelaid is the product on such a B': same A, C and result as qm_gemm_s4,
 * within that kernel's limits (m <= 16 with k <= 8192, or m <= 64 with k <= 4096; QM_ERR_ARG beyond: larger shapes take
 * qm_gemm_s4 with the plain B), k % 32 == 0, 16-byte-aligned A and B'.
 * The reference left the hook for this and never built it (reference kernel.cu:57 `#define PRESHUFFLE false`,
 * kernel.cu:450 `reorganize_packed_B`).
 */
size_t qm_prelayout_b_bytes(int n, int k);
int qm_prelayout_b(const void *B, void *B_pre, int n, int k, void *stream);
int qm_gemm_s4_prelaid(const void *A, const void *B_pre, void *C, int m, int n, int k, void *stream);

/* What the dispatcher would run for (m, n, k): fills *opts with the resolved choices. */
int qm_plan(int m, int n, int k, qm_gemm_opts_t *opts);

#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
/*
 * The reference's C++ entry point, kept with its exact signature and linkage (reference
 * extension.cpp:6, kernel.cu:334) so code that declares it links unchanged.  Errors, which the
 * reference drops, are reported on stderr once per distinct status.
 */
struct CUstream_st;
void wrapper(void *A, void *B, void *C, const int m, const int n, const int k, CUstream_st *stream);
#endif

#endif /* QUADMUL_B200_H */
