// Build shim for the UNMODIFIED reference sources (carsonpo/quadmul).
//
// TEST INFRASTRUCTURE ONLY.  The reference's translation unit is compiled from where it
// lies (the include path is given by oracle/Makefile); nothing of it is copied here.  The
// shim only adds C-linkage doors to functions the reference already defines, plus template
// instantiations of its own kernel for problem sizes its dispatch chain (kernel.cu:343-384)
// does not list, so the reference can serve as a second oracle at those sizes.
#include "kernel.cu"  // reference TU: igemm<>, launch_igemm<>, wrapper, cpu_gemm_int8, unpack_int4_matrix

extern "C" {

// kernel.cu:291-306
void qm_ref_cpu_gemm_int8(const int8_t *A, const int8_t *B, int32_t *C, int M, int N, int K)
{
    cpu_gemm_int8(A, B, C, M, N, K);
}

// kernel.cu:389-408
void qm_ref_unpack_int4_matrix(uint8_t *B, int8_t *B_unpacked, int N, int K)
{
    unpack_int4_matrix(B, B_unpacked, N, K);
}

// kernel.cu:334-385, the reference's own dispatcher (silent no-op on an unlisted shape).
void qm_ref_wrapper(void *A, void *B, void *C, int m, int n, int k, void *stream)
{
    wrapper(A, B, C, m, n, k, (cudaStream_t)stream);
}

// The reference kernel in its most common tile family (configs.cu: BlockRowWarps=4,
// BlockColWarps=4, WarpRowTiles=4, WarpColTiles=4, PatchM=4, PatchN=1, ChunkK=4, 2 stages,
// 128x128x128 tile) instantiated for extra (N, K) pairs.  Needs M % 8 == 0.
// Returns 0 if launched, 1 if (n, k) is not instantiated.
#define QM_REF_FAMILY(NN, KK) IGemmConfig<4, 4, 4, 4, 4, 1, 4, 2, 1, 8, 8, 32, NN, KK>
#define QM_REF_CASE(NN, KK)                                                                      \
    if (n == NN && k == KK) {                                                                    \
        launch_igemm<QM_REF_FAMILY(NN, KK)>((const uint8_t *)A, (const uint8_t *)B, (int32_t *)C, \
                                             m, (cudaStream_t)stream);                           \
        return 0;                                                                                \
    }
int qm_ref_gpu_gemm(void *A, void *B, void *C, int m, int n, int k, void *stream)
{
    QM_REF_CASE(1024, 1024)
    QM_REF_CASE(8192, 8192)
    QM_REF_CASE(4096, 4096)
    QM_REF_CASE(11008, 4096)
    QM_REF_CASE(12288, 4096)
    QM_REF_CASE(22016, 4096)
    QM_REF_CASE(4096, 11008)
    return 1;
}

}  // extern "C"
