/*
 * CPU oracle for the packed signed-int4 GEMM  C[M,N] (int32) = A[M,K] (s4) * B[N,K]^T (s4).
 *
 * THIS FILE IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the
 * smoke check and the CPU-baseline leg of the benchmark may call it; the shipped
 * library never links or loads it.
 *
 * It restates, in plain C, the host-side semantics of the reference project
 * (carsonpo/quadmul):
 *   - nibble order and sign rule      kernel.cu:387        (U4_TO_S4: x > 7 ? x - 16 : x)
 *   - unpacking of a packed matrix    kernel.cu:389-408    (low nibble = even k, high nibble = odd k)
 *   - packing                         test.py:6-15         (negatives + 16, even | odd << 4)
 *   - the GEMM itself                 kernel.cu:291-306    (C[m,n] = sum_k A[m,k] * B[n,k])
 * The reference accumulates in int32; this restatement accumulates in int64 and
 * reports how many outputs do not fit int32 (none do for any K < 2^25), so the
 * two agree bit for bit wherever the reference itself is well defined.
 *
 * Parity pin: tests/test_oracle.py checks every function here against fixtures
 * produced by the reference's own compiled host functions and its Python packer
 * (tests/golden/make_golden.py), and against the reference binary when present.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* kernel.cu:387 */
static inline int8_t nibble_to_s4(unsigned x)
{
    x &= 0xFu;
    return (int8_t)(x > 7u ? (int)x - 16 : (int)x);
}

int qm_oracle_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void qm_oracle_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* kernel.cu:389-408: packed[rows, K/2] -> out[rows, K]; byte j/2 holds element j in its low
 * nibble and element j+1 in its high nibble. */
void qm_oracle_unpack(const uint8_t *packed, int8_t *out, int64_t rows, int64_t K)
{
    const int64_t kb = K / 2;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint8_t *src = packed + r * kb;
        int8_t *dst = out + r * K;
        for (int64_t j = 0; j < kb; ++j) {
            dst[2 * j] = nibble_to_s4(src[j] & 0xFu);
            dst[2 * j + 1] = nibble_to_s4((unsigned)src[j] >> 4);
        }
    }
}

/* test.py:6-15: in[rows, K] with values in [-8, 7] -> packed[rows, K/2].
 * Returns the number of input values outside [-8, 7] (they are packed modulo 16). */
int64_t qm_oracle_pack(const int8_t *in, uint8_t *packed, int64_t rows, int64_t K)
{
    const int64_t kb = K / 2;
    int64_t bad = 0;
#pragma omp parallel for schedule(static) reduction(+ : bad)
    for (int64_t r = 0; r < rows; ++r) {
        const int8_t *src = in + r * K;
        uint8_t *dst = packed + r * kb;
        for (int64_t j = 0; j < kb; ++j) {
            int e = src[2 * j], o = src[2 * j + 1];
            bad += (e < -8 || e > 7) + (o < -8 || o > 7);
            unsigned ue = (unsigned)(e < 0 ? e + 16 : e) & 0xFu;
            unsigned uo = (unsigned)(o < 0 ? o + 16 : o) & 0xFu;
            dst[j] = (uint8_t)(ue | (uo << 4));
        }
    }
    return bad;
}

/* Dot product of two unpacked rows with an int64 total.  Partial sums over blocks of
 * 16384 elements stay below 2^20 in magnitude, so an int32 inner accumulator is exact
 * and lets the compiler vectorise. */
static int64_t dot_s8(const int8_t *a, const int8_t *b, int64_t K)
{
    int64_t total = 0;
    for (int64_t k0 = 0; k0 < K; k0 += 16384) {
        int64_t k1 = k0 + 16384 < K ? k0 + 16384 : K;
        int32_t acc = 0;
        for (int64_t k = k0; k < k1; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
        total += acc;
    }
    return total;
}

/* kernel.cu:291-306 on packed operands, for the row range [m0, m1) of C.
 * C has leading dimension ldc (elements) and receives rows m0..m1-1 at C[(m - c_row0) * ldc + n].
 * Returns the number of outputs that did not fit int32 (stored truncated). */
int64_t qm_oracle_gemm_s4_rows(const uint8_t *A, const uint8_t *B, int32_t *C, int64_t M, int64_t N,
                               int64_t K, int64_t m0, int64_t m1, int64_t c_row0, int64_t ldc)
{
    (void)M;
    const int64_t kb = K / 2;
    int64_t overflow = 0;
    if (m1 <= m0 || N <= 0) return 0;
    if (K <= 0) {
        for (int64_t m = m0; m < m1; ++m)
            memset(C + (m - c_row0) * ldc, 0, (size_t)N * sizeof(int32_t));
        return 0;
    }
    int8_t *Bu = (int8_t *)malloc((size_t)N * (size_t)K);
    int8_t *Au = (int8_t *)malloc((size_t)(m1 - m0) * (size_t)K);
    if (!Bu || !Au) {
        free(Bu);
        free(Au);
        return -1;
    }
    qm_oracle_unpack(B, Bu, N, K);
    qm_oracle_unpack(A + m0 * kb, Au, m1 - m0, K);
    /* 8x8 blocking keeps the B rows of a block in cache while the A rows stream. */
    const int64_t MB = 8, NB = 64;
    const int64_t mblocks = (m1 - m0 + MB - 1) / MB, nblocks = (N + NB - 1) / NB;
#pragma omp parallel for schedule(dynamic, 4) reduction(+ : overflow) collapse(2)
    for (int64_t bm = 0; bm < mblocks; ++bm) {
        for (int64_t bn = 0; bn < nblocks; ++bn) {
            int64_t me = (bm + 1) * MB < (m1 - m0) ? (bm + 1) * MB : (m1 - m0);
            int64_t ne = (bn + 1) * NB < N ? (bn + 1) * NB : N;
            for (int64_t mi = bm * MB; mi < me; ++mi) {
                const int8_t *a = Au + mi * K;
                int32_t *crow = C + (mi + m0 - c_row0) * ldc;
                for (int64_t n = bn * NB; n < ne; ++n) {
                    int64_t s = dot_s8(a, Bu + n * K, K);
                    overflow += (s > INT32_MAX || s < INT32_MIN);
                    crow[n] = (int32_t)s;
                }
            }
        }
    }
    free(Bu);
    free(Au);
    return overflow;
}

int64_t qm_oracle_gemm_s4(const uint8_t *A, const uint8_t *B, int32_t *C, int64_t M, int64_t N, int64_t K)
{
    return qm_oracle_gemm_s4_rows(A, B, C, M, N, K, 0, M, 0, N);
}

/* The same sum for a list of (row, col) positions only: out[i] = C[rows[i], cols[i]] as int64.
 * Used where a full product is too large to recompute on the host. */
void qm_oracle_gemm_s4_points(const uint8_t *A, const uint8_t *B, int64_t K, const int64_t *rows,
                              const int64_t *cols, int64_t npoints, int64_t *out)
{
    const int64_t kb = K / 2;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < npoints; ++i) {
        const uint8_t *a = A + rows[i] * kb, *b = B + cols[i] * kb;
        int64_t s = 0;
        for (int64_t j = 0; j < kb; ++j) {
            s += (int64_t)nibble_to_s4(a[j] & 0xFu) * nibble_to_s4(b[j] & 0xFu);
            s += (int64_t)nibble_to_s4((unsigned)a[j] >> 4) * nibble_to_s4((unsigned)b[j] >> 4);
        }
        out[i] = s;
    }
}

/* Counter-based input generator shared with the CUDA fill kernel: element (row, col) of a
 * matrix with K columns is ((mix64(seed + row*K + col) >> 33) & 15) - 8, uniform on [-8, 7].
 * mix64 is the splitmix64 finaliser. */
static inline uint64_t mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

int qm_oracle_value(uint64_t seed, int64_t row, int64_t col, int64_t K)
{
    return (int)((mix64(seed + (uint64_t)(row * K + col)) >> 33) & 15u) - 8;
}

void qm_oracle_fill_packed(uint8_t *packed, int64_t rows, int64_t K, uint64_t seed)
{
    const int64_t kb = K / 2;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t j = 0; j < kb; ++j) {
            unsigned e = (unsigned)(mix64(seed + (uint64_t)(r * K + 2 * j)) >> 33) & 15u;
            unsigned o = (unsigned)(mix64(seed + (uint64_t)(r * K + 2 * j + 1)) >> 33) & 15u;
            /* value v = u - 8; its nibble is v mod 16 = (u + 8) & 15 */
            packed[r * kb + j] = (uint8_t)(((e + 8u) & 15u) | (((o + 8u) & 15u) << 4));
        }
    }
}
