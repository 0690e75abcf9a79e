/*
 * TEST INFRASTRUCTURE — CPU restatement of the reference's FP32 GEMM path.
 *
 * This file is the checker, never the product: only the test-suite, the smoke
 * check and the benchmark's CPU-baseline leg may build or call it.  The
 * shipped SGEMM path is the CUDA kernel loaded by libsgemm_runner.so and has
 * no CPU fallback.
 *
 * What is restated (paths are relative to the reference project):
 *   - runner/generator_runner.cpp:16-33  cpuGemm: column-major NN,
 *       d[i + j*m] = beta*c[i + j*m] + alpha * sum_l a[i + l*m] * b[l + j*k],
 *     FP32 throughout, k ascending, one multiply then one add per term
 *     (build with -ffp-contract=off so no FMA is formed).
 *   - runner/generator_runner.cpp:133-148 leading dimensions lda=M, ldb=K,
 *     ldc=ldd=M (generalised here to explicit lda/ldb/ldc/ldd because the
 *     kernel ABI carries them, generator/generator.py:2603-2618).
 *   - runner/Utils/Math.hpp:5-8 and generator_runner.cpp:289-304: the
 *     reference's own comparison rule |gpu - cpu| < 1e-3.
 *   - runner/generator_runner.cpp:75-83 the Gflops / "GiB/s" formulas.
 *
 * oracle_gemm_ref_order  : the reference's i -> j -> l loop nest verbatim in
 *                          behaviour (single thread, strided A reads).
 * oracle_gemm            : the same per-element arithmetic (sequential l, mul
 *                          then add, same epilogue expression) with the loop
 *                          nest reordered j -> l -> i and OpenMP over j.  Only
 *                          the order in which *different* elements are visited
 *                          changes, so the output is bit-identical to
 *                          oracle_gemm_ref_order (tests assert memcmp-equality).
 * oracle_abs_bound       : S[i,j] = sum_l |a[i,l]| * |b[l,j]| in FP64, the
 *                          per-element scale of the parity tolerance
 *                          max|D - D_ref| <= 1e-5 * S.
 * oracle_fill_uniform    : the seeded index-hash generator U[-1,1) that the
 *                          NumPy helper and the device fill kernel restate
 *                          bit-for-bit (this replaces the reference's unseeded
 *                          mt19937, runner/Utils/BufferUtils.hpp:6-14).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* Launchers such as torchrun export OMP_NUM_THREADS=1; the timed CPU baseline asks for all cores explicitly. */
ORACLE_API void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* runner/generator_runner.cpp:16-33, loop order and arithmetic unchanged. */
ORACLE_API void oracle_gemm_ref_order(const float *a, const float *b, const float *c, float *d,
                                      float alpha, float beta, uint32_t m, uint32_t n, uint32_t k,
                                      uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd) {
    for (uint32_t i = 0; i < m; ++i) {
        for (uint32_t j = 0; j < n; ++j) {
            float acc = 0.0f;
            for (uint32_t l = 0; l < k; ++l) {
                acc += a[i + (size_t)l * lda] * b[l + (size_t)j * ldb];
            }
            const float cv = c ? c[i + (size_t)j * ldc] : 0.0f;
            d[i + (size_t)j * ldd] = beta * cv + alpha * acc;
        }
    }
}

/* Same arithmetic per element, j -> l -> i with a column accumulator. */
ORACLE_API void oracle_gemm(const float *a, const float *b, const float *c, float *d,
                            float alpha, float beta, uint32_t m, uint32_t n, uint32_t k,
                            uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd) {
#pragma omp parallel
    {
        float *acc = (float *)malloc(sizeof(float) * (m ? m : 1));
#pragma omp for schedule(dynamic, 4)
        for (int64_t j = 0; j < (int64_t)n; ++j) {
            memset(acc, 0, sizeof(float) * m);
            for (uint32_t l = 0; l < k; ++l) {
                const float bv = b[l + (size_t)j * ldb];
                const float *acol = a + (size_t)l * lda;
                for (uint32_t i = 0; i < m; ++i) {
                    acc[i] += acol[i] * bv;
                }
            }
            for (uint32_t i = 0; i < m; ++i) {
                const float cv = c ? c[i + (size_t)j * ldc] : 0.0f;
                d[i + (size_t)j * ldd] = beta * cv + alpha * acc[i];
            }
        }
        free(acc);
    }
}

/* S = |A|*|B| in FP64: the tolerance scale of the parity rule. */
ORACLE_API void oracle_abs_bound(const float *a, const float *b, double *s, uint32_t m, uint32_t n,
                                 uint32_t k, uint32_t lda, uint32_t ldb, uint32_t lds) {
#pragma omp parallel
    {
        double *acc = (double *)malloc(sizeof(double) * (m ? m : 1));
#pragma omp for schedule(dynamic, 4)
        for (int64_t j = 0; j < (int64_t)n; ++j) {
            memset(acc, 0, sizeof(double) * m);
            for (uint32_t l = 0; l < k; ++l) {
                const double bv = fabs((double)b[l + (size_t)j * ldb]);
                const float *acol = a + (size_t)l * lda;
                for (uint32_t i = 0; i < m; ++i) {
                    acc[i] += fabs((double)acol[i]) * bv;
                }
            }
            for (uint32_t i = 0; i < m; ++i) s[i + (size_t)j * lds] = acc[i];
        }
        free(acc);
    }
}

/* FP64-accumulated product, for error statistics (not a parity oracle). */
ORACLE_API void oracle_gemm_f64(const float *a, const float *b, const float *c, double *d,
                                float alpha, float beta, uint32_t m, uint32_t n, uint32_t k,
                                uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd) {
#pragma omp parallel
    {
        double *acc = (double *)malloc(sizeof(double) * (m ? m : 1));
#pragma omp for schedule(dynamic, 4)
        for (int64_t j = 0; j < (int64_t)n; ++j) {
            memset(acc, 0, sizeof(double) * m);
            for (uint32_t l = 0; l < k; ++l) {
                const double bv = (double)b[l + (size_t)j * ldb];
                const float *acol = a + (size_t)l * lda;
                for (uint32_t i = 0; i < m; ++i) acc[i] += (double)acol[i] * bv;
            }
            for (uint32_t i = 0; i < m; ++i) {
                const double cv = c ? (double)c[i + (size_t)j * ldc] : 0.0;
                d[i + (size_t)j * ldd] = (double)beta * cv + (double)alpha * acc[i];
            }
        }
        free(acc);
    }
}

/* splitmix64 finaliser over (element index, stream); top 24 bits -> [-1, 1). */
static inline uint64_t oracle_hash(uint64_t idx, uint64_t stream) {
    uint64_t x = idx + 0x9E3779B97F4A7C15ull * (stream + 1ull);
    x ^= x >> 30;
    x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27;
    x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return x;
}

ORACLE_API void oracle_fill_uniform(float *dst, uint64_t count, uint64_t first_index,
                                    uint64_t stream) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)count; ++i) {
        const uint64_t h = oracle_hash(first_index + (uint64_t)i, stream);
        dst[i] = (float)(h >> 40) * 0x1p-23f - 1.0f;
    }
}

/* runner/Utils/Math.hpp:5-8 + generator_runner.cpp:293-303: count of elements
 * with |x - y| >= delta (NaN counts as a mismatch, as `!(diff < delta)`). */
ORACLE_API uint64_t oracle_count_mismatches(const float *x, const float *y, uint64_t count,
                                            float delta) {
    uint64_t bad = 0;
#pragma omp parallel for reduction(+ : bad) schedule(static)
    for (int64_t i = 0; i < (int64_t)count; ++i) {
        if (!(fabsf(x[i] - y[i]) < delta)) ++bad;
    }
    return bad;
}

/* Parity rule of the build: worst ratio |x - ref| / (rel * S) over all
 * elements (<= 1 passes).  Elements with S == 0 must match exactly. */
ORACLE_API double oracle_worst_ratio(const float *x, const float *ref, const double *s,
                                     uint64_t count, double rel) {
    double worst = 0.0;
#pragma omp parallel for reduction(max : worst) schedule(static)
    for (int64_t i = 0; i < (int64_t)count; ++i) {
        const double diff = fabs((double)x[i] - (double)ref[i]);
        double r;
        if (diff != diff) r = INFINITY;
        else if (s[i] > 0.0) r = diff / (rel * s[i]);
        else r = (diff == 0.0) ? 0.0 : INFINITY;
        if (r > worst) worst = r;
    }
    return worst;
}

/* runner/generator_runner.cpp:75-83. */
ORACLE_API double oracle_gflops(uint32_t m, uint32_t n, uint32_t k, double ms) {
    return 2.0 * m * n * k / ms * 1e-6;
}
ORACLE_API double oracle_mem_bw(uint64_t m, uint64_t n, uint64_t k, double ms) {
    return (double)(m * k + n * k + 2 * m * n) * 4.0 / ms / 1024.0 / 1024.0;
}
