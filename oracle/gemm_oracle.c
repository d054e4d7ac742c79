/*
 * TEST INFRASTRUCTURE — not part of the product.  Only tests/, __graft_entry__.smoke()
 * and bench.py's CPU-baseline legs may build, load or call this file.
 *
 * CPU restatement of the reference project's correctness oracle for the
 * half-precision GEMM:
 *
 *   sgemm::sgemm_naive_kernel<T>            src/impl/sgemm_impl.h:9-26
 *       float acc = 0;
 *       for (ki = 0; ki < k; ki++) acc += (float)a[mi*k+ki] * (float)b[ni*k+ki];
 *       c[mi*n+ni] = (T)acc;
 *   (the kernel test/cpp/test_gemm_half.cpp:62-63 validates hgemm_peak against),
 *   and the host triple loop of test/cpp/test_wmma_compute.cpp:81-94, same formula.
 *
 * The sum runs over k in increasing order in fp32.  A product of two bf16 (8-bit
 * significand) or two fp16 (11-bit significand) values is exact in fp32, so a
 * fused multiply-add and a separate multiply and add round identically: this
 * C loop and the reference's GPU kernel produce the same bits.
 *
 * Layout as the reference: A [m,k] row-major, B [n,k] row-major, C [m,n].
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round to nearest even, as __float2bfloat16_rn */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff; /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline float f16_to_f32(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}

/* round to nearest even, as __float2half_rn */
static inline uint16_t f32_to_f16(float f) {
    _Float16 v = (_Float16)f;
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}

/*
 * acc[m,n] (fp32, unrounded) of the reference formula.  B is first widened and
 * transposed to [k,n] fp32 so the inner loop runs over n with unit stride; the
 * order of the k-sum of every output is unchanged.
 * is_bf16: 1 = bf16 inputs, 0 = fp16 inputs.  Returns 0, or -1 if out of memory.
 */
int oracle_gemm_acc(float *acc, const uint16_t *a, const uint16_t *b, int64_t m, int64_t n, int64_t k,
                    int is_bf16) {
    float *bt = (float *)malloc(sizeof(float) * (size_t)(k > 0 ? k : 1) * (size_t)(n > 0 ? n : 1));
    if (!bt) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t ni = 0; ni < n; ++ni)
        for (int64_t ki = 0; ki < k; ++ki)
            bt[ki * n + ni] = is_bf16 ? bf16_to_f32(b[ni * k + ki]) : f16_to_f32(b[ni * k + ki]);
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t mi = 0; mi < m; ++mi) {
        float *row = acc + mi * n;
        for (int64_t ni = 0; ni < n; ++ni) row[ni] = 0.f;
        for (int64_t ki = 0; ki < k; ++ki) {
            const float av = is_bf16 ? bf16_to_f32(a[mi * k + ki]) : f16_to_f32(a[mi * k + ki]);
            const float *brow = bt + ki * n;
            for (int64_t ni = 0; ni < n; ++ni) row[ni] += av * brow[ni];
        }
    }
    free(bt);
    return 0;
}

/* c[m,n] in the input type: (T)acc, round to nearest even. */
int oracle_gemm(uint16_t *c, const uint16_t *a, const uint16_t *b, int64_t m, int64_t n, int64_t k,
                int is_bf16) {
    float *acc = (float *)malloc(sizeof(float) * (size_t)(m > 0 ? m : 1) * (size_t)(n > 0 ? n : 1));
    if (!acc) return -1;
    int r = oracle_gemm_acc(acc, a, b, m, n, k, is_bf16);
    if (r == 0) {
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < m * n; ++i) c[i] = is_bf16 ? f32_to_bf16(acc[i]) : f32_to_f16(acc[i]);
    }
    free(acc);
    return r;
}
