/*
 * oracle.c -- CPU restatement of MIND's deterministic integer BLAS rules.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA path is
 * compared against; the shipped library never links, loads or calls it.
 *
 * Every function restates, in plain scalar C, an oracle that the reference
 * (star-ga/mind) keeps beside its own kernels.  The reference file:line each one
 * follows is given above the function.  Parity of this restatement is PINNED:
 * the test-suite checks it against the seven committed sha256 values in
 * tests/cross_substrate_identity/<workload>/reference_hashes.toml of the reference and against
 * the reference's own C runtime (runtime-support/mind_intrinsics.c) compiled as
 * a black box.
 *
 * All arithmetic is two's-complement; every result is "exact i64 sum,
 * truncated once to i32" (wrap, never saturate).
 */
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_EXPORT __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- *
 * Seeded input generator.
 * tests/cross_substrate_identity.rs:589-601 (struct Lcg), xnode_driver.c:112-120.
 *   s <- s*1664525 + 1013904223 (mod 2^64);  u32 = s >> 16
 *   q16 = (i32)u32 >> shift   (the reference uses shift = 12)
 *   i8  = (i8)(u32 >> 16),  i16 = (i16)(u32 >> 16)
 * The state is passed by pointer so that a second operand continues the
 * stream of the first ("A is drawn completely before B").
 * ------------------------------------------------------------------------- */
static inline uint32_t lcg_next(uint64_t *s) {
    *s = *s * 1664525ULL + 1013904223ULL;
    return (uint32_t)(*s >> 16);
}

ORACLE_EXPORT void oracle_lcg_fill_q16(uint64_t *state, int32_t *out, int64_t n, int shift) {
    for (int64_t i = 0; i < n; ++i) out[i] = (int32_t)lcg_next(state) >> shift;
}

ORACLE_EXPORT void oracle_lcg_fill_i8(uint64_t *state, int8_t *out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = (int8_t)(lcg_next(state) >> 16);
}

ORACLE_EXPORT void oracle_lcg_fill_i16(uint64_t *state, int16_t *out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = (int16_t)(lcg_next(state) >> 16);
}

/* ------------------------------------------------------------------------- *
 * int8 GEMM.  tests/cross_substrate_identity.rs:1345-1357 (ref_gemm_i8_scalar).
 * A is M x K, B is K x N (NOT transposed), both row-major; C is M x N i32.
 * ------------------------------------------------------------------------- */
ORACLE_EXPORT void oracle_gemm_i8(const int8_t *a, const int8_t *b, int32_t *c,
                                  int64_t m, int64_t k, int64_t n) {
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
            int64_t acc = 0;
            for (int64_t kk = 0; kk < k; ++kk)
                acc += (int64_t)a[i * k + kk] * (int64_t)b[kk * n + j];
            c[i * n + j] = (int32_t)acc;
        }
}

/* ------------------------------------------------------------------------- *
 * Q16.16 dot.  runtime-support/mind_intrinsics.c:1462-1475
 * (mind_blas_dot_q16_scalar) and tests/cross_substrate_identity.rs:613-619.
 * Each product is shifted right by 16 (arithmetic: floor) BEFORE it is added.
 * Returns the i32 result sign-extended to i64.
 * ------------------------------------------------------------------------- */
ORACLE_EXPORT int64_t oracle_dot_q16(const int32_t *a, const int32_t *b, int64_t len) {
    int64_t acc = 0;
    for (int64_t i = 0; i < len; ++i)
        acc += ((int64_t)a[i] * (int64_t)b[i]) >> 16;
    return (int64_t)(int32_t)acc;
}

/* Q16.16 L1 distance.  runtime-support/mind_intrinsics.c:1551-1563. */
ORACLE_EXPORT int64_t oracle_dot_l1_q16(const int32_t *a, const int32_t *b, int64_t len) {
    int64_t acc = 0;
    for (int64_t i = 0; i < len; ++i) {
        int64_t d = (int64_t)a[i] - (int64_t)b[i];
        if (d < 0) d = -d;
        acc += d;
    }
    return (int64_t)(int32_t)acc;
}

/* Q16.16 matrix x vector.  benches/det_gemv_q16_mt.rs:186-196
 * (ref_gemv_q16_scalar); tests/cross_substrate_identity.rs:797-801. */
ORACLE_EXPORT void oracle_gemv_q16(const int32_t *w, const int32_t *x, int32_t *y,
                                   int64_t rows, int64_t cols) {
    for (int64_t r = 0; r < rows; ++r)
        y[r] = (int32_t)oracle_dot_q16(w + r * cols, x, cols);
}

/* Q16.16 GEMM over un-transposed B (K x N).  benches/det_matmul_q16.rs:227-239
 * (ref_gemm_q16_scalar). */
ORACLE_EXPORT void oracle_gemm_q16(const int32_t *a, const int32_t *b, int32_t *c,
                                   int64_t m, int64_t k, int64_t n) {
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
            int64_t acc = 0;
            for (int64_t kk = 0; kk < k; ++kk)
                acc += ((int64_t)a[i * k + kk] * (int64_t)b[kk * n + j]) >> 16;
            c[i * n + j] = (int32_t)acc;
        }
}

/* Q16.16 GEMM composed from row dots over B-transposed (N x K).
 * tests/cross_substrate_identity.rs:1254-1264 (ref_gemm_q16_scalar). */
ORACLE_EXPORT void oracle_gemm_q16_bt(const int32_t *a, const int32_t *bt, int32_t *c,
                                      int64_t m, int64_t k, int64_t n) {
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j)
            c[i * n + j] = (int32_t)oracle_dot_q16(a + i * k, bt + j * k, k);
}

/* int16 dot and matrix x vector: no shift, exact i64 sum, one truncation.
 * tests/cross_substrate_identity.rs:1706-1719; benches/det_matmul_i16.rs:218-231. */
ORACLE_EXPORT int64_t oracle_dot_i16(const int16_t *a, const int16_t *b, int64_t len) {
    int64_t acc = 0;
    for (int64_t i = 0; i < len; ++i) acc += (int64_t)a[i] * (int64_t)b[i];
    return (int64_t)(int32_t)acc;
}

ORACLE_EXPORT void oracle_gemv_i16(const int16_t *w, const int16_t *x, int32_t *y,
                                   int64_t rows, int64_t cols) {
    for (int64_t r = 0; r < rows; ++r)
        y[r] = (int32_t)oracle_dot_i16(w + r * cols, x, cols);
}

/* int16 GEMM.  The reference has no such kernel; this composes its int16 row
 * rule (benches/det_matmul_i16.rs:218-224, `acc as i32`) for every (i, j) with
 * x = column j of an un-transposed K x N B, the operand layout its i8 and Q16
 * GEMMs use.  Output is i32 (wrap). */
ORACLE_EXPORT void oracle_gemm_i16(const int16_t *a, const int16_t *b, int32_t *c,
                                   int64_t m, int64_t k, int64_t n) {
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
            int64_t acc = 0;
            for (int64_t kk = 0; kk < k; ++kk)
                acc += (int64_t)a[i * k + kk] * (int64_t)b[kk * n + j];
            c[i * n + j] = (int32_t)acc;
        }
}

/* ------------------------------------------------------------------------- *
 * Row-band partition of the reference's multithreaded kernels.
 * src/mlir/lowering.rs:10146-10205: T = max(1, min(ncpu, M, 256)),
 * band = ceil(M / T); band t owns rows [t*band, min((t+1)*band, M)).
 * Returns the number of non-empty bands; writes [start, end) pairs.
 * ------------------------------------------------------------------------- */
ORACLE_EXPORT int64_t oracle_row_bands(int64_t m, int64_t ncpu, int64_t *starts, int64_t *ends) {
    int64_t upper = m < 256 ? m : 256;
    int64_t t = ncpu < upper ? ncpu : upper;
    if (t < 1) t = 1;
    int64_t band = (m + t - 1) / t;
    int64_t used = 0;
    for (int64_t i = 0; i < t; ++i) {
        int64_t s = i * band, e = s + band;
        if (e > m) e = m;
        if (s >= e) break;
        starts[used] = s;
        ends[used] = e;
        ++used;
    }
    return used;
}
