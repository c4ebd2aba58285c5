/*
 * cpu_baseline.c -- threaded, cache-blocked CPU ports of the reference's
 * deterministic kernels, used ONLY to time a CPU baseline beside the GPU numbers
 * (and cross-checked against oracle.c in the tests).
 *
 * TEST / MEASUREMENT INFRASTRUCTURE ONLY: never linked into the shipped library.
 *
 * The reference's kernels for this path exist only as MLIR text that its Rust
 * compiler prints (src/mlir/lowering.rs) and that LLVM tools compile; neither
 * toolchain can be run where this is built, so these are PORTS that keep the
 * reference's structure:
 *   - int8 GEMM: BLIS-style jc/ic/pc blocking with the reference's block sizes
 *     (src/mlir/gemm_tuning.rs: I8_MC=1024, I8_KC=512, I8_NC=128), operands
 *     packed to i16 K-pairs, MR=4 x NR=16 micro-kernel on vpmaddwd
 *     (src/mlir/lowering.rs:7798 emit_i8_microkernel_avx2, :8371 emit_mm_i8_blocked);
 *   - Q16.16 GEMM: per row, broadcast A[i,k], 64-bit multiply of a B row
 *     segment, arithmetic >>16, 64-bit add (src/mlir/lowering.rs:9274-9282, :9433);
 *   - Q16.16 / int16 GEMV: one reduction per row
 *     (src/mlir/lowering.rs:9822-9996, :10723);
 *   - int8 GEMM, second rung: the reference's opt-in VNNI path (vpdpbusd), see below;
 *   - threading: contiguous owner-computes row bands, T = min(ncpu, M, 256),
 *     band = ceil(M/T) (src/mlir/lowering.rs:10146-10205), no reduction.
 * Build with -O3 -march=x86-64-v3 (the reference's level, src/target.rs:267-272).
 */
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>
#if defined(__x86_64__)
#include <immintrin.h>
#endif

#define BASELINE_EXPORT __attribute__((visibility("default")))

/* ---------------------------- row-band threading -------------------------- */
typedef void (*band_fn)(void *ctx, int64_t row_start, int64_t row_end);
typedef struct {
    band_fn fn;
    void *ctx;
    int64_t s, e;
} band_job;

static void *band_trampoline(void *p) {
    band_job *j = (band_job *)p;
    j->fn(j->ctx, j->s, j->e);
    return NULL;
}

/* Runs fn over [0, m) split as the reference splits it; returns threads used. */
static int64_t run_bands(band_fn fn, void *ctx, int64_t m, int64_t threads) {
    if (m <= 0) return 0;
    int64_t ncpu = threads > 0 ? threads : sysconf(_SC_NPROCESSORS_ONLN);
    int64_t upper = m < 256 ? m : 256;
    int64_t t = ncpu < upper ? ncpu : upper;
    if (t < 1) t = 1;
    int64_t band = (m + t - 1) / t;
    pthread_t tid[256];
    band_job job[256];
    int64_t used = 0;
    for (int64_t i = 0; i < t; ++i) {
        int64_t s = i * band, e = s + band;
        if (e > m) e = m;
        if (s >= e) break;
        job[used] = (band_job){fn, ctx, s, e};
        ++used;
    }
    for (int64_t i = 1; i < used; ++i) pthread_create(&tid[i], NULL, band_trampoline, &job[i]);
    band_trampoline(&job[0]);
    for (int64_t i = 1; i < used; ++i) pthread_join(tid[i], NULL);
    return used;
}

BASELINE_EXPORT int64_t baseline_online_cpus(void) { return sysconf(_SC_NPROCESSORS_ONLN); }

/* ------------------------------- int8 GEMM -------------------------------- */
enum { I8_MC = 1024, I8_KC = 512, I8_NC = 128, I8_MR = 4, I8_NR = 16 };

typedef struct {
    const int8_t *a, *b;
    int32_t *c;
    int64_t m, k, n;
} gemm_i8_ctx;

/* B block [kc x nc] -> i16 pairs: bp[(p*ncp + j)*2 + h] = B[k0+2p+h][j0+j]. */
static void pack_b_i8(const int8_t *b, int64_t n, int64_t k0, int64_t kc, int64_t j0, int64_t nc,
                      int64_t ncp, int16_t *bp) {
    int64_t kp = (kc + 1) / 2;
    for (int64_t p = 0; p < kp; ++p)
        for (int64_t j = 0; j < ncp; ++j)
            for (int h = 0; h < 2; ++h) {
                int64_t kk = 2 * p + h;
                bp[(p * ncp + j) * 2 + h] =
                    (kk < kc && j < nc) ? (int16_t)b[(k0 + kk) * n + j0 + j] : 0;
            }
}

/* A block [mc x kc] -> i16 pairs: ap[(i*kp + p)*2 + h] = A[i0+i][k0+2p+h]. */
static void pack_a_i8(const int8_t *a, int64_t k, int64_t i0, int64_t mc, int64_t k0, int64_t kc,
                      int16_t *ap) {
    int64_t kp = (kc + 1) / 2;
    for (int64_t i = 0; i < mc; ++i)
        for (int64_t p = 0; p < kp; ++p)
            for (int h = 0; h < 2; ++h) {
                int64_t kk = 2 * p + h;
                ap[(i * kp + p) * 2 + h] = kk < kc ? (int16_t)a[(i0 + i) * k + k0 + kk] : 0;
            }
}

static void micro_i8(const int16_t *ap, const int16_t *bp, int64_t kp, int64_t ncp, int64_t rows,
                     int64_t cols, int32_t *c, int64_t ldc, int first) {
#if defined(__AVX2__)
    __m256i acc[I8_MR][2];
    for (int r = 0; r < I8_MR; ++r) acc[r][0] = acc[r][1] = _mm256_setzero_si256();
    for (int64_t p = 0; p < kp; ++p) {
        __m256i b0 = _mm256_loadu_si256((const __m256i *)(bp + (p * ncp) * 2));
        __m256i b1 = _mm256_loadu_si256((const __m256i *)(bp + (p * ncp + 8) * 2));
        for (int r = 0; r < I8_MR; ++r) {
            int32_t pair;
            memcpy(&pair, ap + (r * kp + p) * 2, 4);
            __m256i av = _mm256_set1_epi32(pair);
            acc[r][0] = _mm256_add_epi32(acc[r][0], _mm256_madd_epi16(av, b0));
            acc[r][1] = _mm256_add_epi32(acc[r][1], _mm256_madd_epi16(av, b1));
        }
    }
    int32_t tile[I8_MR][I8_NR];
    for (int r = 0; r < I8_MR; ++r) {
        _mm256_storeu_si256((__m256i *)&tile[r][0], acc[r][0]);
        _mm256_storeu_si256((__m256i *)&tile[r][8], acc[r][1]);
    }
#else
    int32_t tile[I8_MR][I8_NR];
    memset(tile, 0, sizeof tile);
    for (int64_t p = 0; p < kp; ++p)
        for (int r = 0; r < I8_MR; ++r)
            for (int j = 0; j < I8_NR; ++j)
                tile[r][j] += (int32_t)ap[(r * kp + p) * 2] * bp[(p * ncp + j) * 2] +
                              (int32_t)ap[(r * kp + p) * 2 + 1] * bp[(p * ncp + j) * 2 + 1];
#endif
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t j = 0; j < cols; ++j) {
            uint32_t prev = first ? 0u : (uint32_t)c[r * ldc + j];
            c[r * ldc + j] = (int32_t)(prev + (uint32_t)tile[r][j]);
        }
}

static void gemm_i8_band(void *vctx, int64_t rs, int64_t re) {
    gemm_i8_ctx *g = (gemm_i8_ctx *)vctx;
    const int64_t k = g->k, n = g->n;
    if (n <= 0) return;
    if (k <= 0) {
        for (int64_t i = rs; i < re; ++i) memset(g->c + i * n, 0, (size_t)n * 4);
        return;
    }
    int16_t *ap = (int16_t *)malloc((size_t)(I8_MC + I8_MR) * (I8_KC + 2) * 2);
    int16_t *bp = (int16_t *)malloc((size_t)(I8_KC + 2) * (I8_NC + I8_NR) * 2);
    for (int64_t jc = 0; jc < n; jc += I8_NC) {
        int64_t nc = n - jc < I8_NC ? n - jc : I8_NC;
        int64_t ncp = (nc + I8_NR - 1) / I8_NR * I8_NR;
        for (int64_t ic = rs; ic < re; ic += I8_MC) {
            int64_t mc = re - ic < I8_MC ? re - ic : I8_MC;
            int64_t mcp = (mc + I8_MR - 1) / I8_MR * I8_MR;
            for (int64_t pc = 0; pc < k; pc += I8_KC) {
                int64_t kc = k - pc < I8_KC ? k - pc : I8_KC;
                int64_t kp = (kc + 1) / 2;
                pack_b_i8(g->b, n, pc, kc, jc, nc, ncp, bp);
                pack_a_i8(g->a, k, ic, mc, pc, kc, ap);
                if (mcp > mc) memset(ap + mc * kp * 2, 0, (size_t)(mcp - mc) * kp * 4);
                for (int64_t jr = 0; jr < nc; jr += I8_NR)
                    for (int64_t ir = 0; ir < mc; ir += I8_MR) {
                        int64_t rows = mc - ir < I8_MR ? mc - ir : I8_MR;
                        int64_t cols = nc - jr < I8_NR ? nc - jr : I8_NR;
                        micro_i8(ap + ir * kp * 2, bp + jr * 2, kp, ncp, rows, cols,
                                 g->c + (ic + ir) * n + jc + jr, n, pc == 0);
                    }
            }
        }
    }
    free(ap);
    free(bp);
}

/* C = A.B for int8 operands; returns the number of threads used. */
BASELINE_EXPORT int64_t baseline_gemm_i8_mt(const int8_t *a, const int8_t *b, int32_t *c, int64_t m,
                                            int64_t k, int64_t n, int64_t threads) {
    gemm_i8_ctx g = {a, b, c, m, k, n};
    return run_bands(gemm_i8_band, &g, m, threads);
}

/* ------------------- int8 GEMM, the reference's VNNI rung ------------------ */
/* Port of the reference's opt-in AVX-512-VNNI int8 path (MIND_INTDOT=vnni,
 * src/mlir/gemm_tuning.rs:200-236): the same jc/ic/pc blocking with its own tile
 * constants (I8_VNNI_MR=8, I8_VNNI_NR=32, I8_VNNI_NC=768, gemm_tuning.rs:177-195),
 * operands packed as raw bytes in K-quads, A pre-biased by xor 0x80 at pack time
 * (signed -> unsigned, src/mlir/lowering.rs:8191-8200), an 8 x 2-ZMM accumulator grid
 * of vpdpbusd (src/mlir/lowering.rs:8186 emit_i8_microkernel_vnni), and the exact
 * correction  sum a.b = sum (a+128).b - 128.sum b  with the column sums of the packed
 * B tile taken once per jr tile (src/mlir/lowering.rs:8053 emit_i8_vnni_bsum_hoist).
 * Every term is exact mod 2^32, so the bytes equal the AVX2 rung's.  Compiled for
 * AVX-512 by a per-function target attribute and only run when the CPU has VNNI. */
enum { V_MC = 1024, V_KC = 512, V_NC = 768, V_MR = 8, V_NR = 32 };

BASELINE_EXPORT int64_t baseline_have_vnni(void) {
#if defined(__x86_64__)
    return __builtin_cpu_supports("avx512vnni") && __builtin_cpu_supports("avx512bw") ? 1 : 0;
#else
    return 0;
#endif
}

#if defined(__x86_64__)
/* B block [kc x nc] -> K-quads: bp[(q*ncp + j)*4 + h] = B[k0+4q+h][j0+j] (zero padded). */
static void pack_b_vnni(const int8_t *b, int64_t n, int64_t k0, int64_t kc, int64_t j0, int64_t nc,
                        int64_t ncp, int8_t *bp) {
    int64_t kq = (kc + 3) / 4;
    for (int64_t q = 0; q < kq; ++q)
        for (int64_t j = 0; j < ncp; ++j)
            for (int h = 0; h < 4; ++h) {
                int64_t kk = 4 * q + h;
                bp[(q * ncp + j) * 4 + h] = (kk < kc && j < nc) ? b[(k0 + kk) * n + j0 + j] : 0;
            }
}

/* A block [mc x kc] -> K-quads per row, biased: ap[(i*kq + q)*4 + h] = A[i0+i][k0+4q+h] ^ 0x80.
 * Padding K positions hold 0x80 (= 0 + 128); B is zero there, and the correction uses the
 * column sums of the padded B, so they cancel. */
static void pack_a_vnni(const int8_t *a, int64_t k, int64_t i0, int64_t mc, int64_t mcp, int64_t k0,
                        int64_t kc, uint8_t *ap) {
    int64_t kq = (kc + 3) / 4;
    for (int64_t i = 0; i < mcp; ++i)
        for (int64_t q = 0; q < kq; ++q)
            for (int h = 0; h < 4; ++h) {
                int64_t kk = 4 * q + h;
                uint8_t v = (i < mc && kk < kc) ? (uint8_t)a[(i0 + i) * k + k0 + kk] : 0;
                ap[(i * kq + q) * 4 + h] = v ^ 0x80u;
            }
}

__attribute__((target("avx512f,avx512bw,avx512vnni")))
static void micro_vnni(const uint8_t *ap, const int8_t *bp, int64_t kq, int64_t ncp, int64_t rows,
                       int64_t cols, int32_t *c, int64_t ldc, int first) {
    __m512i acc[V_MR][2], bsum[2];
    for (int r = 0; r < V_MR; ++r) acc[r][0] = acc[r][1] = _mm512_setzero_si512();
    bsum[0] = bsum[1] = _mm512_setzero_si512();
    const __m512i ones = _mm512_set1_epi8(1);
    for (int64_t q = 0; q < kq; ++q) {
        const __m512i b0 = _mm512_loadu_si512((const void *)(bp + (q * ncp) * 4));
        const __m512i b1 = _mm512_loadu_si512((const void *)(bp + (q * ncp + 16) * 4));
        bsum[0] = _mm512_dpbusd_epi32(bsum[0], ones, b0);
        bsum[1] = _mm512_dpbusd_epi32(bsum[1], ones, b1);
        for (int r = 0; r < V_MR; ++r) {
            int32_t quad;
            memcpy(&quad, ap + (r * kq + q) * 4, 4);
            const __m512i av = _mm512_set1_epi32(quad);
            acc[r][0] = _mm512_dpbusd_epi32(acc[r][0], av, b0);
            acc[r][1] = _mm512_dpbusd_epi32(acc[r][1], av, b1);
        }
    }
    bsum[0] = _mm512_slli_epi32(bsum[0], 7);
    bsum[1] = _mm512_slli_epi32(bsum[1], 7);
    int32_t tile[V_MR][V_NR];
    for (int r = 0; r < V_MR; ++r) {
        _mm512_storeu_si512((void *)&tile[r][0], _mm512_sub_epi32(acc[r][0], bsum[0]));
        _mm512_storeu_si512((void *)&tile[r][16], _mm512_sub_epi32(acc[r][1], bsum[1]));
    }
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t j = 0; j < cols; ++j) {
            uint32_t prev = first ? 0u : (uint32_t)c[r * ldc + j];
            c[r * ldc + j] = (int32_t)(prev + (uint32_t)tile[r][j]);
        }
}

static void gemm_i8_vnni_band(void *vctx, int64_t rs, int64_t re) {
    gemm_i8_ctx *g = (gemm_i8_ctx *)vctx;
    const int64_t k = g->k, n = g->n;
    if (n <= 0) return;
    if (k <= 0) {
        for (int64_t i = rs; i < re; ++i) memset(g->c + i * n, 0, (size_t)n * 4);
        return;
    }
    uint8_t *ap = (uint8_t *)malloc((size_t)(V_MC + V_MR) * (V_KC + 4));
    int8_t *bp = (int8_t *)malloc((size_t)(V_KC + 4) * (V_NC + V_NR));
    for (int64_t jc = 0; jc < n; jc += V_NC) {
        int64_t nc = n - jc < V_NC ? n - jc : V_NC;
        int64_t ncp = (nc + V_NR - 1) / V_NR * V_NR;
        for (int64_t ic = rs; ic < re; ic += V_MC) {
            int64_t mc = re - ic < V_MC ? re - ic : V_MC;
            int64_t mcp = (mc + V_MR - 1) / V_MR * V_MR;
            for (int64_t pc = 0; pc < k; pc += V_KC) {
                int64_t kc = k - pc < V_KC ? k - pc : V_KC;
                int64_t kq = (kc + 3) / 4;
                pack_b_vnni(g->b, n, pc, kc, jc, nc, ncp, bp);
                pack_a_vnni(g->a, k, ic, mc, mcp, pc, kc, ap);
                for (int64_t jr = 0; jr < nc; jr += V_NR)
                    for (int64_t ir = 0; ir < mc; ir += V_MR) {
                        int64_t rows = mc - ir < V_MR ? mc - ir : V_MR;
                        int64_t cols = nc - jr < V_NR ? nc - jr : V_NR;
                        micro_vnni(ap + ir * kq * 4, bp + jr * 4, kq, ncp, rows, cols,
                                   g->c + (ic + ir) * n + jc + jr, n, pc == 0);
                    }
            }
        }
    }
    free(ap);
    free(bp);
}
#endif

/* C = A.B for int8 operands on the VNNI rung; returns the threads used, or -1 without VNNI. */
BASELINE_EXPORT int64_t baseline_gemm_i8_vnni_mt(const int8_t *a, const int8_t *b, int32_t *c, int64_t m,
                                                 int64_t k, int64_t n, int64_t threads) {
#if defined(__x86_64__)
    if (!baseline_have_vnni()) return -1;
    gemm_i8_ctx g = {a, b, c, m, k, n};
    return run_bands(gemm_i8_vnni_band, &g, m, threads);
#else
    (void)a; (void)b; (void)c; (void)m; (void)k; (void)n; (void)threads;
    return -1;
#endif
}

/* ------------------------------ Q16.16 GEMM ------------------------------- */
typedef struct {
    const int32_t *a, *b;
    int32_t *c;
    int64_t m, k, n;
} gemm_q16_ctx;

enum { Q16_NC = 128 };

static void gemm_q16_band(void *vctx, int64_t rs, int64_t re) {
    gemm_q16_ctx *g = (gemm_q16_ctx *)vctx;
    const int64_t k = g->k, n = g->n;
    int64_t acc[Q16_NC];
    for (int64_t i = rs; i < re; ++i)
        for (int64_t jc = 0; jc < n; jc += Q16_NC) {
            int64_t nc = n - jc < Q16_NC ? n - jc : Q16_NC;
            for (int64_t j = 0; j < nc; ++j) acc[j] = 0;
            for (int64_t kk = 0; kk < k; ++kk) {
                const int64_t av = g->a[i * k + kk];
                const int32_t *brow = g->b + kk * n + jc;
                for (int64_t j = 0; j < nc; ++j) acc[j] += (av * (int64_t)brow[j]) >> 16;
            }
            for (int64_t j = 0; j < nc; ++j) g->c[i * n + jc + j] = (int32_t)acc[j];
        }
}

BASELINE_EXPORT int64_t baseline_gemm_q16_mt(const int32_t *a, const int32_t *b, int32_t *c,
                                             int64_t m, int64_t k, int64_t n, int64_t threads) {
    gemm_q16_ctx g = {a, b, c, m, k, n};
    return run_bands(gemm_q16_band, &g, m, threads);
}

/* ------------------------------ int16 GEMM -------------------------------- */
typedef struct {
    const int16_t *a, *b;
    int32_t *c;
    int64_t m, k, n;
} gemm_i16_ctx;

static void gemm_i16_band(void *vctx, int64_t rs, int64_t re) {
    gemm_i16_ctx *g = (gemm_i16_ctx *)vctx;
    const int64_t k = g->k, n = g->n;
    uint32_t acc[Q16_NC];
    for (int64_t i = rs; i < re; ++i)
        for (int64_t jc = 0; jc < n; jc += Q16_NC) {
            int64_t nc = n - jc < Q16_NC ? n - jc : Q16_NC;
            for (int64_t j = 0; j < nc; ++j) acc[j] = 0;
            for (int64_t kk = 0; kk < k; ++kk) {
                const int32_t av = g->a[i * k + kk];
                const int16_t *brow = g->b + kk * n + jc;
                for (int64_t j = 0; j < nc; ++j) acc[j] += (uint32_t)(av * (int32_t)brow[j]);
            }
            for (int64_t j = 0; j < nc; ++j) g->c[i * n + jc + j] = (int32_t)acc[j];
        }
}

BASELINE_EXPORT int64_t baseline_gemm_i16_mt(const int16_t *a, const int16_t *b, int32_t *c,
                                             int64_t m, int64_t k, int64_t n, int64_t threads) {
    gemm_i16_ctx g = {a, b, c, m, k, n};
    return run_bands(gemm_i16_band, &g, m, threads);
}

/* --------------------------------- GEMV ----------------------------------- */
typedef struct {
    const int32_t *w, *x;
    int32_t *y;
    int64_t cols;
} gemv_q16_ctx;

static void gemv_q16_band(void *vctx, int64_t rs, int64_t re) {
    gemv_q16_ctx *g = (gemv_q16_ctx *)vctx;
    for (int64_t r = rs; r < re; ++r) {
        const int32_t *row = g->w + r * g->cols;
        int64_t lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        int64_t i = 0;
        for (; i + 8 <= g->cols; i += 8)
            for (int l = 0; l < 8; ++l) lane[l] += ((int64_t)row[i + l] * (int64_t)g->x[i + l]) >> 16;
        int64_t acc = 0;
        for (int l = 0; l < 8; ++l) acc += lane[l];
        for (; i < g->cols; ++i) acc += ((int64_t)row[i] * (int64_t)g->x[i]) >> 16;
        g->y[r] = (int32_t)acc;
    }
}

BASELINE_EXPORT int64_t baseline_gemv_q16_mt(const int32_t *w, const int32_t *x, int32_t *y,
                                             int64_t rows, int64_t cols, int64_t threads) {
    gemv_q16_ctx g = {w, x, y, cols};
    return run_bands(gemv_q16_band, &g, rows, threads);
}

typedef struct {
    const int16_t *w, *x;
    int32_t *y;
    int64_t cols;
} gemv_i16_ctx;

static void gemv_i16_band(void *vctx, int64_t rs, int64_t re) {
    gemv_i16_ctx *g = (gemv_i16_ctx *)vctx;
    for (int64_t r = rs; r < re; ++r) {
        const int16_t *row = g->w + r * g->cols;
        uint32_t acc = 0;
        for (int64_t i = 0; i < g->cols; ++i) acc += (uint32_t)((int32_t)row[i] * (int32_t)g->x[i]);
        g->y[r] = (int32_t)acc;
    }
}

BASELINE_EXPORT int64_t baseline_gemv_i16_mt(const int16_t *w, const int16_t *x, int32_t *y,
                                             int64_t rows, int64_t cols, int64_t threads) {
    gemv_i16_ctx g = {w, x, y, cols};
    return run_bands(gemv_i16_band, &g, rows, threads);
}

/* ------------------------------------------------------------------------- *
 * The reference's OWN code as the timed baseline for the Q16.16 paths: rows are
 * computed by its `__mind_blas_dot_q16` (runtime-support/mind_intrinsics.c:1536-1547,
 * AVX2 when the host has it) and scheduled by its persistent pool
 * `__mind_blas_mt_dispatch` (:2017-2046) with its band rule
 * (src/mlir/lowering.rs:10146-10205).  Both functions are passed in as addresses
 * taken from the separately built reference library; nothing of it is compiled here.
 * The GEMM is composed from row dots over B-transposed, as the reference's own
 * gate composes it (tests/cross_substrate_identity.rs:82-94).
 * ------------------------------------------------------------------------- */
typedef int64_t (*ref_dot_fn)(int64_t, int64_t, int64_t);
typedef void (*ref_dispatch_fn)(void *(*)(void *), char *, long, long);

typedef struct {
    ref_dot_fn dot;
    const int32_t *w, *x;   /* GEMV: matrix, vector.  GEMM: A, B-transposed */
    int32_t *y;
    int64_t cols, n;        /* n == 0: GEMV; else GEMM with N = n */
    int64_t rs, re;
} ref_band;

static void *ref_band_worker(void *p) {
    ref_band *b = (ref_band *)p;
    for (int64_t r = b->rs; r < b->re; ++r) {
        const int32_t *row = b->w + r * b->cols;
        if (b->n == 0) {
            b->y[r] = (int32_t)b->dot((int64_t)(intptr_t)row, (int64_t)(intptr_t)b->x, b->cols);
        } else {
            for (int64_t j = 0; j < b->n; ++j)
                b->y[r * b->n + j] =
                    (int32_t)b->dot((int64_t)(intptr_t)row, (int64_t)(intptr_t)(b->x + j * b->cols), b->cols);
        }
    }
    return NULL;
}

static int64_t ref_run(void *dot, void *dispatch, const int32_t *w, const int32_t *x, int32_t *y,
                       int64_t rows, int64_t cols, int64_t n) {
    if (rows <= 0) return 0;
    int64_t ncpu = sysconf(_SC_NPROCESSORS_ONLN);
    int64_t upper = rows < 256 ? rows : 256;
    int64_t t = ncpu < upper ? ncpu : upper;
    if (t < 1) t = 1;
    int64_t band = (rows + t - 1) / t;
    ref_band jobs[256];
    int64_t used = 0;
    for (int64_t i = 0; i < t; ++i) {
        int64_t s = i * band, e = s + band;
        if (e > rows) e = rows;
        if (s >= e) break;
        jobs[used++] = (ref_band){(ref_dot_fn)dot, w, x, y, cols, n, s, e};
    }
    ((ref_dispatch_fn)dispatch)(ref_band_worker, (char *)jobs, (long)sizeof(ref_band), (long)used);
    return used;
}

BASELINE_EXPORT int64_t reference_gemv_q16_mt(void *dot, void *dispatch, const int32_t *w,
                                              const int32_t *x, int32_t *y, int64_t rows, int64_t cols) {
    return ref_run(dot, dispatch, w, x, y, rows, cols, 0);
}

BASELINE_EXPORT int64_t reference_gemm_q16_bt_mt(void *dot, void *dispatch, const int32_t *a,
                                                 const int32_t *bt, int32_t *c, int64_t m, int64_t k,
                                                 int64_t n) {
    return ref_run(dot, dispatch, a, bt, c, m, k, n);
}
