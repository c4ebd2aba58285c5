/*
 * mind_b200_native.c -- link-time definitions of MIND's deterministic BLAS intrinsics that
 * forward to libmind_b200.so (NVIDIA B200).
 *
 * How it is used.  A MIND project lists this file under `[targets.<name>].native_sources`
 * (src/project/mod.rs:525-540 of star-ga/mind): mindc compiles it with its own deterministic
 * clang invocation and links the object into the executable (src/project/mod.rs:1104-1135),
 * next to `-ldl -lpthread -lm`, which its Linux link line already carries
 * (src/project/link.rs:113-115).  Every `func.call @__mind_blas_*` that the lowering leaves as
 * an external call is then resolved by the definitions below.  They load libmind_b200.so on
 * first use -- from the path in the environment variable MIND_B200_LIB, else by the name
 * "libmind_b200.so" through the normal library search -- and forward the call unchanged: same
 * names, same i64 arguments, same meaning (include/mind_b200.h of the mind-b200 tree names the
 * reference file and line each one replaces).
 *
 * Nothing here computes.  If the library cannot be loaded, or has no usable GPU, the kernels
 * return a negative status (the library's MIND_B200_ERR_* codes; -3 = no device / no library)
 * and the dots return 0, as the reference's dot does on bad input
 * (runtime-support/mind_intrinsics.c:1538); mind_b200_native_last_error() gives the reason.
 * There is no CPU fallback on purpose: a caller that wants the CPU kernels simply does not
 * list this file.
 *
 * Plain C99 + POSIX (dlopen, pthread_once); no CUDA headers are needed to compile it.
 */
#include <dlfcn.h>
#include <pthread.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define MIND_B200_NATIVE_NO_LIBRARY (-3)

typedef int64_t (*fn6_t)(int64_t, int64_t, int64_t, int64_t, int64_t, int64_t);
typedef int64_t (*fn5_t)(int64_t, int64_t, int64_t, int64_t, int64_t);
typedef int64_t (*fn3_t)(int64_t, int64_t, int64_t);
typedef const char *(*err_t)(void);

static struct {
    void *handle;
    fn6_t mm_i8, mm_i8_mt, mm_q16, mm_q16_mt, mm_i16;
    fn5_t gemv_q16_mt, rmajor_q16, rmajor_i16;
    fn3_t dot_q16, dot_l1_q16, dot_i16;
    err_t last_error;
    char load_error[512];
} g_b200;

static pthread_once_t g_b200_once = PTHREAD_ONCE_INIT;

static void *b200_sym(const char *name) {
    void *p = dlsym(g_b200.handle, name);
    if (!p && !g_b200.load_error[0])
        snprintf(g_b200.load_error, sizeof g_b200.load_error, "libmind_b200: missing symbol %s", name);
    return p;
}

static void b200_load(void) {
    const char *path = getenv("MIND_B200_LIB");
    if (!path || !*path) path = "libmind_b200.so";
    g_b200.handle = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (!g_b200.handle) {
        const char *why = dlerror();
        snprintf(g_b200.load_error, sizeof g_b200.load_error, "cannot load %s: %s", path, why ? why : "unknown error");
        return;
    }
    g_b200.mm_i8 = (fn6_t)b200_sym("__mind_blas_matmul_mm_i8_v");
    g_b200.mm_i8_mt = (fn6_t)b200_sym("__mind_blas_matmul_mm_i8_mt_v");
    g_b200.mm_q16 = (fn6_t)b200_sym("__mind_blas_matmul_mm_q16_v");
    g_b200.mm_q16_mt = (fn6_t)b200_sym("__mind_blas_matmul_mm_q16_mt_v");
    g_b200.mm_i16 = (fn6_t)b200_sym("__mind_b200_matmul_mm_i16");
    g_b200.gemv_q16_mt = (fn5_t)b200_sym("__mind_blas_gemv_q16_mt");
    g_b200.rmajor_q16 = (fn5_t)b200_sym("__mind_blas_matmul_rmajor_q16_v");
    g_b200.rmajor_i16 = (fn5_t)b200_sym("__mind_blas_matmul_rmajor_i16_v");
    g_b200.dot_q16 = (fn3_t)b200_sym("__mind_blas_dot_q16_v");
    g_b200.dot_l1_q16 = (fn3_t)b200_sym("__mind_blas_dot_l1_q16_v");
    g_b200.dot_i16 = (fn3_t)b200_sym("__mind_blas_dot_i16_v");
    g_b200.last_error = (err_t)b200_sym("mind_b200_last_error");
}

static int b200_ready(void) {
    pthread_once(&g_b200_once, b200_load);
    return g_b200.handle && !g_b200.load_error[0];
}

/* Why the last call of this thread's library failed, or why the library could not be loaded;
 * NULL when there is nothing to report. */
const char *mind_b200_native_last_error(void) {
    pthread_once(&g_b200_once, b200_load);
    if (g_b200.load_error[0]) return g_b200.load_error;
    return g_b200.last_error ? g_b200.last_error() : NULL;
}

#define FORWARD6(name, slot)                                                                        \
    int64_t name(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n) {                \
        return b200_ready() ? g_b200.slot(a, b, c, m, k, n) : MIND_B200_NATIVE_NO_LIBRARY;          \
    }
#define FORWARD5(name, slot)                                                                        \
    int64_t name(int64_t w, int64_t x, int64_t y, int64_t rows, int64_t cols) {                     \
        return b200_ready() ? g_b200.slot(w, x, y, rows, cols) : MIND_B200_NATIVE_NO_LIBRARY;       \
    }
#define FORWARD3(name, slot)                                                                        \
    int64_t name(int64_t a, int64_t b, int64_t len) { return b200_ready() ? g_b200.slot(a, b, len) : 0; }

/* int8 GEMM: src/mlir/lowering.rs:7687-7752 and its _mt twin :10368 */
FORWARD6(__mind_blas_matmul_mm_i8_v, mm_i8)
FORWARD6(__mind_blas_matmul_mm_i8_mt_v, mm_i8_mt)
/* Q16.16 GEMM: src/mlir/lowering.rs:9300-9407 and :10019-10341 */
FORWARD6(__mind_blas_matmul_mm_q16_v, mm_q16)
FORWARD6(__mind_blas_matmul_mm_q16_mt_v, mm_q16_mt)
/* int16 GEMM: no counterpart in the reference (new name) */
FORWARD6(__mind_b200_matmul_mm_i16, mm_i16)
/* Q16.16 GEMV and row-major matrix x vector: src/mlir/lowering.rs:10019-10032, :6675, :10723 */
FORWARD5(__mind_blas_gemv_q16_mt, gemv_q16_mt)
FORWARD5(__mind_blas_matmul_rmajor_q16_v, rmajor_q16)
FORWARD5(__mind_blas_matmul_rmajor_i16_v, rmajor_i16)
/* dots: src/mlir/lowering.rs:5695-5830, :6057, :5861-6033 */
FORWARD3(__mind_blas_dot_q16_v, dot_q16)
FORWARD3(__mind_blas_dot_l1_q16_v, dot_l1_q16)
FORWARD3(__mind_blas_dot_i16_v, dot_i16)
