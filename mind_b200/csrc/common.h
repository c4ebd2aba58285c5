// Host-side plumbing shared by every translation unit of libmind_b200:
// status codes, the thread-local error message, the per-device context (stream,
// scratch arena, device error word) and the launch counter.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <atomic>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/mind_b200.h"

namespace mb200 {

// Sets the calling thread's error message and returns `code`.
int64_t fail(int64_t code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
void clear_error();
const char* last_error_cstr();
long long launches();
int usable_device_count();

// Process-wide kernel-choice knobs (mind_b200_set_gemm_path and friends).  They exist for tests
// and measurements; each is an atomic read once per call, so a setter running beside a call on
// another thread is a benign race: that call uses either the old or the new value, and every
// value gives the same bytes.
struct Tuning {
    std::atomic<int> gemm_path{0};        // 0 = tensor cores, 1 = CUDA-core cross-check kernels
    std::atomic<int> force_transpose{0};  // tensor cores: always re-lay B out K-contiguous
    std::atomic<int> q16_mode{0};         // Q16.16 GEMM: 0 = by size, 6 = FP64-pipe kernel alone, 7 = hybrid
    std::atomic<int> q16_fused{1};        // hybrid: 1 = one fused kernel where it can run, 0 = the two-kernel forms
    std::atomic<int> q16_floor{0};        // hybrid: the per-product floor on 0 = the FP32 pipe (low halves), 1 = the FP64 pipe
    std::atomic<int> q16_side_sms{-1};    // hybrid: SMs of the tensor-core half beside the FP64 half (-1 = by size)
    std::atomic<int> pair_mode{0};        // CTAs per int8 tile: 1, 2, or 0 = pick per call
    std::atomic<int> small_tile{-1};      // int8 GEMM narrow-tile kernel: -1 = by shape, 0 = never, 1 = always
    std::atomic<int> wide_pair{-1};       // int8 GEMM 256 x 512-tile pair kernel: -1 = by shape, 0 = never, 1 = always
    std::atomic<int> group_m{0};          // int8 tile order: m-tiles per group (0 = default)
    std::atomic<int> raster{0};           // int8 tile order variant (0 = default)
};
Tuning& tuning();

#define MB200_CUDA(expr)                                                                   \
    do {                                                                                   \
        cudaError_t _e = (expr);                                                           \
        if (_e != cudaSuccess)                                                             \
            return ::mb200::fail(MIND_B200_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,       \
                                 cudaGetErrorString(_e), __FILE__, __LINE__);              \
    } while (0)

#define MB200_TRY(expr)            \
    do {                           \
        int64_t _s = (expr);       \
        if (_s != 0) return _s;    \
    } while (0)

// Grow-only device scratch: one allocation per device, reused by every call on
// that device (calls on one device are serialised by the context lock).
struct Arena {
    char* base = nullptr;
    size_t cap = 0;
    size_t used = 0;
};

// Streams and events of the host-operand pipelines (copies run beside the kernels): made on
// first use, per device, and kept.
struct Pipe {
    cudaStream_t in = nullptr, out = nullptr;
    cudaEvent_t start = nullptr, gemm_done[2] = {}, out_done[2] = {};
    cudaEvent_t b_ready = nullptr;   // multi-device calls: this device's share of B has reached every peer
    std::vector<cudaEvent_t> ready;  // uploads: A bands, then B chunks
    bool made = false;
};

struct DeviceCtx {
    int device = -1;
    int sm_count = 0;
    // Calls on one device are serialised by this lock (they share the arenas and the side
    // streams); calls on different devices run side by side.
    std::mutex mu;
    cudaStream_t stream = nullptr;  // the stream every launch and copy goes to
    Arena scratch;                  // operand re-layouts (transposed B, limb planes, padded A)
    Arena staging;                  // device copies of host-pointer operands
    // Once a stream capture has been seen on this device, outgrown arena blocks are kept (a
    // captured graph may still hold their addresses) and only freed at shutdown.
    bool capture_seen = false;
    std::vector<void*> retired;
    cudaEvent_t order_ev = nullptr;  // orders a new library stream after the old one (set_stream)
    Pipe pipe;
    int* err_word = nullptr;        // word a kernel sets when a bounded wait runs out (device view)
    int* err_host = nullptr;        // the same word, host view (mapped pinned memory)
    int* scalar_host = nullptr;     // where a kernel leaves a scalar result for the host (mapped pinned memory)
    int32_t* scalar_dev = nullptr;  // the same word, device view
    // A second stream for work that runs beside the kernels on `stream` inside one call (forked
    // and joined with the two events).
    cudaStream_t side = nullptr;
    cudaEvent_t fork_ev = nullptr, join_ev = nullptr;
    // Optional timing of the main kernel of each call (CUDA events on `stream`).
    static constexpr int PROF_RING = 512;
    bool profile = false;
    int prof_count = 0;
    cudaEvent_t prof_ev[2 * PROF_RING] = {};
};

// Bracket the dominant kernel of a call; no-ops unless profiling is on.
void prof_begin(DeviceCtx* ctx);
void prof_end(DeviceCtx* ctx);

// Context of the CURRENT device (created on first use); nullptr + error set on failure.
DeviceCtx* current_ctx();
// Frees everything the library holds on every device (arenas, streams, events, mapped words).
// Safe to call more than once; the contexts are rebuilt on the next call.
void destroy_all_contexts();

// Bump-allocates `bytes` (1024-byte aligned) from an arena, growing it if needed.
// Growing replaces the block (after a stream sync), so pointers handed out earlier in
// the same call must be re-derived: reserve the total first.  Growth is refused while the
// library's stream is being captured (it would need cudaMalloc and a synchronisation).
int64_t arena_reserve(DeviceCtx* ctx, Arena& a, size_t total_bytes);
void* arena_take(Arena& a, size_t bytes);
inline void arena_reset(Arena& a) { a.used = 0; }
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---- host-operand pipelines and multi-device dispatch (abi.cu, multi.cu) ----
int64_t pipe_for(DeviceCtx* ctx, size_t n_ready, Pipe** out);
int64_t check_err_word(DeviceCtx* ctx);
// 1 = host memory, 0 = memory of ctx's device, negative = error (memory of another device).
int64_t pointer_is_host(DeviceCtx* ctx, const void* p);
// Returned by the multi_* functions when the call should run on the current device alone.
constexpr int64_t MULTI_NOT_TAKEN = INT64_MIN;
int multi_device_count();
int64_t multi_set_devices(int64_t count);
void multi_shutdown();
// int8 GEMM with host operands over several devices: device g owns row band g of A and C; B
// goes up once in K-slices, one per device, and the devices pass the slices on to each other.
int64_t multi_gemm_i8(const int8_t* a, const int8_t* b, int32_t* c, int64_t m, int64_t k, int64_t n);
// Any row-banded call with host operands: `band(a_band, c_band, rows)` runs on each device with
// that device current (a: rows of a_row_bytes, c: rows of c_row_bytes, `shared` is read by all).
int64_t multi_banded(const void* a, size_t a_row_bytes, const void* shared, size_t shared_bytes, void* c,
                     size_t c_row_bytes, int64_t m,
                     const std::function<int64_t(const void*, void*, int64_t)>& band);

// ---- pageable host operands through pinned slots (staging.cu) ----
// A set of chunk copies handed to the staging threads; `last` runs on whichever thread finishes
// the set (it records the CUDA event the consumers wait for), wait() blocks the submitting
// thread until that has happened.  A group that was never armed counts as done.
struct StageGroup {
    std::mutex mu;
    std::condition_variable cv;
    int left = 0;
    bool done = true;
    std::function<void()> last;
    void arm(int chunks, std::function<void()> on_last);
    void finish_one();
    void wait();
};
struct StageStatus {
    std::atomic<int> failed{0};
    void fail(const char*) { failed = 1; }
};
bool stager_start();     // pins the slots and starts the threads (first pageable call); false if it cannot
size_t stager_slot_bytes();  // a staged row (its device pitch) must fit one slot
void stager_drain();     // every chunk submitted so far has reached its destination
void stager_shutdown();
bool host_pointer_is_pageable(const void* p);
void stage_upload(int device, char* dst, size_t dpitch, const char* src, size_t spitch, size_t width, size_t rows,
                  cudaStream_t stream, StageGroup* group, std::function<void()> on_last, StageStatus* status);
void stage_download(int device, char* dst, const char* src, size_t bytes, cudaStream_t stream, StageGroup* group,
                    std::function<void()> on_last, StageStatus* status);

// Kernel launch accounting (reported through mind_b200_kernel_launches()).
void count_launch(int n = 1);

// Checks the launch status of the last kernel and the device error word policy.
int64_t check_launch(const char* what);

// cuTensorMapEncodeTiled, resolved through the runtime (no link-time libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();
// Tensor map over a row-major 8-bit matrix [rows][k] (row pitch in bytes): boxes of box_bytes (128
// or 64, = the swizzle width) along k by box_rows rows.  Cached per thread (gemm_tc.cu).
int64_t make_tmap_u8(CUtensorMap* tm, const void* base, int64_t k, int64_t rows, int64_t pitch, int box_rows,
                     int box_bytes);
// Tensor map over the int32 output c[m][n] (16-byte aligned, n % 4 == 0): boxes of 32 x 32 elements in
// the 128-byte swizzle, for tensor stores / reductions from shared memory.
int64_t make_tmap_c32(CUtensorMap* tm, int32_t* c, int64_t n, int64_t m);

// ---- kernels' host launchers (device pointers only, asynchronous on ctx->stream) ----
// int8 GEMM on tensor cores: C[M,N] (i32) = A[M,K] . Bt[N,K]^T, both operands
// K-contiguous with row pitch `kp` bytes (kp % 16 == 0, bases 16-byte aligned).
int64_t launch_gemm_i8_tc(DeviceCtx* ctx, const int8_t* a, const int8_t* bt, int32_t* c, int64_t m,
                          int64_t n, int64_t k, int64_t kp_a, int64_t kp_b);
// int16 GEMM as four 8-bit limb products on tensor cores; operands are limb planes: A high
// (signed) / low (unsigned), B high (signed) / low minus 128 (signed), and the int32 row sums
// of A, which put the 128 back.
int64_t launch_gemm_i16_tc(DeviceCtx* ctx, const int8_t* a_hi, const uint8_t* a_lo,
                           const int8_t* bt_hi, const uint8_t* bt_lo, const int32_t* a_row_sums,
                           int32_t* c, int64_t m, int64_t n, int64_t k, int64_t kp);
// Same products with B used as the caller has it (B[K][N], row pitch `pitch_b` bytes,
// pitch_b % 16 == 0, base 16-byte aligned): no transpose pass.
int64_t launch_gemm_i8_tc_bmn(DeviceCtx* ctx, const int8_t* a, const int8_t* b, int32_t* c, int64_t m,
                              int64_t n, int64_t k, int64_t kp_a, int64_t pitch_b);
int64_t launch_gemm_i16_tc_bmn(DeviceCtx* ctx, const int8_t* a_hi, const uint8_t* a_lo,
                               const int8_t* b_hi, const uint8_t* b_lo, const int32_t* a_row_sums,
                               int32_t* c, int64_t m, int64_t n, int64_t k, int64_t kp_a, int64_t pitch_b);
bool tc_pair_forced();
// Q16.16 hybrid: byte planes of an int32 matrix (what = 0: all four bytes; 1: the two bytes
// of element >> 16), and the tensor-core product of those planes (see gemm_tc.cu).
int64_t launch_split_i32_bytes(DeviceCtx* ctx, const int32_t* src, uint8_t* const planes[4], int what,
                               int64_t rows, int64_t cols, int64_t pitch);
int64_t launch_gemm_q16_linear_tc(DeviceCtx* ctx, const uint8_t* const a_limb[4], const uint8_t* const b_limb[4],
                                  int32_t* p_out, int64_t m, int64_t n, int64_t k, int64_t kp_a,
                                  int64_t pitch_b, bool accumulate, int max_ctas);
// The per-product floor term of the low halves on the FP32 pipe, added onto c (gemm_q16_f32.cu).
int64_t launch_gemm_q16_floor_f32(DeviceCtx* ctx, const int32_t* a, const int32_t* b, int32_t* c, int64_t m,
                                  int64_t k, int64_t n, int max_blocks);
int64_t measure_fp32_fma_peak(DeviceCtx* ctx, double* fma_per_s, double* sm_mhz);
// The fused form (gemm_q16_fused.cu): limb products and floor term in one kernel.  a_low_t /
// b_low are the binary32 planes launch_split_q16_ab writes; c must be zero where tiles are shared.
bool gemm_q16_fused_usable(DeviceCtx* ctx);
int64_t launch_gemm_q16_fused(DeviceCtx* ctx, const uint8_t* const a_limb[4], const uint8_t* const b_limb[4],
                              const float* a_low_t, const float* b_low, int32_t* c, int64_t m, int64_t n, int64_t k,
                              int64_t kp_a, int64_t pitch_b, int64_t mp, int64_t np);
// One launch that prepares everything the fused kernel reads (prep.cu: split_q16_ab_kernel):
// a[m][k] -> its four byte planes [m][kp] and (a & 0xffff) as binary32, transposed: a_low_t[k][mp]
// (mp % 4 == 0, mp >= m); b[k][n] -> the byte planes of b >> 16 (bp[0..1]) and of b & 0xffff
// (bp[2..3]), [k][np], and (b & 0xffff) * 2^-16 as binary32, b_low[k][np]; zero_c: c[m][n] = 0.
// k % 4 == 0, n % 4 == 0, 16-byte aligned a, b (and c when zeroed).
int64_t launch_split_q16_ab(DeviceCtx* ctx, const int32_t* a, const int32_t* b, uint8_t* const ap[4],
                            uint8_t* const bp[4], float* a_low_t, float* b_low, int32_t* c, bool zero_c, int64_t m,
                            int64_t k, int64_t n, int64_t kp, int64_t np, int64_t mp);
// Whether the fused kernel will add onto c for this shape (some tile is shared between CTAs), so c must start at zero.
bool gemm_q16_fused_shares_tiles(DeviceCtx* ctx, int64_t m, int64_t n, int64_t k);

// Low halves of Q16.16 operands as binary32, exactly, without the integer-to-float unit: the
// 16-bit value is or-ed into the mantissa of 2^23 and 2^23 taken off again.
constexpr uint32_t Q16_TWO23_BITS = 0x4B000000u;  // binary32 2^23: the low 23 bits are an integer field
__device__ __forceinline__ float q16_low_half_f32(int32_t v) {  // (v & 0xffff)
    return __uint_as_float(Q16_TWO23_BITS | ((uint32_t)v & 0xffffu)) - 8388608.0f;
}
__device__ __forceinline__ float q16_low_half_scaled_f32(int32_t v) {  // (v & 0xffff) * 2^-16: (2^23 + bl) * 2^-16 - 2^7
    return __fmaf_rn(__uint_as_float(Q16_TWO23_BITS | ((uint32_t)v & 0xffffu)), 1.52587890625e-05f, -128.0f);
}
// Floor part of the Q16.16 product on the FP64 pipe, added onto the linear part already in c.
int64_t launch_gemm_q16_floor_add(DeviceCtx* ctx, const int32_t* a, const int32_t* b, int32_t* c, int64_t m,
                                  int64_t k, int64_t n, int max_blocks);
int64_t launch_wait_selftest(DeviceCtx* ctx, int64_t limit_ms);
// Re-layout kernels.
int64_t launch_transpose_i8(DeviceCtx* ctx, const int8_t* b, int8_t* bt, int64_t k, int64_t n,
                            int64_t kp);
int64_t launch_transpose_i32(DeviceCtx* ctx, const int32_t* src, int32_t* dst, int64_t rows,
                             int64_t cols);
int64_t launch_pad_rows_i8(DeviceCtx* ctx, const int8_t* a, int8_t* ap, int64_t m, int64_t k,
                           int64_t kp);
// lo_minus_128: store the low plane minus 128 (the B operand); row_sums: if not null, receives
// the int32 sum of every row (the A operand; sums_are_zero says an earlier launch cleared it);
// zero_buf / zero_n: a buffer this launch clears on the way (the next launch's row sums).
int64_t launch_split_rows_i16(DeviceCtx* ctx, const int16_t* a, int8_t* hi, uint8_t* lo, int64_t m,
                              int64_t k, int64_t kp, bool lo_minus_128, int32_t* row_sums, bool sums_are_zero,
                              int32_t* zero_buf, int64_t zero_n);
// Both operands of the int16 GEMM in one launch (dense rows, K % 16 == 0, N % 16 == 0, aligned bases).
bool split_i16_pair_usable(const int16_t* a, int64_t k, const int16_t* b, int64_t n);
int64_t launch_split_i16_pair(DeviceCtx* ctx, const int16_t* a, int8_t* a_hi, uint8_t* a_lo, int32_t* a_row_sums,
                              int64_t m, int64_t k, const int16_t* b, int8_t* b_hi, uint8_t* b_lo, int64_t n);
int64_t launch_split_transpose_i16(DeviceCtx* ctx, const int16_t* b, int8_t* bt_hi, uint8_t* bt_lo,
                                   int64_t k, int64_t n, int64_t kp);
// CUDA-core kernels.
int64_t launch_gemm_q16(DeviceCtx* ctx, const int32_t* a, const int32_t* b, int32_t* c, int64_t m,
                        int64_t k, int64_t n);
// Q16.16 GEMM with the per-product floor on the FP64 pipe (needs aligned, 4-divisible shapes).
bool gemm_q16_fp64_usable(const int32_t* a, const int32_t* b, int64_t k, int64_t n);
int64_t launch_gemm_q16_fp64(DeviceCtx* ctx, const int32_t* a, const int32_t* b, int32_t* c, int64_t m,
                             int64_t k, int64_t n);
int64_t launch_gemm_i8_simt(DeviceCtx* ctx, const int8_t* a, const int8_t* b, int32_t* c, int64_t m,
                            int64_t k, int64_t n);
int64_t launch_gemm_i16_simt(DeviceCtx* ctx, const int16_t* a, const int16_t* b, int32_t* c,
                             int64_t m, int64_t k, int64_t n);
int64_t launch_gemv_q16(DeviceCtx* ctx, const int32_t* w, const int32_t* x, int32_t* y,
                        int64_t rows, int64_t cols);
int64_t launch_gemv_i16(DeviceCtx* ctx, const int16_t* w, const int16_t* x, int32_t* y,
                        int64_t rows, int64_t cols);
int64_t launch_dist_l1_q16(DeviceCtx* ctx, const int32_t* a, const int32_t* b, int32_t* out,
                           int64_t len);
int64_t launch_lcg_fill(DeviceCtx* ctx, void* dst, int64_t n, int kind, uint64_t seed,
                        uint64_t offset, int shift);
int64_t measure_fp64_fma_peak(DeviceCtx* ctx, double* fma_per_s, double* sm_mhz);
int64_t launch_matvec_wrap(DeviceCtx* ctx, const void* mat, int elem_bytes, int64_t rows,
                           int64_t cols, const int32_t* v, int32_t* out);

}  // namespace mb200
