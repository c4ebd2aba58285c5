/*
 * mind_b200.h -- C ABI of libmind_b200: MIND's deterministic integer BLAS
 * (int8 / int16 / Q16.16 GEMM, GEMV, dot) on NVIDIA B200 (sm_100a).
 *
 * Every entry point follows the calling convention of MIND's `__mind_blas_*`
 * compiler intrinsics: all arguments and the result are int64_t, pointers are raw
 * addresses cast to int64_t, matrices are dense row-major without a leading-
 * dimension argument, B is the UN-transposed K x N operand, the caller owns every
 * buffer and the output is fully overwritten.  Citations name files of the
 * reference project (star-ga/mind) whose interface each symbol replaces.
 *
 * Pointers may be HOST addresses (the reference's semantics: the call copies the
 * operands to the GPU, computes, copies the result back and returns when it is in
 * place) or DEVICE addresses of the current CUDA device (the call only enqueues
 * work on the library's stream, see mind_b200_set_stream; the result is complete in
 * stream order).  Each pointer of a call is classified on its own, so host and
 * device operands may be mixed; a call with any host pointer is synchronous.
 *
 * Several GPUs: like the reference's `_mt` entry points, which spread one call over the
 * host's cores, a call whose operands are all HOST buffers is spread over the GPUs named
 * by the environment variable MINDB200_DEVICES (a count, "4", or a list, "0,2,3"; default
 * 1) or by mind_b200_set_devices: contiguous owner-computes bands of the M output rows,
 * one per device, no reduction between them, so the bytes do not depend on the device
 * count.  Calls with device pointers always run on the current device alone.
 *
 * Results are bit-identical to the reference's rules: exact 64-bit sums truncated
 * once to int32 (two's-complement wrap, never saturation); Q16.16 products are
 * shifted right by 16 (arithmetic) BEFORE they are added.
 *
 * Errors: kernels return 0 on success, as the reference's do.  On failure they
 * return a negative MIND_B200_ERR_* code, never abort, and leave a message for
 * mind_b200_last_error() (thread-local, like mind_last_error in src/ffi/mod.rs:172-181
 * of the reference).  There is no CPU fallback: without a usable B200 every compute
 * entry point fails with MIND_B200_ERR_NO_DEVICE.  The dot entry points return the
 * dot value itself, so they report failure only through mind_b200_last_error()
 * (and return 0, as the reference's dot does on bad input,
 * runtime-support/mind_intrinsics.c:1538).
 */
#ifndef MIND_B200_H
#define MIND_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MIND_B200_OK 0
#define MIND_B200_ERR_INVALID (-1)    /* null pointer with non-empty shape, negative size, ... */
#define MIND_B200_ERR_CUDA (-2)       /* a CUDA runtime / driver call failed                  */
#define MIND_B200_ERR_NO_DEVICE (-3)  /* no CUDA device, or the device is not sm_100           */
#define MIND_B200_ERR_TIMEOUT (-4)    /* a bounded in-kernel wait ran out; result is invalid   */
#define MIND_B200_ERR_TOO_LARGE (-5)  /* shape beyond a documented limit                       */

/* ---- int8 GEMM:  C[i,j] = (i32) sum_k (i64)A[i,k] * (i64)B[k,j] -------------------------
 * a: M x K int8, b: K x N int8, c: M x N int32.
 * Replaces __mind_blas_matmul_mm_i8_v (src/mlir/lowering.rs:7687-7752, registry
 * src/type_checker/mod.rs:2304) and its multithreaded twin __mind_blas_matmul_mm_i8_mt_v
 * (src/mlir/lowering.rs:10368, registry :2310); the two are the same kernel here. */
int64_t __mind_blas_matmul_mm_i8_v(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n);
int64_t __mind_blas_matmul_mm_i8_mt_v(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n);

/* ---- Q16.16 GEMM:  C[i,j] = (i32) sum_k ( ((i64)A[i,k] * (i64)B[k,j]) >> 16 ) -----------
 * a, b, c: int32 holding Q16.16.  Replaces __mind_blas_matmul_mm_q16_v
 * (src/mlir/lowering.rs:9300-9407, registry src/type_checker/mod.rs:2316) and
 * __mind_blas_matmul_mm_q16_mt_v (src/mlir/lowering.rs:10019-10341, registry :2322). */
int64_t __mind_blas_matmul_mm_q16_v(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n);
int64_t __mind_blas_matmul_mm_q16_mt_v(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n);

/* ---- Q16.16 GEMV:  scores[i] = (i32) sum_k ( (catalog[i,k] * query[k]) >> 16 ) -----------
 * Replaces __mind_blas_gemv_q16_mt (src/mlir/lowering.rs:10019-10032, :9822-9996, registry
 * src/type_checker/mod.rs:2332) and __mind_blas_matmul_rmajor_q16_v (src/mlir/lowering.rs:6675,
 * registry :2294): same rule, same argument order (matrix, vector, out, rows, cols). */
int64_t __mind_blas_gemv_q16_mt(int64_t catalog, int64_t query, int64_t scores, int64_t m, int64_t k);
int64_t __mind_blas_matmul_rmajor_q16_v(int64_t w, int64_t x, int64_t y, int64_t rows, int64_t cols);

/* ---- int16 GEMV:  y[r] = (i32) sum_i (i64)W[r,i] * (i64)x[i]  (no shift) ------------------
 * Replaces __mind_blas_matmul_rmajor_i16_v (src/mlir/lowering.rs:10723, registry
 * src/type_checker/mod.rs:2285). */
int64_t __mind_blas_matmul_rmajor_i16_v(int64_t w, int64_t x, int64_t y, int64_t rows, int64_t cols);

/* ---- dots: return (i64)(i32)acc -------------------------------------------------------------
 * __mind_blas_dot_q16_v     src/mlir/lowering.rs:5695-5830, registry src/type_checker/mod.rs:2271
 *                           (same value as __mind_blas_dot_q16, runtime-support/mind_intrinsics.c:1459-1547)
 * __mind_blas_dot_l1_q16_v  src/mlir/lowering.rs:6057, registry :2260: sum |a[i] - b[i]|
 * __mind_blas_dot_i16_v     src/mlir/lowering.rs:5861-6033, registry :2246 */
int64_t __mind_blas_dot_q16_v(int64_t a, int64_t b, int64_t len);
int64_t __mind_blas_dot_l1_q16_v(int64_t a, int64_t b, int64_t len);
int64_t __mind_blas_dot_i16_v(int64_t a, int64_t b, int64_t len);

/* ---- int16 GEMM:  C[i,j] = (i32) sum_k (i64)A[i,k] * (i64)B[k,j] -------------------------
 * The reference has NO int16 GEMM; this composes its int16 row rule
 * (benches/det_matmul_i16.rs:218-231, src/mlir/lowering.rs:5861) over the columns of an
 * un-transposed K x N B, the layout of its int8 and Q16.16 GEMMs.  New symbol name. */
int64_t __mind_b200_matmul_mm_i16(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n);

/* ---- int8 GEMM that allocates nothing -----------------------------------------------------------
 * This entry point has no counterpart in the reference.  It is for hosts that cannot call
 * cudaMalloc when they need the product: a serving loop in which an allocation (and the device
 * synchronisation it may bring) is not allowed, or a process whose GPU memory is wholly owned
 * by another allocator.  Same rule, same kernels and same bytes as __mind_blas_matmul_mm_i8_v,
 * but the operand copies that call keeps in a buffer grown with cudaMalloc - B transposed, when
 * N % 16 != 0 or B is not 16-byte aligned; A padded, when K % 16 != 0 or A is not 16-byte
 * aligned - live in a fixed array inside the library image, and no per-device context is
 * created.  It calls no cudaMalloc, cudaFree, cudaMallocHost or other allocating routine.
 *   - a, b, c must be DEVICE pointers of the current device (host operands would need staging
 *     memory); cuda_stream is the stream to run on (0 = legacy default stream).
 *   - limit: (N*ceil16(K) if B needs transposing) + (M*ceil16(K) if A needs padding), each
 *     rounded up to 256 bytes, must not exceed MIND_B200_STATIC_SCRATCH_BYTES, else
 *     MIND_B200_ERR_TOO_LARGE; operands that TMA can read in place need no room.  Every GPU
 *     that loads the library holds that array until the process exits.
 *   - it is an ordinary synchronous host call: it waits for its own work (also when it fails
 *     half way) and reports a kernel time-out itself.  Do not call it from a CUDA host callback
 *     (cudaLaunchHostFunc), where CUDA calls are forbidden, nor on a stream being captured.
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress);
 *     make that first call before starting any stream capture on that device.
 *   - all calls share the one array, which keeps the previous call's contents (each call
 *     rewrites what it reads and zeroes its error word first).  Two calls overlapping on the
 *     GPU would race on it; inside one process a lock and the final wait rule that out, and
 *     every process has its own copy of the array. */
#define MIND_B200_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
int64_t mind_b200_matmul_mm_i8_static(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n,
                                      int64_t cuda_stream);

/* ---- names of the reference's identity-gate library -----------------------------------------
 * The gate compiles a MIND source whose public functions wrap the intrinsics
 * (tests/cross_substrate_identity.rs:69-144) and its drivers dlsym these names
 * (tests/cross_substrate_identity/xnode_driver.c:148-156).  Exported so that the unmodified
 * driver runs against this library.  NOTE gemmq takes B TRANSPOSED (N x K), as the gate's does
 * (:82-94); gemmqmm and gemmq_kn take the un-transposed K x N B. */
int64_t dotq(int64_t a, int64_t b, int64_t n);
int64_t dotl1q(int64_t a, int64_t b, int64_t n);
int64_t doti16(int64_t a, int64_t b, int64_t n);
int64_t mmq(int64_t w, int64_t x, int64_t y, int64_t rows, int64_t cols);
int64_t mmi16(int64_t w, int64_t x, int64_t y, int64_t rows, int64_t cols);
int64_t gemvq(int64_t catalog, int64_t query, int64_t scores, int64_t m, int64_t k);
int64_t gemmq(int64_t a, int64_t bt, int64_t c, int64_t m, int64_t k, int64_t n);
int64_t gemmq_kn(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n);
int64_t gemmqmm(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n);
int64_t gemmi8(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n);
int64_t gemmi8mt(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n);

/* ---- library control (no counterpart in the reference's intrinsic surface) -------------------- */
/* Message of the calling thread's last failure, or NULL (src/ffi/mod.rs:172-181). */
const char* mind_b200_last_error(void);
/* CUDA stream (cudaStream_t cast to int64_t; 0 = the legacy default stream) that every later
 * call on the CURRENT device uses.  Default: the legacy default stream.  Device-pointer calls
 * are asynchronous and share one scratch buffer per device, so the new stream is made to wait
 * (by an event) for whatever the library has queued on the old one.  That ordering cannot be
 * set up while either stream is being captured: there, synchronise before switching. */
int64_t mind_b200_set_stream(int64_t cuda_stream);
/* Blocks until the library's stream on the current device is idle; reports a kernel
 * time-out recorded since the last call (MindRuntime::synchronize, src/runtime_interface.rs:41). */
int64_t mind_b200_synchronize(void);
/* Number of usable (sm_100) devices; 0 when none, never an error. */
int64_t mind_b200_device_count(void);
/* Kernels launched by this library in this process so far. */
int64_t mind_b200_kernel_launches(void);
/* Pre-sizes the current device's scratch (operand re-layouts) and staging (host operands)
 * buffers so that later calls allocate nothing.  CUDA graphs: a captured call records the
 * scratch addresses it was given, so reserve the largest size (or run the largest shapes once)
 * BEFORE capturing.  A call that would have to grow a buffer while its stream is being captured
 * is refused with MIND_B200_ERR_INVALID (growing needs cudaMalloc and a wait); after a capture
 * has been seen on a device, outgrown buffers are kept alive until mind_b200_shutdown, so that
 * graphs captured earlier stay valid. */
int64_t mind_b200_reserve(int64_t scratch_bytes, int64_t staging_bytes);
/* How many GPUs a host-operand call may be spread over (1 = the current device only); overrides
 * MINDB200_DEVICES.  The devices are ordinals 0 .. count-1 unless the variable gave a list.
 * One persistent host thread per device is started on first use (the reference's pool does the
 * same for cores, runtime-support/mind_intrinsics.c:1956-2046); fork() after that is unsupported. */
int64_t mind_b200_set_devices(int64_t count);
int64_t mind_b200_devices(void);
/* Joins the device threads and frees everything the library holds on every GPU (scratch and
 * staging buffers, streams, events, pinned words).  Also run by the library's destructor on
 * dlclose() / exit, as the reference's runtime joins its pool
 * (runtime-support/mind_intrinsics.c:2065-2081).  The library stays usable: the next call
 * rebuilds what it needs.  No call may be in flight on another thread. */
int64_t mind_b200_shutdown(void);
/* Which kernel the int8 / int16 GEMMs use: 0 = tensor cores (tcgen05), the library picks
 * between its two kernels per call (default); 2 = tensor cores, one output tile per pair of
 * CTAs (cta_group::2); 3 = tensor cores, one CTA per tile; 4 / 5 = as 2 / 3 but B is always
 * transposed into scratch first (otherwise B is read in place whenever its pitch and base are
 * 16-byte aligned); 1 = the independent CUDA-core kernels kept as an on-device cross-check
 * (for Q16.16: the all-integer kernel); 6 / 7 = Q16.16 GEMM only: the FP64-pipe kernel alone /
 * the tensor-core hybrid at every size (default: hybrid from 2^25 products up, i.e. about 320^3).
 * The hybrid is ONE kernel that forms the limb products on the tensor cores and the per-product
 * floor term on the FP32 pipe of the same SM; 8 / 9 = the hybrid as two kernels instead, one
 * after the other / side by side on two streams, both adding onto C;
 * 10 / 11 = int8 GEMM: the narrow-tile kernel (128 x 64 tiles, for products with few tiles)
 * always / never (default: when the wide tiles would leave most SMs idle); 12 / 13 = int8 GEMM:
 * the kernel with 256 x 512 tiles on CTA pairs always / never (default: for long K and many tiles);
 * 14 = Q16.16 GEMM only: the two-kernel hybrid in its earlier form, floor(a * (b & 0xffff) / 65536)
 * on the FP64 pipe beside seven limb products (default: floor((a & 0xffff) * (b & 0xffff) / 65536)
 * on the FP32 pipe beside eleven).
 * Every path gives identical bytes.  The setting is process-wide and meant for tests and
 * measurements; a call that is already running keeps the kernels it chose. */
int64_t mind_b200_set_gemm_path(int64_t path);
/* Measurement knob of the int8 GEMM's tile order: m-tiles walked together before moving on in
 * N (0 = default, 8) and the order variant (0 = default: odd groups walk N backwards; 1 = the
 * same; 2 = every group walks N forwards; 3 = the default order with the epilogue storing rows
 * itself instead of handing its blocks to TMA stores).  Every setting gives identical bytes. */
int64_t mind_b200_set_tile_order(int64_t group_m, int64_t raster);
/* Self-test of the bounded waits inside the GEMM kernels: launches a one-warp kernel that waits
 * (with the given limit, 1..1000 ms) on a barrier nothing will ever complete.  The expected
 * result is MIND_B200_ERR_TIMEOUT with the CUDA context still usable. */
int64_t mind_b200_selftest_wait_timeout(int64_t limit_ms);
/* Kernel timing for measurements: while enabled, the dominant kernel of every call (the
 * GEMM / GEMV kernel itself, not the operand re-layout) is bracketed by CUDA events on the
 * library's stream.  mind_b200_profile_read waits for the stream, returns how many kernels
 * were timed since the last read (at most 512 are kept) and their summed duration. */
int64_t mind_b200_profile(int64_t enable);
int64_t mind_b200_profile_read(int64_t* launches_out, double* total_ms_out);

/* Measured FP64 FMA rate of the current device (FMA per second): a register-only fma.rm.f64
 * loop timed with CUDA events; the ceiling of the Q16.16 GEMM in the forms that keep the
 * per-product floor on the FP64 pipe (one such FMA per product: the single-kernel form of small
 * products and set_gemm_path(14)).  sm_mhz_out (may be NULL) receives the SM clock the loop ran at (cycle
 * counter over wall clock inside the kernel).  Synchronous; a few milliseconds. */
int64_t mind_b200_fp64_fma_peak(double* fma_per_s_out, double* sm_mhz_out);
/* The same for the FP32 pipe in its packed round-down form (fma.rm.f32x2, two FMAs per
 * instruction, both counted): the ceiling of the Q16.16 GEMM in its default form for large
 * products (the fused kernel), which spends one FP32 FMA per product on
 * floor((a & 0xffff) * (b & 0xffff) / 65536) while the tensor cores form the linear terms. */
int64_t mind_b200_fp32_fma_peak(double* fma_per_s_out, double* sm_mhz_out);
/* Q16.16 GEMM in its two-kernel forms (set_gemm_path 8 / 9 / 14), measurement knob: SMs given to
 * the tensor-core half while the floor kernel runs beside it on the others; 0 = the halves in
 * sequence, -1 = chosen by size (the default).  Any value other than -1 also keeps the fused
 * kernel from being chosen. */
int64_t mind_b200_set_q16_split(int64_t side_sms);

/* ---- seeded inputs and large-shape checking on the device ------------------------------------- */
/* Fills dst (device or host pointer) with elements [offset, offset + n) of the reference's
 * generator stream (tests/cross_substrate_identity.rs:589-601): kind 0 = Q16.16 int32
 * ((i32)u32 >> shift), 1 = int8, 2 = int16.  Element i uses the state after i + 1 steps from
 * `seed`, so a second operand continues the first by passing offset = the first one's length. */
int64_t mind_b200_lcg_fill(int64_t dst, int64_t n, int64_t kind, int64_t seed, int64_t offset, int64_t shift);
/* out[r] = (i32) sum_c mat[r,c] * v[c] with 32-bit wrap; mat has elem_bytes in {1, 2, 4} (signed).
 * Building block of the exact Freivalds check C.v == A.(B.v) in Z/2^32. */
int64_t mind_b200_matvec_wrap(int64_t mat, int64_t elem_bytes, int64_t rows, int64_t cols, int64_t v, int64_t out);

/* ---- MindRuntime mirror (src/runtime_interface.rs:26-52) ---------------------------------------
 * allocate / run_op / synchronize / deallocate over device buffers.  Handles are the
 * reference's TensorHandle (usize).  dtype codes: 0 = i8, 1 = i16, 2 = i32 (also Q16.16).
 * run_op names are the intrinsic names without the "__mind_blas_" prefix
 * ("matmul_mm_i8_v", "matmul_mm_q16_v", "gemv_q16_mt", "matmul_rmajor_i16_v", "matmul_mm_i16", ...);
 * shapes are taken from the handles.  All return 0 or a negative code. */
int64_t mind_b200_rt_allocate(int64_t dtype, const int64_t* shape, int64_t rank, int64_t* handle_out);
int64_t mind_b200_rt_deallocate(int64_t handle);
/* The reference's DType has no int8 / int16 (src/types/mod.rs:32-47): a MindRuntime shim
 * allocates such operands as int32 buffers whose last dimension is the row length in bytes / 4
 * and re-tags them with the element type the op reads (same bytes, last dimension rescaled). */
int64_t mind_b200_rt_retag(int64_t handle, int64_t dtype);
int64_t mind_b200_rt_upload(int64_t handle, const void* host_src, int64_t bytes);
int64_t mind_b200_rt_download(int64_t handle, void* host_dst, int64_t bytes);
int64_t mind_b200_rt_device_ptr(int64_t handle, int64_t* ptr_out);
int64_t mind_b200_rt_run_op(const char* op, const int64_t* inputs, int64_t n_inputs,
                            const int64_t* outputs, int64_t n_outputs);
int64_t mind_b200_rt_synchronize(void);

#ifdef __cplusplus
}
#endif
#endif /* MIND_B200_H */
