// int8 GEMM for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need a GEMM: code
// running inside a region where allocation is forbidden or would synchronise the device
// (a latency-critical serving loop, a process whose memory pool is owned and capped by
// another component), or code that has handed all of the GPU's memory to its own
// allocator.  The regular entry point (__mind_blas_matmul_mm_i8_v) keeps a transposed B
// (when B's rows are not 16-byte pitched) and a padded A (when A's are not) in a scratch
// buffer that it grows with cudaMalloc on demand, and it creates a small per-device
// context on first use.  The entry point in this file does the same computation with the
// same kernels, but its scratch is a fixed array that is part of the library image: nothing
// here calls cudaMalloc, cudaFree, cudaMallocHost or any routine that allocates on the
// caller's behalf.  It is an ordinary synchronous host call (it launches kernels and waits
// for them), so it must not be made from a CUDA host callback (cudaLaunchHostFunc), where
// CUDA calls are forbidden, nor on a stream that is being captured.
//
// Cost and limits: every GPU on which the library is loaded holds the array
// (MIND_B200_STATIC_SCRATCH_BYTES = 8 MiB, plus a 256-byte header) until the process exits,
// and shapes whose re-laid-out operands do not fit are rejected (see the header file).
// All calls share the one array, which keeps whatever the last call left in it: each call
// rewrites every byte it later reads and clears the error word first, but two calls that
// overlap on the GPU (different streams, or different host threads racing to enqueue)
// would overwrite each other's operands.  Calls are therefore serialised on the host by a
// lock and each call waits for its own work before it returns - also when it fails half way.
#include <mutex>

#include "common.h"

namespace mb200 {
namespace {

constexpr size_t STATIC_SCRATCH_BYTES = 8u << 20;
constexpr size_t HEADER_BYTES = 256;  // [0, 4): kernel error word; rest unused

// The scratch itself.  In HOST code this name is only a handle for the runtime's symbol
// table, not a device address: the address is fetched with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[HEADER_BYTES + STATIC_SCRATCH_BYTES];

constexpr int MAX_DEV = 64;
std::mutex g_static_mutex;
unsigned char* g_static_ptr[MAX_DEV] = {};  // device address of the array, per device

// Once per device, with that device current: resolve the array's device address.
int64_t static_scratch_for_current_device(int* device_out, unsigned char** ptr_out) {
    int dev = -1;
    MB200_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEV) return fail(MIND_B200_ERR_NO_DEVICE, "unsupported device ordinal %d", dev);
    if (!g_static_ptr[dev]) {
        int major = 0;
        MB200_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        if (major != 10)
            return fail(MIND_B200_ERR_NO_DEVICE, "device %d is not sm_100; libmind_b200 has no fallback", dev);
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            return fail(MIND_B200_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed on device %d: %s", dev,
                        cudaGetErrorString(e));
        }
        g_static_ptr[dev] = static_cast<unsigned char*>(p);
    }
    *device_out = dev;
    *ptr_out = g_static_ptr[dev];
    return 0;
}

int64_t require_device_pointer(const void* p, int dev, const char* what) {
    cudaPointerAttributes at;
    cudaError_t e = cudaPointerGetAttributes(&at, p);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(MIND_B200_ERR_INVALID, "%s: cannot classify the pointer (%s)", what, cudaGetErrorString(e));
    }
    if (at.type == cudaMemoryTypeManaged) return 0;
    if (at.type != cudaMemoryTypeDevice)
        return fail(MIND_B200_ERR_INVALID,
                    "%s is a host pointer: this entry point cannot stage host operands without allocating; "
                    "pass device memory or use __mind_blas_matmul_mm_i8_v", what);
    if (at.device != dev)
        return fail(MIND_B200_ERR_INVALID, "%s lives on device %d but the current device is %d", what, at.device, dev);
    return 0;
}

}  // namespace
}  // namespace mb200

using namespace mb200;

extern "C" int64_t mind_b200_matmul_mm_i8_static(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k,
                                                 int64_t n, int64_t cuda_stream) {
    clear_error();
    if (m < 0 || k < 0 || n < 0) return fail(MIND_B200_ERR_INVALID, "negative dimension");
    if (m == 0 || n == 0) return 0;
    if (!c || (k > 0 && (!a || !b))) return fail(MIND_B200_ERR_INVALID, "null operand");
    if (c & 3) return fail(MIND_B200_ERR_INVALID, "C is not 4-byte aligned");

    std::lock_guard<std::mutex> lock(g_static_mutex);
    int dev = -1;
    unsigned char* base = nullptr;
    MB200_TRY(static_scratch_for_current_device(&dev, &base));
    MB200_TRY(require_device_pointer(reinterpret_cast<void*>(c), dev, "C"));
    if (k > 0) {
        MB200_TRY(require_device_pointer(reinterpret_cast<void*>(a), dev, "A"));
        MB200_TRY(require_device_pointer(reinterpret_cast<void*>(b), dev, "B"));
    }

    // A throw-away context on the stack: the kernels' launchers only read it.
    DeviceCtx ctx;
    ctx.device = dev;
    MB200_CUDA(cudaDeviceGetAttribute(&ctx.sm_count, cudaDevAttrMultiProcessorCount, dev));
    ctx.stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    ctx.err_word = reinterpret_cast<int*>(base);  // header of the static array
    int32_t* dc = reinterpret_cast<int32_t*>(c);

    if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff)
        return fail(MIND_B200_ERR_TOO_LARGE, "GEMM dimension above 2^31-1");

    if (k == 0) {
        MB200_CUDA(cudaMemsetAsync(dc, 0, (size_t)m * n * 4, ctx.stream));
        MB200_CUDA(cudaStreamSynchronize(ctx.stream));
        return 0;
    }

    // Same operand rules as the regular entry point: an operand whose rows TMA can address
    // (16-byte pitch and base) is read in place and needs no scratch at all; otherwise B is
    // transposed (N x ceil16(K)) and / or A is padded (M x ceil16(K)) into the array.
    const int64_t kp = (int64_t)align_up((size_t)k, 16);
    const int8_t* da = reinterpret_cast<const int8_t*>(a);
    const int8_t* db = reinterpret_cast<const int8_t*>(b);
    const bool a_direct = kp == k && a % 16 == 0;
    const bool b_direct = n % 16 == 0 && b % 16 == 0;
    // sizes by division first, so that nothing can wrap (dimensions are below 2^31, kp <= 2^31 + 15)
    const size_t cap_rows = STATIC_SCRATCH_BYTES / (size_t)kp;
    if ((!b_direct && (size_t)n > cap_rows) || (!a_direct && (size_t)m > cap_rows))
        return fail(MIND_B200_ERR_TOO_LARGE,
                    "the re-laid-out operands of this shape do not fit the static scratch of %zu bytes; "
                    "use __mind_blas_matmul_mm_i8_v for larger shapes", STATIC_SCRATCH_BYTES);
    const size_t bt_bytes = b_direct ? 0 : align_up((size_t)n * kp, 256);
    const size_t ap_bytes = a_direct ? 0 : align_up((size_t)m * kp, 256);
    if (bt_bytes + ap_bytes > STATIC_SCRATCH_BYTES)
        return fail(MIND_B200_ERR_TOO_LARGE,
                    "shape needs %zu scratch bytes (%s%s) but the static scratch holds %zu; "
                    "use __mind_blas_matmul_mm_i8_v for larger shapes",
                    bt_bytes + ap_bytes, b_direct ? "" : "N*ceil16(K) for the transposed B",
                    a_direct ? "" : " + M*ceil16(K) for the padded A", STATIC_SCRATCH_BYTES);
    int8_t* bt = reinterpret_cast<int8_t*>(base + HEADER_BYTES);
    int8_t* ap = reinterpret_cast<int8_t*>(base + HEADER_BYTES + bt_bytes);

    // From the first enqueue on, every way out waits for the stream: a later call must never
    // rewrite the array under kernels of this one, even when this one fails half way.
    struct Drain {
        cudaStream_t s;
        ~Drain() {
            cudaStreamSynchronize(s);
            cudaGetLastError();
        }
    } drain{ctx.stream};

    // The array keeps the last call's contents: the error word must start at zero; the
    // operand areas are fully rewritten by the re-layout kernels before the GEMM reads them.
    MB200_CUDA(cudaMemsetAsync(ctx.err_word, 0, sizeof(int), ctx.stream));
    if (!b_direct) MB200_TRY(launch_transpose_i8(&ctx, db, bt, k, n, kp));
    if (!a_direct) {
        MB200_TRY(launch_pad_rows_i8(&ctx, da, ap, m, k, kp));
        da = ap;
    }
    if (b_direct)
        MB200_TRY(launch_gemm_i8_tc_bmn(&ctx, da, db, dc, m, n, k, kp, n));
    else
        MB200_TRY(launch_gemm_i8_tc(&ctx, da, bt, dc, m, n, k, kp, kp));

    int code = 0;  // pageable host word: the copy allocates nothing
    MB200_CUDA(cudaMemcpyAsync(&code, ctx.err_word, sizeof(int), cudaMemcpyDeviceToHost, ctx.stream));
    MB200_CUDA(cudaStreamSynchronize(ctx.stream));
    if (code != 0)
        return fail(MIND_B200_ERR_TIMEOUT, "a bounded wait inside the GEMM kernel ran out (role code %d); the output is invalid", code);
    return 0;
}
