// Per-device context, error reporting, scratch arenas, launch accounting.
#include <stdarg.h>
#include <stdio.h>

#include <atomic>
#include <mutex>

#include "common.h"

namespace mb200 {

namespace {
thread_local std::string t_error;
thread_local bool t_has_error = false;
std::atomic<long long> g_launches{0};
constexpr int MAX_DEVICES = 64;
// The context table lives on the heap and is never destroyed by a static destructor: the
// library's own destructor (which runs after the static ones at process exit) still walks it.
DeviceCtx* g_ctx = nullptr;
std::mutex g_ctx_mutex;
Tuning g_tuning;
DeviceCtx* ctx_table() {  // call with g_ctx_mutex held
    if (!g_ctx) g_ctx = new DeviceCtx[MAX_DEVICES];
    return g_ctx;
}
}  // namespace

Tuning& tuning() { return g_tuning; }

int64_t fail(int64_t code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    t_error = buf;
    t_has_error = true;
    return code;
}

void clear_error() { t_has_error = false; }

const char* last_error_cstr() { return t_has_error ? t_error.c_str() : nullptr; }

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launches() { return g_launches.load(std::memory_order_relaxed); }

int64_t check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail(MIND_B200_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return 0;
}

int usable_device_count() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int usable = 0;
    for (int d = 0; d < n; ++d) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d) == cudaSuccess &&
            major == 10)
            ++usable;
    }
    return usable;
}

DeviceCtx* current_ctx() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        cudaGetLastError();
        fail(MIND_B200_ERR_NO_DEVICE, "no CUDA device is visible; libmind_b200 has no CPU fallback");
        return nullptr;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        fail(MIND_B200_ERR_NO_DEVICE, "cudaGetDevice failed");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    DeviceCtx* ctx = &ctx_table()[dev];
    if (ctx->device == dev) return ctx;
    int major = 0, minor = 0, sms = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (major != 10) {
        fail(MIND_B200_ERR_NO_DEVICE,
             "device %d is sm_%d%d; libmind_b200 is built for sm_100a only and has no fallback", dev,
             major, minor);
        return nullptr;
    }
    // The error word lives in mapped pinned host memory: a kernel writes it only when a bounded
    // wait runs out, and the host reads it after a synchronisation without any copy per call.
    // (a second word of the same allocation receives scalar results: the dots)
    if (cudaHostAlloc(&ctx->err_host, 2 * sizeof(int), cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer(reinterpret_cast<void**>(&ctx->err_word), ctx->err_host, 0) != cudaSuccess) {
        fail(MIND_B200_ERR_CUDA, "could not allocate the device error word: %s",
             cudaGetErrorString(cudaGetLastError()));
        return nullptr;
    }
    *ctx->err_host = 0;
    ctx->scalar_host = ctx->err_host + 1;
    ctx->scalar_dev = reinterpret_cast<int32_t*>(ctx->err_word + 1);
    // made here, not on first use: a first use could fall inside a stream capture
    if (cudaStreamCreateWithFlags(&ctx->side, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&ctx->fork_ev, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&ctx->join_ev, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&ctx->order_ev, cudaEventDisableTiming) != cudaSuccess) {
        fail(MIND_B200_ERR_CUDA, "could not create the side stream: %s", cudaGetErrorString(cudaGetLastError()));
        return nullptr;
    }
    ctx->sm_count = sms;
    ctx->stream = nullptr;
    ctx->device = dev;
    return ctx;
}

int64_t arena_reserve(DeviceCtx* ctx, Arena& a, size_t total_bytes) {
    a.used = 0;
    // A captured graph keeps the addresses it was recorded with.  So: never allocate or wait
    // while the stream is being captured, and once a capture has been seen on this device keep
    // every outgrown block alive (until shutdown) instead of freeing it.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(ctx->stream, &cap) != cudaSuccess) {
        cudaGetLastError();
        cap = cudaStreamCaptureStatusNone;
    }
    const bool capturing = cap != cudaStreamCaptureStatusNone;
    if (capturing) ctx->capture_seen = true;
    if (total_bytes <= a.cap) return 0;
    if (capturing)
        return fail(MIND_B200_ERR_INVALID,
                    "this call needs %zu bytes of library scratch but only %zu are reserved, and the stream is "
                    "being captured: call mind_b200_reserve (or run the same shapes once) before the capture",
                    total_bytes, a.cap);
    if (a.base) {
        if (ctx->capture_seen) {
            ctx->retired.push_back(a.base);
        } else {
            MB200_CUDA(cudaStreamSynchronize(ctx->stream));
            MB200_CUDA(cudaFree(a.base));
        }
        a.base = nullptr;
        a.cap = 0;
    }
    size_t want = align_up(total_bytes + (total_bytes >> 3), 1 << 20);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(MIND_B200_ERR_CUDA, "cudaMalloc of %zu scratch bytes failed: %s", want,
                    cudaGetErrorString(e));
    }
    a.base = static_cast<char*>(p);
    a.cap = want;
    return 0;
}

void* arena_take(Arena& a, size_t bytes) {
    size_t off = align_up(a.used, 1024);
    if (off + bytes > a.cap) return nullptr;
    a.used = off + bytes;
    return a.base + off;
}

// Every CUDA call below may fail with "driver shutting down" when this runs from the library's
// destructor at process exit; the results are ignored on purpose.
void destroy_all_contexts() {
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    if (!g_ctx) return;
    int before = -1;
    const bool have_dev = cudaGetDevice(&before) == cudaSuccess;
    for (int d = 0; d < MAX_DEVICES; ++d) {
        DeviceCtx* ctx = &g_ctx[d];
        if (ctx->device != d) continue;
        std::lock_guard<std::mutex> dev_lock(ctx->mu);
        if (cudaSetDevice(d) == cudaSuccess) {
            cudaDeviceSynchronize();
            if (ctx->scratch.base) cudaFree(ctx->scratch.base);
            if (ctx->staging.base) cudaFree(ctx->staging.base);
            for (void* p : ctx->retired) cudaFree(p);
            if (ctx->err_host) cudaFreeHost(ctx->err_host);
            if (ctx->side) cudaStreamDestroy(ctx->side);
            for (cudaEvent_t e : {ctx->fork_ev, ctx->join_ev, ctx->order_ev})
                if (e) cudaEventDestroy(e);
            for (cudaEvent_t& e : ctx->prof_ev)
                if (e) {
                    cudaEventDestroy(e);
                    e = nullptr;
                }
            Pipe& p = ctx->pipe;
            if (p.in) cudaStreamDestroy(p.in);
            if (p.out) cudaStreamDestroy(p.out);
            for (cudaEvent_t e : {p.start, p.gemm_done[0], p.gemm_done[1], p.out_done[0], p.out_done[1], p.b_ready})
                if (e) cudaEventDestroy(e);
            for (cudaEvent_t e : p.ready) cudaEventDestroy(e);
        }
        cudaGetLastError();
        ctx->scratch = Arena();
        ctx->staging = Arena();
        ctx->retired.clear();
        ctx->err_host = ctx->err_word = ctx->scalar_host = nullptr;
        ctx->scalar_dev = nullptr;
        ctx->side = nullptr;
        ctx->fork_ev = ctx->join_ev = ctx->order_ev = nullptr;
        ctx->pipe = Pipe();
        ctx->stream = nullptr;
        ctx->profile = false;
        ctx->prof_count = 0;
        ctx->capture_seen = false;
        ctx->device = -1;  // rebuilt on the next call
    }
    if (have_dev) cudaSetDevice(before);
    cudaGetLastError();
}

void prof_begin(DeviceCtx* ctx) {
    if (!ctx->profile || ctx->prof_count >= DeviceCtx::PROF_RING) return;
    cudaEvent_t& e = ctx->prof_ev[2 * ctx->prof_count];
    if (!e) {
        cudaEventCreate(&e);
        cudaEventCreate(&ctx->prof_ev[2 * ctx->prof_count + 1]);
    }
    cudaEventRecord(e, ctx->stream);
}

void prof_end(DeviceCtx* ctx) {
    if (!ctx->profile || ctx->prof_count >= DeviceCtx::PROF_RING) return;
    cudaEventRecord(ctx->prof_ev[2 * ctx->prof_count + 1], ctx->stream);
    ++ctx->prof_count;
}

// dlclose() and process exit: join the device threads, then give back what the library holds on
// every GPU (the reference joins its pool the same way, runtime-support/mind_intrinsics.c:2065-2081).
__attribute__((destructor)) static void library_unload() {
    multi_shutdown();
    stager_shutdown();
    destroy_all_contexts();
}

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    });
    return fn;
}

}  // namespace mb200
