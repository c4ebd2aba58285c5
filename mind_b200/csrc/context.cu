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
DeviceCtx g_ctx[MAX_DEVICES];
std::mutex g_ctx_mutex;
}  // namespace

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
    DeviceCtx* ctx = &g_ctx[dev];
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
        cudaEventCreateWithFlags(&ctx->join_ev, cudaEventDisableTiming) != cudaSuccess) {
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
    if (total_bytes <= a.cap) return 0;
    if (a.base) {
        MB200_CUDA(cudaStreamSynchronize(ctx->stream));
        MB200_CUDA(cudaFree(a.base));
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
