// One call, several GPUs: the device-side twin of the reference's multithreaded entry points.
//
// The reference parallelises INSIDE one intrinsic call: `__mind_blas_matmul_mm_*_mt_v` and
// `__mind_blas_gemv_q16_mt` cut the M output rows into contiguous owner-computes bands
// (band = ceil(M / T), src/mlir/lowering.rs:10146-10205), pack one argument struct per band
// (:10300-10337) and hand them to a persistent pool (`__mind_blas_mt_dispatch`,
// runtime-support/mind_intrinsics.c:2017-2046).  Here a band owner is a GPU: a call whose
// operands are HOST buffers is spread over the devices named by MINDB200_DEVICES (or
// mind_b200_set_devices), one persistent host thread per device, the same band rule, no
// reduction between bands - so the bytes do not depend on the device count.
//
// What the devices share is the right-hand operand.  For the int8 GEMM it is as large as A, and
// uploading all of it over every PCIe link would cost G times its size in host traffic: instead
// device g uploads only the g-th slice of B's K rows and passes it on to every peer over NVLink
// (cudaMemcpyPeerAsync between the devices' own copies of B), so every byte of A, B and C crosses
// PCIe exactly once, on G links at a time.  The GEMM kernels and their tensor maps only ever
// read the memory of the GPU they run on.
//
// Like the reference's pool, the threads are made on first use and joined at shutdown
// (mind_b200_shutdown or the library's destructor); a fork() after first use is not supported.
#include <condition_variable>
#include <stdlib.h>
#include <string.h>
#include <thread>

#include "common.h"

namespace mb200 {
namespace {

constexpr int MAX_MULTI = 16;

// Reusable barrier for the workers of one call.
class PhaseBarrier {
public:
    void reset(int n) {
        n_ = n;
        waiting_ = 0;
        phase_ = 0;
    }
    void arrive_and_wait() {
        std::unique_lock<std::mutex> lk(mu_);
        const int phase = phase_;
        if (++waiting_ == n_) {
            waiting_ = 0;
            ++phase_;
            cv_.notify_all();
        } else {
            cv_.wait(lk, [&] { return phase_ != phase; });
        }
    }

private:
    std::mutex mu_;
    std::condition_variable cv_;
    int n_ = 1, waiting_ = 0, phase_ = 0;
};

// ---------------------------------------------------------------------------- the pool
struct Worker {
    std::thread thread;
    int device = -1;
    std::function<int64_t(int)> job;  // argument: the worker's index in the call
    bool has_job = false, exit = false;
    int64_t rc = 0;
    std::string error;
};

struct Pool {
    std::mutex call_mu;  // one multi-device call at a time, like the reference's dispatch lock
    std::mutex mu;
    std::condition_variable cv_job, cv_done;
    Worker workers[MAX_MULTI];
    int n_workers = 0;
    int pending = 0;
    int devices[MAX_MULTI] = {};
    int n_devices = -1;  // -1: MINDB200_DEVICES not read yet
    bool peer_ok = false;
};
// On the heap and never destroyed: a static destructor would run before the library's own
// destructor at process exit and find the threads still joinable.
Pool& g_pool = *new Pool;

void worker_main(int idx) {
    Pool& P = g_pool;
    Worker& w = P.workers[idx];
    for (;;) {
        std::function<int64_t(int)> job;
        {
            std::unique_lock<std::mutex> lk(P.mu);
            P.cv_job.wait(lk, [&] { return w.has_job || w.exit; });
            if (w.exit) return;
            job = w.job;
        }
        int64_t rc;
        std::string err;
        if (cudaSetDevice(w.device) != cudaSuccess) {
            cudaGetLastError();
            rc = MIND_B200_ERR_CUDA;
            err = "cudaSetDevice failed in a device thread";
        } else {
            clear_error();
            rc = job(idx);
            if (rc != 0 && last_error_cstr()) err = last_error_cstr();
        }
        {
            std::lock_guard<std::mutex> lk(P.mu);
            w.rc = rc;
            w.error = err;
            w.has_job = false;
            if (--P.pending == 0) P.cv_done.notify_all();
        }
    }
}

// MINDB200_DEVICES: a count ("4": the first four usable devices) or a list ("0,2,3").
void read_env_locked() {
    Pool& P = g_pool;
    if (P.n_devices >= 0) return;
    P.n_devices = 1;
    const char* e = getenv("MINDB200_DEVICES");
    if (!e || !*e) return;
    const int usable = usable_device_count();
    if (strchr(e, ',')) {
        int n = 0;
        const char* s = e;
        while (*s && n < MAX_MULTI) {
            char* end = nullptr;
            const long d = strtol(s, &end, 10);
            if (end == s) break;
            if (d >= 0 && d < usable) P.devices[n++] = (int)d;
            s = *end == ',' ? end + 1 : end;
        }
        if (n >= 1) P.n_devices = n;
    } else {
        long n = strtol(e, nullptr, 10);
        if (n > usable) n = usable;
        if (n > MAX_MULTI) n = MAX_MULTI;
        if (n >= 1) {
            for (int i = 0; i < n; ++i) P.devices[i] = i;
            P.n_devices = (int)n;
        }
    }
}

// Starts the threads for the first `g` devices of the list and opens peer access between
// them (once).  Called with call_mu held.
int64_t ensure_workers(int g) {
    Pool& P = g_pool;
    std::unique_lock<std::mutex> lk(P.mu);
    if (P.n_workers >= g) return 0;
    const int first_new = P.n_workers;
    for (int i = first_new; i < g; ++i) {
        P.workers[i].device = P.devices[i];
        P.workers[i].exit = false;
        P.workers[i].has_job = false;
        P.workers[i].thread = std::thread(worker_main, i);
    }
    P.n_workers = g;
    lk.unlock();
    // Peer access, every ordered pair: a push from device i lands in device j's copy of B.
    int before = 0;
    cudaGetDevice(&before);
    bool all = true;
    for (int i = 0; i < g; ++i) {
        if (cudaSetDevice(P.devices[i]) != cudaSuccess) {
            all = false;
            continue;
        }
        for (int j = 0; j < g; ++j) {
            if (i == j) continue;
            int can = 0;
            if (cudaDeviceCanAccessPeer(&can, P.devices[i], P.devices[j]) != cudaSuccess || !can) {
                all = false;
                continue;
            }
            const cudaError_t e = cudaDeviceEnablePeerAccess(P.devices[j], 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) all = false;
        }
    }
    cudaGetLastError();
    cudaSetDevice(before);
    P.peer_ok = all;
    return 0;
}

// Runs job(i) on the first g device threads and waits for all of them.  The first failure's
// code and message become the calling thread's.
int64_t run_on_devices(int g, const std::function<int64_t(int)>& job) {
    Pool& P = g_pool;
    {
        std::lock_guard<std::mutex> lk(P.mu);
        for (int i = 0; i < g; ++i) {
            P.workers[i].job = job;
            P.workers[i].has_job = true;
        }
        P.pending = g;
    }
    P.cv_job.notify_all();
    std::unique_lock<std::mutex> lk(P.mu);
    P.cv_done.wait(lk, [&] { return P.pending == 0; });
    // report the device that failed first-hand, not one that only stopped because of it
    for (int pass = 0; pass < 2; ++pass)
        for (int i = 0; i < g; ++i) {
            const Worker& w = P.workers[i];
            if (w.rc != 0 && (pass == 1 || w.error.find("another device") == std::string::npos))
                return fail(w.rc, "device %d: %s", w.device, w.error.empty() ? "failed" : w.error.c_str());
        }
    return 0;
}

bool is_plain_host(const void* p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return true;
    }
    return at.type == cudaMemoryTypeUnregistered || at.type == cudaMemoryTypeHost;
}

// How many devices a call of m rows is spread over (1 = not taken).  Bands are
// ceil(m / g) rows, so a small m may use fewer devices than configured.
int plan_devices(int64_t m, size_t total_bytes, int64_t min_rows_per_device) {
    Pool& P = g_pool;
    int g;
    {
        std::lock_guard<std::mutex> lk(P.mu);
        read_env_locked();
        g = P.n_devices;
    }
    if (g <= 1 || total_bytes < ((size_t)8 << 20)) return 1;
    while (g > 1 && m / g < min_rows_per_device) --g;
    if (g <= 1) return 1;
    const int64_t band = (m + g - 1) / g;
    return (int)((m + band - 1) / band);
}

// ------------------------------------------------------------------ int8 GEMM, B exchanged
struct I8Job {
    const int8_t* a;
    const int8_t* b;
    int32_t* c;
    int64_t m, k, n, band;
    int g;
    bool exchange;                 // K-slices of B passed between the devices (needs peer access)
    bool a_page, b_page, c_page;   // pageable host operands: moved by the staging threads (staging.cu)
    int dev[MAX_MULTI];            // device ordinals, by worker
    int8_t* b_dev[MAX_MULTI];      // every device's own full copy of B
    cudaEvent_t b_ready[MAX_MULTI];  // worker i's slice has reached every device
    PhaseBarrier bar;
    std::atomic<int> failed{0};
};

int64_t i8_worker(I8Job& J, int w) {
    const int64_t m = J.m, k = J.k, n = J.n;
    const int64_t r0 = (int64_t)w * J.band, rows = (m - r0 < J.band) ? m - r0 : J.band;
    const int64_t kp = (int64_t)align_up((size_t)k, 16);
    // Sub-bands: the unit of upload -> product -> download overlap on this device.
    const int64_t sub = (int64_t)align_up((size_t)((rows + 7) / 8), 256);
    const int64_t nsub = (rows + sub - 1) / sub;
    const bool b_direct = tuning().force_transpose.load() == 0 && n % 16 == 0;
    constexpr int nslot = 2;

    DeviceCtx* ctx = current_ctx();
    std::unique_lock<std::mutex> lock;
    if (ctx) lock = std::unique_lock<std::mutex>(ctx->mu);
    Pipe* P = nullptr;
    int8_t *b_stage = nullptr, *a_stage = nullptr, *bt = nullptr;
    int32_t* c_slot[nslot] = {nullptr, nullptr};

    // ---- phase 0: buffers; every device publishes where its copy of B lives
    int64_t rc = ctx ? 0 : MIND_B200_ERR_NO_DEVICE;
    if (!rc) rc = pipe_for(ctx, (size_t)nsub, &P);
    if (!rc) {
        const size_t sb = align_up((size_t)k * n, 1024), sa = align_up((size_t)rows * kp, 1024);
        const size_t sc = align_up((size_t)sub * n * 4, 1024);
        rc = arena_reserve(ctx, ctx->staging, sb + sa + nslot * sc + 8192);
        if (!rc) {
            b_stage = static_cast<int8_t*>(arena_take(ctx->staging, sb));
            a_stage = static_cast<int8_t*>(arena_take(ctx->staging, sa));
            for (int s = 0; s < nslot; ++s) c_slot[s] = static_cast<int32_t*>(arena_take(ctx->staging, sc));
        }
    }
    if (!rc && !b_direct) {
        rc = arena_reserve(ctx, ctx->scratch, align_up((size_t)n * kp, 1024) + 2048);
        if (!rc) bt = static_cast<int8_t*>(arena_take(ctx->scratch, (size_t)n * kp));
    }
    if (!rc) {
        J.b_dev[w] = b_stage;
        J.b_ready[w] = P->b_ready;
    } else {
        J.failed = 1;
    }
    J.bar.arrive_and_wait();

    // ---- phase 1: uploads, all queued on this device's in-stream: this device's share of B
    // (passed on to every peer), then the sub-bands of A
    // Host-side completion of copies that the staging threads make (pageable operands): the CUDA
    // event of a group is recorded by the thread that queues its last chunk, and this thread
    // waits on the host until that has happened before it makes a stream wait for the event.
    StageStatus stage_status;
    StageGroup b_group, out_groups[nslot];
    std::vector<StageGroup> up_groups(J.a_page ? (size_t)nsub : 0);
    const int device = J.dev[w];
    auto uploads = [&]() -> int64_t {
        MB200_CUDA(cudaEventRecord(P->start, ctx->stream));
        MB200_CUDA(cudaStreamWaitEvent(P->in, P->start, 0));
        MB200_CUDA(cudaStreamWaitEvent(P->out, P->start, 0));
        if (J.exchange) {
            const int64_t ks = (k + J.g - 1) / J.g, k0 = (int64_t)w * ks, k1 = k0 + ks < k ? k0 + ks : k;
            if (k1 > k0) {
                const size_t off = (size_t)k0 * n, bytes = (size_t)(k1 - k0) * n;
                if (J.b_page) {  // the pushes below must follow the whole slice in stream order
                    stage_upload(device, reinterpret_cast<char*>(b_stage) + off, (size_t)n,
                                 reinterpret_cast<const char*>(J.b) + off, (size_t)n, (size_t)n, (size_t)(k1 - k0), P->in,
                                 &b_group, nullptr, &stage_status);
                    b_group.wait();
                } else {
                    MB200_CUDA(cudaMemcpyAsync(b_stage + off, J.b + off, bytes, cudaMemcpyHostToDevice, P->in));
                }
                for (int h = 1; h < J.g; ++h) {  // start with the next device round: spreads the NVLink load
                    const int peer = (w + h) % J.g;
                    MB200_CUDA(cudaMemcpyPeerAsync(J.b_dev[peer] + off, J.dev[peer], b_stage + off, J.dev[w], bytes, P->in));
                }
            }
        } else if (J.b_page) {
            stage_upload(device, reinterpret_cast<char*>(b_stage), (size_t)n, reinterpret_cast<const char*>(J.b), (size_t)n,
                         (size_t)n, (size_t)k, P->in, &b_group, nullptr, &stage_status);
            b_group.wait();
        } else {
            MB200_CUDA(cudaMemcpyAsync(b_stage, J.b, (size_t)k * n, cudaMemcpyHostToDevice, P->in));
        }
        MB200_CUDA(cudaEventRecord(P->b_ready, P->in));
        for (int64_t i = 0; i < nsub; ++i) {
            const int64_t s0 = i * sub, srows = (rows - s0 < sub) ? rows - s0 : sub;
            int8_t* dst = a_stage + (size_t)s0 * kp;
            const int8_t* src = J.a + (size_t)(r0 + s0) * k;
            if (J.a_page) {
                cudaEvent_t ev = P->ready[i];
                cudaStream_t in = P->in;
                stage_upload(device, reinterpret_cast<char*>(dst), (size_t)kp, reinterpret_cast<const char*>(src), (size_t)k,
                             (size_t)k, (size_t)srows, in, &up_groups[(size_t)i], [ev, in] { cudaEventRecord(ev, in); },
                             &stage_status);
                continue;
            }
            if (kp == k)
                MB200_CUDA(cudaMemcpyAsync(dst, src, (size_t)srows * k, cudaMemcpyHostToDevice, P->in));
            else  // pad to a 16-byte pitch on the way: the pad bytes are never read
                MB200_CUDA(cudaMemcpy2DAsync(dst, (size_t)kp, src, (size_t)k, (size_t)k, (size_t)srows,
                                             cudaMemcpyHostToDevice, P->in));
            MB200_CUDA(cudaEventRecord(P->ready[i], P->in));
        }
        return 0;
    };
    if (!J.failed.load()) {
        rc = uploads();
        if (rc) J.failed = 1;
    }
    J.bar.arrive_and_wait();

    // ---- phase 2: products and downloads.  The kernels wait for every slice of B (events of
    // the devices that pushed them), then run sub-band by sub-band.
    auto products = [&]() -> int64_t {
        for (int h = 0; h < J.g; ++h)
            if (J.exchange || h == w) MB200_CUDA(cudaStreamWaitEvent(ctx->stream, J.b_ready[h], 0));
        if (!b_direct) MB200_TRY(launch_transpose_i8(ctx, b_stage, bt, k, n, kp));
        for (int64_t i = 0; i < nsub; ++i) {
            const int s = (int)(i % nslot);
            const int64_t s0 = i * sub, srows = (rows - s0 < sub) ? rows - s0 : sub;
            if (J.a_page) up_groups[(size_t)i].wait();  // the event below has been recorded
            MB200_CUDA(cudaStreamWaitEvent(ctx->stream, P->ready[i], 0));
            if (i >= nslot) {  // slot free
                if (J.c_page) out_groups[s].wait();
                MB200_CUDA(cudaStreamWaitEvent(ctx->stream, P->out_done[s], 0));
            }
            const int8_t* a_sub = a_stage + (size_t)s0 * kp;
            if (b_direct)
                MB200_TRY(launch_gemm_i8_tc_bmn(ctx, a_sub, b_stage, c_slot[s], srows, n, k, kp, n));
            else
                MB200_TRY(launch_gemm_i8_tc(ctx, a_sub, bt, c_slot[s], srows, n, k, kp, kp));
            MB200_CUDA(cudaEventRecord(P->gemm_done[s], ctx->stream));
            MB200_CUDA(cudaStreamWaitEvent(P->out, P->gemm_done[s], 0));
            if (J.c_page) {
                cudaEvent_t ev = P->out_done[s];
                cudaStream_t out = P->out;
                stage_download(device, reinterpret_cast<char*>(J.c + (size_t)(r0 + s0) * n),
                               reinterpret_cast<const char*>(c_slot[s]), (size_t)srows * n * 4, out, &out_groups[s],
                               [ev, out] { cudaEventRecord(ev, out); }, &stage_status);
            } else {
                MB200_CUDA(cudaMemcpyAsync(J.c + (size_t)(r0 + s0) * n, c_slot[s], (size_t)srows * n * 4,
                                           cudaMemcpyDeviceToHost, P->out));
                MB200_CUDA(cudaEventRecord(P->out_done[s], P->out));
            }
        }
        for (int s = 0; s < nslot && s < nsub; ++s) {
            if (J.c_page) out_groups[s].wait();
            MB200_CUDA(cudaStreamWaitEvent(ctx->stream, P->out_done[s], 0));
        }
        if (J.c_page) stager_drain();  // the last chunks are in the caller's buffer
        MB200_CUDA(cudaStreamSynchronize(ctx->stream));
        if (stage_status.failed.load()) return fail(MIND_B200_ERR_CUDA, "a staged copy of a pageable host operand failed");
        return check_err_word(ctx);
    };
    if (!J.failed.load()) {
        rc = products();
        if (rc) J.failed = 1;
    }
    // Whatever happened, nothing of this call may still be in flight on this device when the
    // arenas are handed to the next call, and no peer may still be copying from or into them.
    if (J.a_page || J.b_page || J.c_page) stager_drain();
    if (P) {
        cudaStreamSynchronize(P->in);
        cudaStreamSynchronize(P->out);
        cudaStreamSynchronize(ctx->stream);
        cudaGetLastError();
    }
    J.bar.arrive_and_wait();
    if (!rc && J.failed.load()) rc = fail(MIND_B200_ERR_CUDA, "another device of this call failed");
    return rc;
}

}  // namespace

int multi_device_count() {
    std::lock_guard<std::mutex> lk(g_pool.mu);
    read_env_locked();
    return g_pool.n_devices;
}

int64_t multi_set_devices(int64_t count) {
    const int usable = usable_device_count();
    if (count < 1 || count > MAX_MULTI) return fail(MIND_B200_ERR_INVALID, "device count must be 1..%d", MAX_MULTI);
    if (count > 1 && count > usable)
        return fail(MIND_B200_ERR_NO_DEVICE, "%lld devices asked for but %d sm_100 devices are usable", (long long)count, usable);
    std::lock_guard<std::mutex> call(g_pool.call_mu);
    std::lock_guard<std::mutex> lk(g_pool.mu);
    for (int i = 0; i < count; ++i)
        if (i >= g_pool.n_workers) g_pool.devices[i] = i;  // a running thread keeps its device
    g_pool.n_devices = (int)count;
    return 0;
}

void multi_shutdown() {
    Pool& P = g_pool;
    std::lock_guard<std::mutex> call(P.call_mu);
    int n;
    {
        std::lock_guard<std::mutex> lk(P.mu);
        n = P.n_workers;
        for (int i = 0; i < n; ++i) P.workers[i].exit = true;
    }
    P.cv_job.notify_all();
    for (int i = 0; i < n; ++i)
        if (P.workers[i].thread.joinable()) P.workers[i].thread.join();
    std::lock_guard<std::mutex> lk(P.mu);
    P.n_workers = 0;
}

int64_t multi_gemm_i8(const int8_t* a, const int8_t* b, int32_t* c, int64_t m, int64_t k, int64_t n) {
    const size_t total = (size_t)m * k + (size_t)k * n + (size_t)m * n * 4;
    const int g = plan_devices(m, total, 256);
    if (g <= 1 || !is_plain_host(a) || !is_plain_host(b) || !is_plain_host(c)) return MULTI_NOT_TAKEN;
    Pool& P = g_pool;
    std::lock_guard<std::mutex> call(P.call_mu);
    MB200_TRY(ensure_workers(g));
    I8Job J;
    J.a = a;
    J.b = b;
    J.c = c;
    J.m = m;
    J.k = k;
    J.n = n;
    J.g = g;
    J.band = (m + g - 1) / g;
    J.exchange = P.peer_ok;
    // pageable operands go through the staging threads when a row fits one of their slots
    const bool row_fits = align_up((size_t)k, 16) <= stager_slot_bytes() && (size_t)n * 4 <= stager_slot_bytes();
    const bool may_stage = row_fits && (host_pointer_is_pageable(a) || host_pointer_is_pageable(b) || host_pointer_is_pageable(c)) &&
                           stager_start();
    J.a_page = may_stage && host_pointer_is_pageable(a);
    J.b_page = may_stage && host_pointer_is_pageable(b);
    J.c_page = may_stage && host_pointer_is_pageable(c);
    for (int i = 0; i < g; ++i) {
        J.dev[i] = P.devices[i];
        J.b_dev[i] = nullptr;
        J.b_ready[i] = nullptr;
    }
    J.bar.reset(g);
    return run_on_devices(g, [&J](int w) { return i8_worker(J, w); });
}

int64_t multi_banded(const void* a, size_t a_row_bytes, const void* shared, size_t shared_bytes, void* c,
                     size_t c_row_bytes, int64_t m,
                     const std::function<int64_t(const void*, void*, int64_t)>& band_fn) {
    const size_t total = (size_t)m * (a_row_bytes + c_row_bytes) + shared_bytes;
    const int g = plan_devices(m, total, 256);
    if (g <= 1 || !is_plain_host(a) || !is_plain_host(shared) || !is_plain_host(c)) return MULTI_NOT_TAKEN;
    // The shared operand goes to every device: only worth it while it is the smaller part.
    if (shared_bytes * (size_t)g > total) return MULTI_NOT_TAKEN;
    Pool& P = g_pool;
    std::lock_guard<std::mutex> call(P.call_mu);
    MB200_TRY(ensure_workers(g));
    const int64_t band = (m + g - 1) / g;
    return run_on_devices(g, [&](int w) -> int64_t {
        const int64_t r0 = (int64_t)w * band, rows = (m - r0 < band) ? m - r0 : band;
        return band_fn(static_cast<const char*>(a) + (size_t)r0 * a_row_bytes,
                       static_cast<char*>(c) + (size_t)r0 * c_row_bytes, rows);
    });
}

}  // namespace mb200
