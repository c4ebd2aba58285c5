// extern "C" entry points of libmind_b200: argument checks, host / device pointer
// classification, staging of host operands, operand re-layout, kernel dispatch.
#include <mutex>
#include <vector>

#include "common.h"

namespace mb200 {
namespace {

// Calls on one device are serialised by that device's lock (DeviceCtx::mu), like the
// reference's MT dispatch lock; calls on different devices do not wait for each other.
using DevLock = std::lock_guard<std::mutex>;

// One operand of a call: where the caller keeps it and where the kernels see it.
struct Operand {
    void* user = nullptr;
    size_t bytes = 0;
    bool output = false;
    bool host = false;
    bool staged = false;  // pageable and large: moved by the staging threads
    void* dev = nullptr;
};
constexpr size_t STAGED_MIN_BYTES = (size_t)8 << 20;

// Classifies each operand, gives host operands a device copy in the staging arena,
// uploads inputs before the kernels and downloads outputs after them.
class Call {
public:
    explicit Call(DeviceCtx* ctx) : ctx_(ctx) {}

    int add(const void* p, size_t bytes, bool output) {
        Operand& o = store_[n_];
        o = Operand();
        o.user = const_cast<void*>(p);
        o.bytes = bytes;
        o.output = output;
        return n_++;
    }

    int64_t begin() {
        size_t staged = 0;
        for (auto& o : Range{store_, store_ + n_}) {
            if (o.bytes == 0) continue;
            cudaPointerAttributes at;
            cudaError_t e = cudaPointerGetAttributes(&at, o.user);
            if (e != cudaSuccess) {
                cudaGetLastError();
                o.host = true;
            } else if (at.type == cudaMemoryTypeDevice) {
                if (at.device != ctx_->device)
                    return fail(MIND_B200_ERR_INVALID,
                                "operand lives on device %d but the current device is %d", at.device,
                                ctx_->device);
                o.host = false;
            } else {
                o.host = at.type != cudaMemoryTypeManaged;
            }
            if (o.host) {
                staged += align_up(o.bytes, 1024);
                any_host_ = true;
            }
        }
        if (any_host_) MB200_TRY(arena_reserve(ctx_, ctx_->staging, staged + 1024));
        for (auto& o : Range{store_, store_ + n_}) {
            if (o.bytes == 0) continue;
            if (!o.host) {
                o.dev = o.user;
                continue;
            }
            o.dev = arena_take(ctx_->staging, o.bytes);
            if (!o.dev) return fail(MIND_B200_ERR_CUDA, "staging arena exhausted");
            // a large pageable operand goes through the staging threads' pinned slots (several
            // cores copy, the DMAs overlap them) instead of the driver's one-thread staging
            o.staged = o.bytes >= STAGED_MIN_BYTES && host_pointer_is_pageable(o.user) && stager_start();
            if (o.output) continue;
            if (o.staged) {
                const size_t row = (size_t)1 << 20, rows = o.bytes / row, rest = o.bytes - rows * row;
                StageGroup body, tail;
                char* dst = static_cast<char*>(o.dev);
                const char* src = static_cast<const char*>(o.user);
                stage_upload(ctx_->device, dst, row, src, row, row, rows, ctx_->stream, &body, nullptr, &status_);
                if (rest) stage_upload(ctx_->device, dst + rows * row, rest, src + rows * row, rest, rest, 1, ctx_->stream, &tail, nullptr, &status_);
                body.wait();
                tail.wait();  // every DMA is queued on the stream: the kernels that follow see the data
            } else {
                MB200_CUDA(cudaMemcpyAsync(o.dev, o.user, o.bytes, cudaMemcpyHostToDevice, ctx_->stream));
            }
        }
        return 0;
    }

    template <typename T>
    T* dev(int i) const { return static_cast<T*>(store_[i].dev); }

    // Downloads outputs; with any host operand, also waits and reports kernel time-outs.
    // `waits_inside` says a kernel with bounded waits ran, whose error word must be fetched.
    int64_t end(bool waits_inside = false) {
        bool any_staged = false;
        for (auto& o : Range{store_, store_ + n_})
            if (o.host && o.output && o.bytes) {
                if (o.staged) {
                    StageGroup g;
                    stage_download(ctx_->device, static_cast<char*>(o.user), static_cast<const char*>(o.dev), o.bytes,
                                   ctx_->stream, &g, nullptr, &status_);
                    g.wait();
                    any_staged = true;
                } else {
                    MB200_CUDA(cudaMemcpyAsync(o.user, o.dev, o.bytes, cudaMemcpyDeviceToHost, ctx_->stream));
                }
            }
        (void)waits_inside;  // the error word is host-mapped: nothing to fetch
        if (any_host_) {
            if (any_staged) stager_drain();
            MB200_CUDA(cudaStreamSynchronize(ctx_->stream));
            if (status_.failed.load()) return fail(MIND_B200_ERR_CUDA, "a staged copy of a pageable host operand failed");
            return check_err_word(ctx_);
        }
        return 0;
    }

    ~Call() {
        // a call that failed half way may still have staged chunks in flight that point into it
        for (auto& o : Range{store_, store_ + n_})
            if (o.staged) {
                stager_drain();
                break;
            }
    }

    static int64_t check_err_word(DeviceCtx* ctx) { return ::mb200::check_err_word(ctx); }

private:
    // at most four operands per call; iterated as a range
    struct Range {
        Operand *b, *e;
        Operand* begin() const { return b; }
        Operand* end() const { return e; }
    };
    DeviceCtx* ctx_;
    Operand store_[4];
    int n_ = 0;
    bool any_host_ = false;
    StageStatus status_;
};

int64_t check_dims(int64_t m, int64_t k, int64_t n) {
    if (m < 0 || k < 0 || n < 0) return fail(MIND_B200_ERR_INVALID, "negative dimension");
    return 0;
}

// ---------------------------------------------- host-operand pipeline (int8 GEMM)
// With A and / or C in host memory a large GEMM is cut into row bands (independent, like
// the reference's thread bands) and, when C goes back to the host, into column chunks, so
// that uploads, products and downloads overlap: copies run on two side streams, the kernels
// on the library's stream.  Uploads alternate between B chunks and A bands; the first C tile
// is on its way back after one of each has arrived, and after about two rounds the download
// link stays busy.  C tiles are double-buffered in staging.
}  // namespace

int64_t pipe_for(DeviceCtx* ctx, size_t n_ready, Pipe** out) {
    Pipe& p = ctx->pipe;
    if (!p.made) {
        MB200_CUDA(cudaStreamCreateWithFlags(&p.in, cudaStreamNonBlocking));
        MB200_CUDA(cudaStreamCreateWithFlags(&p.out, cudaStreamNonBlocking));
        MB200_CUDA(cudaEventCreateWithFlags(&p.start, cudaEventDisableTiming));
        for (int i = 0; i < 2; ++i) {
            MB200_CUDA(cudaEventCreateWithFlags(&p.gemm_done[i], cudaEventDisableTiming));
            MB200_CUDA(cudaEventCreateWithFlags(&p.out_done[i], cudaEventDisableTiming));
        }
        MB200_CUDA(cudaEventCreateWithFlags(&p.b_ready, cudaEventDisableTiming));
        p.made = true;
    }
    while (p.ready.size() < n_ready) {
        cudaEvent_t e;
        MB200_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        p.ready.push_back(e);
    }
    *out = &p;
    return 0;
}

int64_t check_err_word(DeviceCtx* ctx) {
    const int code = *ctx->err_host;
    if (code == 0) return 0;
    *ctx->err_host = 0;
    return fail(MIND_B200_ERR_TIMEOUT,
                "a bounded wait inside the GEMM kernel ran out (role code %d); the output is invalid", code);
}

// 1 = host, 0 = device of ctx, negative = error.
int64_t pointer_is_host(DeviceCtx* ctx, const void* p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return 1;
    }
    if (at.type == cudaMemoryTypeDevice) {
        if (at.device != ctx->device)
            return fail(MIND_B200_ERR_INVALID, "operand lives on device %d but the current device is %d",
                        at.device, ctx->device);
        return 0;
    }
    return at.type != cudaMemoryTypeManaged;
}

namespace {

constexpr int64_t PIPE_MIN_ROWS = 1024;  // below this one band is as good as several

int64_t gemm_i8_pipelined(DeviceCtx* ctx, const int8_t* a, bool a_host, const int8_t* b, bool b_host,
                          int32_t* c, bool c_host, int64_t m, int64_t k, int64_t n) {
    const int64_t kp = (int64_t)align_up((size_t)k, 16);
    const int64_t band = (int64_t)align_up((size_t)((m + 7) / 8), 256);
    const int64_t bands = (m + band - 1) / band;
    // Pageable host operands (an ordinary malloc / Vec) go through the staging threads' pinned
    // slots instead of the driver's own one-thread staging; page-locked ones are copied directly.
    const bool row_fits = (size_t)kp <= stager_slot_bytes() && (size_t)n * 4 <= stager_slot_bytes();
    const bool a_page = a_host && row_fits && host_pointer_is_pageable(a);
    const bool b_page = b_host && row_fits && host_pointer_is_pageable(b);
    const bool c_page = c_host && row_fits && host_pointer_is_pageable(c);
    const bool staged = (a_page || b_page || c_page) && stager_start();
    // Column chunks only pay when C is downloaded, and need B readable in place per chunk.
    const bool b_inplace_ok = !(tuning().force_transpose.load() != 0) && n % 16 == 0 && (b_host || reinterpret_cast<uintptr_t>(b) % 16 == 0);
    // Four, not more: a strided download slows down beside running kernels as its rows get shorter
    // (measured with a GEMM on another stream: 57 GB/s for 64 KiB rows, 48 for 16 KiB, 31 for 8 KiB).
    // (staged copies move whole rows: one chunk)
    const int64_t chunks = (c_host && b_inplace_ok && n >= 4096 && n % 64 == 0 && !staged) ? 4 : 1;
    const int64_t nj = n / chunks;  // columns per chunk (a multiple of 16 when chunks > 1)
    Pipe* pp = nullptr;
    MB200_TRY(pipe_for(ctx, (size_t)(bands + chunks), &pp));
    Pipe& P = *pp;

    // staging: all of B (as dense chunks), all of A (pitch kp), two C tiles
    const size_t sb = b_host ? align_up((size_t)k * n, 1024) : 0;
    const size_t sa = a_host ? align_up((size_t)m * kp, 1024) : 0;
    // (with column chunks, the bands that arrive after all of B are multiplied full-width: see below)
    const size_t sc = c_host ? align_up((size_t)band * n * 4, 1024) : 0;
    constexpr int nslot = 2;
    MB200_TRY(arena_reserve(ctx, ctx->staging, sb + sa + nslot * sc + 8192));
    int8_t* b_stage = b_host ? static_cast<int8_t*>(arena_take(ctx->staging, sb)) : nullptr;
    int8_t* a_stage = a_host ? static_cast<int8_t*>(arena_take(ctx->staging, sa)) : nullptr;
    int32_t* c_slot[nslot] = {nullptr, nullptr};
    for (int s = 0; s < nslot; ++s)
        if (c_host) c_slot[s] = static_cast<int32_t*>(arena_take(ctx->staging, sc));

    // B as the kernels will see it: a K x N matrix of pitch n (the staged copy of a host B, or the
    // caller's device B); chunk j is its column window [j * nj, (j + 1) * nj).
    const int64_t b_pitch = n;
    const int8_t* b_dev = b_host ? b_stage : b;
    auto b_chunk = [&](int64_t j) -> const int8_t* { return b_dev + (size_t)j * nj; };
    const bool b_direct = b_inplace_ok;  // with a host B the staged chunks are 1024-byte aligned
    const bool a_dev_direct = a_host || (kp == k && reinterpret_cast<uintptr_t>(a) % 16 == 0);
    const size_t bt_bytes = b_direct ? 0 : (size_t)n * kp, ap_bytes = a_dev_direct ? 0 : (size_t)m * kp;
    MB200_TRY(arena_reserve(ctx, ctx->scratch, align_up(bt_bytes, 1024) + align_up(ap_bytes, 1024) + 2048));

    // side streams start after everything already queued on the library's stream
    MB200_CUDA(cudaEventRecord(P.start, ctx->stream));
    MB200_CUDA(cudaStreamWaitEvent(P.in, P.start, 0));
    MB200_CUDA(cudaStreamWaitEvent(P.out, P.start, 0));

    // ---- the order of work.  A tile (band i, chunk j) can be multiplied once A band i and B
    // chunk j are on the device.  Uploads alternate between the two operands so that the set of
    // finished uploads grows as a square (t bands and t chunks give t^2 tiles: the download link
    // is fed after about two rounds, instead of after all of A as with "every band, then the
    // next chunk"); operands that are already on the device count as uploaded from the start.
    // A band that arrives when all of B is already there is multiplied full-width (chunk -1): its
    // C rows go back as one contiguous copy, which keeps the full link rate beside running kernels
    // where the strided chunk copies lose a sixth of it (16384^3: the second half of C).
    struct Step { bool is_a; int64_t idx; };
    std::vector<Step> uploads;
    std::vector<std::pair<int64_t, int64_t>> tiles;  // (band, chunk) in the order they become possible
    {
        int64_t ia = a_host ? 0 : bands, jb = b_host ? 0 : chunks;
        if (jb == chunks && chunks > 1) {
            for (int64_t i = 0; i < ia; ++i) tiles.emplace_back(i, -1);
        } else {
            for (int64_t j = 0; j < jb; ++j)
                for (int64_t i = 0; i < ia; ++i) tiles.emplace_back(i, j);
        }
        while (ia < bands || jb < chunks) {
            // B first (no product needs only A), then whichever operand is behind in proportion
            const bool take_b = jb < chunks && (ia == bands || jb == 0 || jb * bands < ia * chunks);
            if (take_b) {
                uploads.push_back({false, jb});
                for (int64_t i = 0; i < ia; ++i) tiles.emplace_back(i, jb);
                ++jb;
            } else {
                uploads.push_back({true, ia});
                if (jb == chunks && chunks > 1) {
                    tiles.emplace_back(ia, -1);
                } else {
                    for (int64_t j = 0; j < jb; ++j) tiles.emplace_back(ia, j);
                }
                ++ia;
            }
        }
    }

    // Host-side completion of staged copies: one group per upload (its event is recorded by the
    // staging thread that queues its last chunk) and one per C slot.  Before the library's
    // stream is told to wait for such an event, this thread waits until it has been recorded.
    StageStatus stage_status;
    std::vector<StageGroup> up_groups(staged ? (size_t)(bands + chunks) : 0);
    StageGroup out_groups[nslot];
    // Whatever happens below, no staging thread may still hold pointers into this call.
    struct DrainGuard {
        bool on;
        ~DrainGuard() {
            if (on) stager_drain();
        }
    } drain_guard{staged};
    const int device = ctx->device;

    // ---- uploads, all queued now on the in-stream in that order
    for (const Step& u : uploads) {
        if (!u.is_a) {
            const int64_t j = u.idx;
            cudaEvent_t ev = P.ready[bands + j];
            if (staged && b_page) {  // chunks == 1
                cudaStream_t in = P.in;
                stage_upload(device, reinterpret_cast<char*>(b_stage), (size_t)n, reinterpret_cast<const char*>(b),
                             (size_t)n, (size_t)n, (size_t)k, in, &up_groups[bands + j],
                             [ev, in] { cudaEventRecord(ev, in); }, &stage_status);
                continue;
            }
            if (chunks == 1)
                MB200_CUDA(cudaMemcpyAsync(b_stage, b, (size_t)k * n, cudaMemcpyHostToDevice, P.in));
            else  // a column window of the staged K x N copy
                MB200_CUDA(cudaMemcpy2DAsync(b_stage + (size_t)j * nj, (size_t)n, b + (size_t)j * nj, (size_t)n,
                                             (size_t)nj, (size_t)k, cudaMemcpyHostToDevice, P.in));
            MB200_CUDA(cudaEventRecord(ev, P.in));
        } else {
            const int64_t i = u.idx;
            const int64_t r0 = i * band, rows = (m - r0 < band) ? m - r0 : band;
            int8_t* dst = a_stage + (size_t)r0 * kp;
            const int8_t* src = a + (size_t)r0 * k;
            cudaEvent_t ev = P.ready[i];
            if (staged && a_page) {
                cudaStream_t in = P.in;
                stage_upload(device, reinterpret_cast<char*>(dst), (size_t)kp, reinterpret_cast<const char*>(src),
                             (size_t)k, (size_t)k, (size_t)rows, in, &up_groups[i],
                             [ev, in] { cudaEventRecord(ev, in); }, &stage_status);
                continue;
            }
            if (kp == k)
                MB200_CUDA(cudaMemcpyAsync(dst, src, (size_t)rows * k, cudaMemcpyHostToDevice, P.in));
            else  // pad to a 16-byte pitch on the way: the pad bytes are never read
                MB200_CUDA(cudaMemcpy2DAsync(dst, (size_t)kp, src, (size_t)k, (size_t)k, (size_t)rows,
                                             cudaMemcpyHostToDevice, P.in));
            MB200_CUDA(cudaEventRecord(ev, P.in));
        }
    }
    auto upload_recorded = [&](int64_t idx) {  // host wait: the event of upload `idx` exists on its stream
        if (staged) up_groups[(size_t)idx].wait();
    };

    // ---- one-off re-layouts on the library's stream
    int8_t* bt = nullptr;
    if (!b_direct) {  // chunks == 1 here
        if (b_host) {
            upload_recorded(bands);
            MB200_CUDA(cudaStreamWaitEvent(ctx->stream, P.ready[bands], 0));
        }
        bt = static_cast<int8_t*>(arena_take(ctx->scratch, bt_bytes));
        MB200_TRY(launch_transpose_i8(ctx, b_chunk(0), bt, k, n, kp));
    }
    const int8_t* a_dev = a_host ? a_stage : a;
    int64_t a_pitch = a_host ? kp : k;
    if (!a_host && !a_dev_direct) {
        int8_t* ap = static_cast<int8_t*>(arena_take(ctx->scratch, ap_bytes));
        MB200_TRY(launch_pad_rows_i8(ctx, a, ap, m, k, kp));
        a_dev = ap;
        a_pitch = kp;
    }

    // ---- products and downloads
    int64_t t = 0;  // running C tile count: picks the staging slot
    std::vector<char> a_waited((size_t)bands, 0), b_waited((size_t)chunks, 0);
    for (const auto& ij : tiles) {
        const int64_t i = ij.first, j = ij.second;
        const bool full = j < 0;  // every chunk of B is in: one product over all N columns
        const int s = (int)(t % nslot);
        const int64_t r0 = i * band, rows = (m - r0 < band) ? m - r0 : band;
        for (int64_t jj = full ? 0 : j; jj < (full ? chunks : j + 1); ++jj)
            if (b_host && b_direct && !b_waited[jj]) {
                upload_recorded(bands + jj);
                MB200_CUDA(cudaStreamWaitEvent(ctx->stream, P.ready[bands + jj], 0));
                b_waited[jj] = 1;
            }
        if (a_host && !a_waited[i]) {
            upload_recorded(i);
            MB200_CUDA(cudaStreamWaitEvent(ctx->stream, P.ready[i], 0));
            a_waited[i] = 1;
        }
        if (c_host && t >= nslot) {  // slot free
            out_groups[s].wait();
            MB200_CUDA(cudaStreamWaitEvent(ctx->stream, P.out_done[s], 0));
        }
        int32_t* c_tile = c_host ? c_slot[s] : c + (size_t)r0 * n;  // a device C is never cut into chunks
        const int8_t* a_band = a_dev + (size_t)r0 * a_pitch;
        if (b_direct)
            MB200_TRY(launch_gemm_i8_tc_bmn(ctx, a_band, full ? b_dev : b_chunk(j), c_tile, rows, full ? n : nj, k,
                                            a_pitch, b_pitch));
        else
            MB200_TRY(launch_gemm_i8_tc(ctx, a_band, bt, c_tile, rows, n, k, a_pitch, kp));
        if (c_host) {
            MB200_CUDA(cudaEventRecord(P.gemm_done[s], ctx->stream));
            MB200_CUDA(cudaStreamWaitEvent(P.out, P.gemm_done[s], 0));
            int32_t* dst = c + (size_t)r0 * n + (full ? 0 : (size_t)j * nj);
            if (staged && c_page) {  // chunks == 1: whole rows, contiguous on both sides
                cudaEvent_t ev = P.out_done[s];
                cudaStream_t out = P.out;
                stage_download(device, reinterpret_cast<char*>(dst), reinterpret_cast<const char*>(c_slot[s]),
                               (size_t)rows * n * 4, out, &out_groups[s], [ev, out] { cudaEventRecord(ev, out); },
                               &stage_status);
            } else {
                if (chunks == 1 || full)
                    MB200_CUDA(cudaMemcpyAsync(dst, c_slot[s], (size_t)rows * n * 4, cudaMemcpyDeviceToHost, P.out));
                else
                    MB200_CUDA(cudaMemcpy2DAsync(dst, (size_t)n * 4, c_slot[s], (size_t)nj * 4, (size_t)nj * 4,
                                                 (size_t)rows, cudaMemcpyDeviceToHost, P.out));
                MB200_CUDA(cudaEventRecord(P.out_done[s], P.out));
            }
        }
        ++t;
    }
    if (c_host)
        for (int s = 0; s < nslot && s < t; ++s) {
            out_groups[s].wait();
            MB200_CUDA(cudaStreamWaitEvent(ctx->stream, P.out_done[s], 0));
        }
    if (staged) stager_drain();  // the last chunks are in the caller's buffer
    MB200_CUDA(cudaStreamSynchronize(ctx->stream));
    if (stage_status.failed.load()) return fail(MIND_B200_ERR_CUDA, "a staged copy of a pageable host operand failed");
    return Call::check_err_word(ctx);
}

// ------------------------------------------------------------------ GEMMs
// The *_local functions run one call on the CURRENT device (arguments already checked).
int64_t gemm_i8_local(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n) {
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    DevLock lock(ctx->mu);
    const int g_gemm_path = tuning().gemm_path.load();
    if (k > 0 && g_gemm_path != 1 && m >= PIPE_MIN_ROWS) {
        const int64_t ah = pointer_is_host(ctx, (void*)a), bh = pointer_is_host(ctx, (void*)b),
                      ch = pointer_is_host(ctx, (void*)c);
        if (ah < 0 || bh < 0 || ch < 0) return MIND_B200_ERR_INVALID;
        if (ah || ch)
            return gemm_i8_pipelined(ctx, (const int8_t*)a, ah != 0, (const int8_t*)b, bh != 0, (int32_t*)c,
                                     ch != 0, m, k, n);
    }
    Call call(ctx);
    const int ia = call.add((void*)a, (size_t)m * k, false);
    const int ib = call.add((void*)b, (size_t)k * n, false);
    const int ic = call.add((void*)c, (size_t)m * n * 4, true);
    MB200_TRY(call.begin());
    if (k == 0) {
        MB200_CUDA(cudaMemsetAsync(call.dev<void>(ic), 0, (size_t)m * n * 4, ctx->stream));
    } else if (g_gemm_path == 1) {
        MB200_TRY(launch_gemm_i8_simt(ctx, call.dev<int8_t>(ia), call.dev<int8_t>(ib), call.dev<int32_t>(ic), m, k, n));
    } else {
        const int64_t kp = (int64_t)align_up((size_t)k, 16);
        const int8_t* da = call.dev<int8_t>(ia);
        const bool a_direct = kp == k && reinterpret_cast<uintptr_t>(da) % 16 == 0;
        // B is read in place (N-contiguous tiles) when TMA can address it: 16-byte pitch and
        // base.  Otherwise it is transposed into K-contiguous scratch first.
        const int8_t* db = call.dev<int8_t>(ib);
        const bool b_direct = !(tuning().force_transpose.load() != 0) && n % 16 == 0 && reinterpret_cast<uintptr_t>(db) % 16 == 0;
        const size_t bt_bytes = b_direct ? 0 : (size_t)n * kp, ap_bytes = a_direct ? 0 : (size_t)m * kp;
        MB200_TRY(arena_reserve(ctx, ctx->scratch, align_up(bt_bytes, 1024) + align_up(ap_bytes, 1024) + 2048));
        int8_t* bt = b_direct ? nullptr : static_cast<int8_t*>(arena_take(ctx->scratch, bt_bytes));
        if (!b_direct) MB200_TRY(launch_transpose_i8(ctx, db, bt, k, n, kp));
        if (!a_direct) {
            int8_t* ap = static_cast<int8_t*>(arena_take(ctx->scratch, ap_bytes));
            MB200_TRY(launch_pad_rows_i8(ctx, da, ap, m, k, kp));
            da = ap;
        }
        if (b_direct)
            MB200_TRY(launch_gemm_i8_tc_bmn(ctx, da, db, call.dev<int32_t>(ic), m, n, k, kp, n));
        else
            MB200_TRY(launch_gemm_i8_tc(ctx, da, bt, call.dev<int32_t>(ic), m, n, k, kp, kp));
    }
    return call.end(true);
}

int64_t gemm_i8(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n) {
    clear_error();
    MB200_TRY(check_dims(m, k, n));
    if (m == 0 || n == 0) return 0;
    if (!c || (k > 0 && (!a || !b))) return fail(MIND_B200_ERR_INVALID, "null operand");
    if (k > 0 && tuning().gemm_path.load() != 1) {
        const int64_t rc = multi_gemm_i8((const int8_t*)a, (const int8_t*)b, (int32_t*)c, m, k, n);
        if (rc != MULTI_NOT_TAKEN) return rc;
    }
    return gemm_i8_local(a, b, c, m, k, n);
}

int64_t gemm_i16_local(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n) {
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    DevLock lock(ctx->mu);
    const int g_gemm_path = tuning().gemm_path.load();
    Call call(ctx);
    const int ia = call.add((void*)a, (size_t)m * k * 2, false);
    const int ib = call.add((void*)b, (size_t)k * n * 2, false);
    const int ic = call.add((void*)c, (size_t)m * n * 4, true);
    MB200_TRY(call.begin());
    if (k == 0) {
        MB200_CUDA(cudaMemsetAsync(call.dev<void>(ic), 0, (size_t)m * n * 4, ctx->stream));
    } else if (g_gemm_path == 1) {
        MB200_TRY(launch_gemm_i16_simt(ctx, call.dev<int16_t>(ia), call.dev<int16_t>(ib), call.dev<int32_t>(ic), m, k, n));
    } else {
        const int64_t kp = (int64_t)align_up((size_t)k, 16);
        const int64_t np = (int64_t)align_up((size_t)n, 16);
        // B's limb planes keep B's own orientation ([K][np], N contiguous) unless a transposed B
        // is asked for (paths 4 / 5, and 2: the int16 kernel has no CTA-pair form).
        const bool b_transposed = (tuning().force_transpose.load() != 0) || tc_pair_forced();
        const size_t a_plane = align_up((size_t)m * kp, 1024);
        const size_t b_plane = align_up(b_transposed ? (size_t)n * kp : (size_t)k * np, 1024);
        const size_t sums = align_up((size_t)m * 4, 1024);
        MB200_TRY(arena_reserve(ctx, ctx->scratch, 2 * a_plane + 2 * b_plane + sums + 5120));
        int8_t* a_hi = static_cast<int8_t*>(arena_take(ctx->scratch, a_plane));
        uint8_t* a_lo = static_cast<uint8_t*>(arena_take(ctx->scratch, a_plane));
        int8_t* b_hi = static_cast<int8_t*>(arena_take(ctx->scratch, b_plane));
        uint8_t* b_lo = static_cast<uint8_t*>(arena_take(ctx->scratch, b_plane));
        // a = 256 * a_hi + a_lo (a_lo unsigned); b = 256 * b_hi + (b_lo' + 128) with b_lo' signed, so
        // that B's two planes share a signedness and one MMA takes both; 128 * sum_k a[i][k] goes
        // back in the epilogue.
        int32_t* a_sums = static_cast<int32_t*>(arena_take(ctx->scratch, sums));
        if (b_transposed) {
            MB200_TRY(launch_split_rows_i16(ctx, call.dev<int16_t>(ia), a_hi, a_lo, m, k, kp, false, a_sums, false,
                                            nullptr, 0));
            MB200_TRY(launch_split_transpose_i16(ctx, call.dev<int16_t>(ib), b_hi, b_lo, k, n, kp));
            MB200_TRY(launch_gemm_i16_tc(ctx, a_hi, a_lo, b_hi, b_lo, a_sums, call.dev<int32_t>(ic), m, n, k, kp));
        } else {
            if (split_i16_pair_usable(call.dev<int16_t>(ia), k, call.dev<int16_t>(ib), n)) {
                // dense, 16-divisible operands: one launch splits both and stores the row sums
                MB200_TRY(launch_split_i16_pair(ctx, call.dev<int16_t>(ia), a_hi, a_lo, a_sums, m, k,
                                                call.dev<int16_t>(ib), b_hi, b_lo, n));
            } else {
                // B first: its launch also clears the row sums that A's launch then adds into
                MB200_TRY(launch_split_rows_i16(ctx, call.dev<int16_t>(ib), b_hi, b_lo, k, n, np, true, nullptr, false,
                                                a_sums, m));
                MB200_TRY(launch_split_rows_i16(ctx, call.dev<int16_t>(ia), a_hi, a_lo, m, k, kp, false, a_sums, true,
                                                nullptr, 0));
            }
            MB200_TRY(launch_gemm_i16_tc_bmn(ctx, a_hi, a_lo, b_hi, b_lo, a_sums, call.dev<int32_t>(ic), m, n, k, kp, np));
        }
    }
    return call.end(true);
}

int64_t gemm_i16(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n) {
    clear_error();
    MB200_TRY(check_dims(m, k, n));
    if (m == 0 || n == 0) return 0;
    if (!c || (k > 0 && (!a || !b))) return fail(MIND_B200_ERR_INVALID, "null operand");
    if ((a | b) & 1) return fail(MIND_B200_ERR_INVALID, "int16 operand is not 2-byte aligned");
    if (k > 0) {
        // row bands are independent (the reference's own thread-band rule): several devices
        const int64_t rc = multi_banded(
            (const void*)a, (size_t)k * 2, (const void*)b, (size_t)k * n * 2, (void*)c, (size_t)n * 4, m,
            [=](const void* ab, void* cb, int64_t rows) { return gemm_i16_local((int64_t)ab, b, (int64_t)cb, rows, k, n); });
        if (rc != MULTI_NOT_TAKEN) return rc;
    }
    return gemm_i16_local(a, b, c, m, k, n);
}

// b_transposed: b is N x K (the identity gate's composition) instead of K x N.
int64_t gemm_q16_local(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n, bool b_transposed) {
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    DevLock lock(ctx->mu);
    const int g_gemm_path = tuning().gemm_path.load(), g_q16_mode = tuning().q16_mode.load(),
              g_q16_side_sms = tuning().q16_side_sms.load();
    const bool floor_f32 = tuning().q16_floor.load() == 0;
    const bool want_fused = floor_f32 && tuning().q16_fused.load() == 1 && g_q16_side_sms < 0;
    Call call(ctx);
    const int ia = call.add((void*)a, (size_t)m * k * 4, false);
    const int ib = call.add((void*)b, (size_t)k * n * 4, false);
    const int ic = call.add((void*)c, (size_t)m * n * 4, true);
    MB200_TRY(call.begin());
    if (k == 0) {
        MB200_CUDA(cudaMemsetAsync(call.dev<void>(ic), 0, (size_t)m * n * 4, ctx->stream));
    } else {
        const int32_t* db = call.dev<int32_t>(ib);
        // one reservation for everything this call may put in scratch: the re-transposed B and
        // the byte planes of the tensor-core hybrid
        const int64_t kp = (int64_t)align_up((size_t)k, 16), np = (int64_t)align_up((size_t)n, 16);
        const size_t a_plane = align_up((size_t)m * kp, 1024), b_plane = align_up((size_t)k * np, 1024);
        const int64_t mp = (int64_t)align_up((size_t)m, 4);
        const size_t a_low_bytes = align_up((size_t)k * mp * 4, 1024), b_low_bytes = align_up((size_t)k * np * 4, 1024);
        // measured cross-over of the single FP64-pipe kernel and the fused kernel (warm, back to back):
        // level at 256^3 (13 us both), 19.5 / 14.0 us at 384^3, 29.8 / 18.5 at 512^3, 74.8 / 32.8 at 768^3
        const bool big = (double)m * (double)n * (double)k >= 33554432.0;
        const bool hybrid_size = g_gemm_path != 1 && (g_q16_mode == 7 || (g_q16_mode == 0 && big));
        // the two-kernel forms read the operands with 16-byte loads; the fused form takes any shape and base
        const bool may_hybrid = hybrid_size && k % 4 == 0 && n % 4 == 0;
        const bool may_fuse = hybrid_size && want_fused;
        MB200_TRY(arena_reserve(ctx, ctx->scratch, (b_transposed ? align_up((size_t)k * n * 4, 1024) : 0) +
                                                       ((may_hybrid || may_fuse) ? 4 * a_plane + 4 * b_plane : 0) +
                                                       (may_fuse ? a_low_bytes + b_low_bytes : 0) + 16384));
        if (b_transposed) {
            int32_t* bkn = static_cast<int32_t*>(arena_take(ctx->scratch, (size_t)k * n * 4));
            MB200_TRY(launch_transpose_i32(ctx, db, bkn, n, k));
            db = bkn;
        }
        // Path 1 keeps the all-integer kernel (the cross-check).  Otherwise, when the operands
        // allow 16-byte loads: large products split into a linear part on the tensor cores (byte
        // planes, limb products mod 2^32) plus the per-product floor on the CUDA cores, added onto
        // it.  In the default form the linear part is a * (b >> 16) + (a >> 16) * (b & 0xffff)
        // (eleven limb products) and what is left, floor((a & 0xffff) * (b & 0xffff) / 65536), fits
        // the FP32 pipe; in the earlier form (q16_floor = 1) the linear part is a * (b >> 16) alone
        // (seven) and floor(a * (b & 0xffff) / 65536) runs on the FP64 pipe at half the rate.
        // Smaller products run the single FP64-pipe kernel (everything on the CUDA cores), where
        // three extra launches would cost more than they save.
        const int32_t* da = call.dev<int32_t>(ia);
        int32_t* dc = call.dev<int32_t>(ic);
        const bool fp64_ok = g_gemm_path != 1 && gemm_q16_fp64_usable(da, db, k, n);
        const bool fuse = may_fuse && gemm_q16_fused_usable(ctx);
        const bool hybrid = fuse || (fp64_ok && may_hybrid && reinterpret_cast<uintptr_t>(dc) % 16 == 0);
        if (hybrid) {
            uint8_t* ap[4];
            uint8_t* bp[4] = {nullptr, nullptr, nullptr, nullptr};
            for (int i = 0; i < 4; ++i) ap[i] = static_cast<uint8_t*>(arena_take(ctx->scratch, a_plane));
            for (int i = 0; i < (floor_f32 ? 4 : 2); ++i) bp[i] = static_cast<uint8_t*>(arena_take(ctx->scratch, b_plane));
            // One kernel for both halves (gemm_q16_fused.cu) where it can run: the limb products
            // hide behind the FMAs of the floor term on the same SM, and C is written once.  Its
            // operand split pads every plane, so ragged shapes and odd bases take this path too.
            if (fuse) {
                float* a_low_t = static_cast<float*>(arena_take(ctx->scratch, a_low_bytes));
                float* b_low = static_cast<float*>(arena_take(ctx->scratch, b_low_bytes));
                MB200_TRY(launch_split_q16_ab(ctx, da, db, ap, bp, a_low_t, b_low, dc,
                                              gemm_q16_fused_shares_tiles(ctx, m, n, k), m, k, n, kp, np, mp));
                MB200_TRY(launch_gemm_q16_fused(ctx, ap, bp, a_low_t, b_low, dc, m, n, k, kp, np, mp, np));
                return call.end(true);
            }
            const int b_what = floor_f32 ? 2 : 1;
            auto launch_floor = [&](int max_blocks) {
                return floor_f32 ? launch_gemm_q16_floor_f32(ctx, da, db, dc, m, k, n, max_blocks)
                                 : launch_gemm_q16_floor_add(ctx, da, db, dc, m, k, n, max_blocks);
            };
            // Products up to 2^31 (1024^3 is 2^30): the tensor-core half is latency-bound (a few
            // k-blocks per tile, fewer tiles than SMs), so the two halves run side by side: c is
            // zeroed, the byte split and the tensor-core kernel go to a second stream on a few SMs,
            // the floor kernel keeps the rest, and both add onto c with red.global.add (sums mod
            // 2^32 commute).  Measured at 1024^3 with the FP32 floor kernel: 86 us with 32 SMs for
            // the tensor-core half (8 / 16 / 24 / 48 SMs: 203 / 116 / 93 / 95 us) against 103 us in
            // sequence; from 2048^3 up the sequence is as fast or faster (525 / 530 us at 2048^3).
            // With the FP64 floor kernel, which takes twice as long: 16 SMs, 113 us against 121 us.
            // In sequence the tensor-core half runs 64-column tiles when it has fewer 128 x 128 tiles
            // than SMs.
            const double work = (double)m * (double)n * (double)k;
            // (not with a short K: there the outputs dominate, and side by side every output is an atomic)
            const int side_sms = g_q16_side_sms >= 0 ? g_q16_side_sms : (work <= 2147483648.0 && k >= 512 ? (floor_f32 ? 32 : 16) : 0);
            if (side_sms > 0 && side_sms < ctx->sm_count) {
                MB200_CUDA(cudaMemsetAsync(dc, 0, (size_t)m * n * 4, ctx->stream));
                MB200_CUDA(cudaEventRecord(ctx->fork_ev, ctx->stream));
                MB200_CUDA(cudaStreamWaitEvent(ctx->side, ctx->fork_ev, 0));
                // the long kernel first, so that a lone call does not start it behind the host work
                // of the three short launches
                int64_t rc = launch_floor(ctx->sm_count - side_sms);
                cudaStream_t main_stream = ctx->stream;
                const bool profiling = ctx->profile;
                ctx->stream = ctx->side;  // the launchers below use the context's stream
                ctx->profile = false;     // kernel timing covers the FP64 kernel, which spans the call
                if (!rc) rc = launch_split_i32_bytes(ctx, da, ap, 0, m, k, kp);
                if (!rc) rc = launch_split_i32_bytes(ctx, db, bp, b_what, k, n, np);
                if (!rc) rc = launch_gemm_q16_linear_tc(ctx, ap, bp, dc, m, n, k, kp, np, true, side_sms);
                ctx->stream = main_stream;
                ctx->profile = profiling;
                // join even after a failed launch, so that the side stream never outlives the call
                MB200_CUDA(cudaEventRecord(ctx->join_ev, ctx->side));
                MB200_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->join_ev, 0));
                if (rc) return rc;
                return call.end(true);
            }
            MB200_TRY(launch_split_i32_bytes(ctx, da, ap, 0, m, k, kp));
            MB200_TRY(launch_split_i32_bytes(ctx, db, bp, b_what, k, n, np));
            MB200_TRY(launch_gemm_q16_linear_tc(ctx, ap, bp, dc, m, n, k, kp, np, false, 0));
            MB200_TRY(launch_floor(0));
            return call.end(true);
        }
        if (fp64_ok)
            MB200_TRY(launch_gemm_q16_fp64(ctx, da, db, dc, m, k, n));
        else
            MB200_TRY(launch_gemm_q16(ctx, da, db, dc, m, k, n));
    }
    return call.end();
}

int64_t gemm_q16(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n, bool b_transposed) {
    clear_error();
    MB200_TRY(check_dims(m, k, n));
    if (m == 0 || n == 0) return 0;
    if (!c || (k > 0 && (!a || !b))) return fail(MIND_B200_ERR_INVALID, "null operand");
    if ((a | b | c) & 3) return fail(MIND_B200_ERR_INVALID, "int32 operand is not 4-byte aligned");
    if (k > 0) {
        const int64_t rc = multi_banded(
            (const void*)a, (size_t)k * 4, (const void*)b, (size_t)k * n * 4, (void*)c, (size_t)n * 4, m,
            [=](const void* ab, void* cb, int64_t rows) {
                return gemm_q16_local((int64_t)ab, b, (int64_t)cb, rows, k, n, b_transposed);
            });
        if (rc != MULTI_NOT_TAKEN) return rc;
    }
    return gemm_q16_local(a, b, c, m, k, n, b_transposed);
}

// ------------------------------------------------------------ row reductions
// kind: 0 = Q16.16 matrix x vector, 1 = int16 matrix x vector.
int64_t gemv_local(int kind, int64_t w, int64_t x, int64_t y, int64_t rows, int64_t cols) {
    const int es = kind == 0 ? 4 : 2;
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    DevLock lock(ctx->mu);
    Call call(ctx);
    const int iw = call.add((void*)w, (size_t)rows * cols * es, false);
    const int ix = call.add((void*)x, (size_t)cols * es, false);
    const int iy = call.add((void*)y, (size_t)rows * 4, true);
    MB200_TRY(call.begin());
    if (kind == 0)
        MB200_TRY(launch_gemv_q16(ctx, call.dev<int32_t>(iw), call.dev<int32_t>(ix), call.dev<int32_t>(iy), rows, cols));
    else
        MB200_TRY(launch_gemv_i16(ctx, call.dev<int16_t>(iw), call.dev<int16_t>(ix), call.dev<int32_t>(iy), rows, cols));
    return call.end();
}

int64_t gemv(int kind, int64_t w, int64_t x, int64_t y, int64_t rows, int64_t cols) {
    clear_error();
    if (rows < 0 || cols < 0) return fail(MIND_B200_ERR_INVALID, "negative dimension");
    if (rows == 0) return 0;
    if (!y || (cols > 0 && (!w || !x))) return fail(MIND_B200_ERR_INVALID, "null operand");
    const int es = kind == 0 ? 4 : 2;
    if (((w | x) & (es - 1)) || (y & 3)) return fail(MIND_B200_ERR_INVALID, "misaligned operand");
    if (cols > 0) {
        const int64_t rc = multi_banded(
            (const void*)w, (size_t)cols * es, (const void*)x, (size_t)cols * es, (void*)y, 4, rows,
            [=](const void* wb, void* yb, int64_t r) { return gemv_local(kind, (int64_t)wb, x, (int64_t)yb, r, cols); });
        if (rc != MULTI_NOT_TAKEN) return rc;
    }
    return gemv_local(kind, w, x, y, rows, cols);
}

// kind: 0 = Q16.16 dot, 1 = int16 dot, 2 = Q16.16 L1 distance.  Returns the value;
// failures leave a message and return 0 (the reference's dot returns 0 on bad input).
int64_t dot(int kind, int64_t a, int64_t b, int64_t len) {
    clear_error();
    if (len <= 0 || !a || !b) return 0;
    const int es = kind == 1 ? 2 : 4;
    if ((a | b) & (es - 1)) {
        fail(MIND_B200_ERR_INVALID, "misaligned operand");
        return 0;
    }
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return 0;
    DevLock lock(ctx->mu);
    // The kernel writes the scalar straight into mapped pinned memory: no staging, no copy back.
    Call call(ctx);
    const int ia = call.add((void*)a, (size_t)len * es, false);
    const int ib = call.add((void*)b, (size_t)len * es, false);
    if (call.begin() != 0) return 0;
    int32_t* out = ctx->scalar_dev;
    int64_t st;
    if (kind == 0)
        st = launch_gemv_q16(ctx, call.dev<int32_t>(ia), call.dev<int32_t>(ib), out, 1, len);
    else if (kind == 1)
        st = launch_gemv_i16(ctx, call.dev<int16_t>(ia), call.dev<int16_t>(ib), out, 1, len);
    else
        st = launch_dist_l1_q16(ctx, call.dev<int32_t>(ia), call.dev<int32_t>(ib), out, len);
    if (st != 0 || call.end() != 0) return 0;
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) {  // device operands: end() did not wait
        fail(MIND_B200_ERR_CUDA, "synchronisation failed: %s", cudaGetErrorString(cudaGetLastError()));
        return 0;
    }
    const int32_t result = *reinterpret_cast<volatile int32_t*>(ctx->scalar_host);
    return (int64_t)result;
}

}  // namespace
}  // namespace mb200

using namespace mb200;

extern "C" {

int64_t __mind_blas_matmul_mm_i8_v(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n) { return gemm_i8(a, b, c, m, k, n); }
int64_t __mind_blas_matmul_mm_i8_mt_v(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n) { return gemm_i8(a, b, c, m, k, n); }
int64_t __mind_blas_matmul_mm_q16_v(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n) { return gemm_q16(a, b, c, m, k, n, false); }
int64_t __mind_blas_matmul_mm_q16_mt_v(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n) { return gemm_q16(a, b, c, m, k, n, false); }
int64_t __mind_b200_matmul_mm_i16(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n) { return gemm_i16(a, b, c, m, k, n); }
int64_t __mind_blas_gemv_q16_mt(int64_t w, int64_t x, int64_t y, int64_t m, int64_t k) { return gemv(0, w, x, y, m, k); }
int64_t __mind_blas_matmul_rmajor_q16_v(int64_t w, int64_t x, int64_t y, int64_t rows, int64_t cols) { return gemv(0, w, x, y, rows, cols); }
int64_t __mind_blas_matmul_rmajor_i16_v(int64_t w, int64_t x, int64_t y, int64_t rows, int64_t cols) { return gemv(1, w, x, y, rows, cols); }
int64_t __mind_blas_dot_q16_v(int64_t a, int64_t b, int64_t len) { return dot(0, a, b, len); }
int64_t __mind_blas_dot_i16_v(int64_t a, int64_t b, int64_t len) { return dot(1, a, b, len); }
int64_t __mind_blas_dot_l1_q16_v(int64_t a, int64_t b, int64_t len) { return dot(2, a, b, len); }

int64_t dotq(int64_t a, int64_t b, int64_t n) { return dot(0, a, b, n); }
int64_t dotl1q(int64_t a, int64_t b, int64_t n) { return dot(2, a, b, n); }
int64_t doti16(int64_t a, int64_t b, int64_t n) { return dot(1, a, b, n); }
int64_t mmq(int64_t w, int64_t x, int64_t y, int64_t rows, int64_t cols) { return gemv(0, w, x, y, rows, cols); }
int64_t mmi16(int64_t w, int64_t x, int64_t y, int64_t rows, int64_t cols) { return gemv(1, w, x, y, rows, cols); }
int64_t gemvq(int64_t w, int64_t x, int64_t y, int64_t m, int64_t k) { return gemv(0, w, x, y, m, k); }
int64_t gemmq(int64_t a, int64_t bt, int64_t c, int64_t m, int64_t k, int64_t n) { return gemm_q16(a, bt, c, m, k, n, true); }
int64_t gemmq_kn(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n) { return gemm_q16(a, b, c, m, k, n, false); }
int64_t gemmqmm(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n) { return gemm_q16(a, b, c, m, k, n, false); }
int64_t gemmi8(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n) { return gemm_i8(a, b, c, m, k, n); }
int64_t gemmi8mt(int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n) { return gemm_i8(a, b, c, m, k, n); }

const char* mind_b200_last_error(void) { return last_error_cstr(); }

int64_t mind_b200_set_stream(int64_t cuda_stream) {
    clear_error();
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    DevLock lock(ctx->mu);
    cudaStream_t next = reinterpret_cast<cudaStream_t>(cuda_stream);
    if (next == ctx->stream) return 0;
    // Device-pointer calls are asynchronous and share the per-device scratch, so work queued on
    // the new stream must not start before what is still queued on the old one: the new stream
    // waits for an event recorded on the old one.  Not while either is being captured (an event
    // cannot cross a capture boundary): synchronise yourself before switching streams there.
    cudaStreamCaptureStatus c0 = cudaStreamCaptureStatusNone, c1 = cudaStreamCaptureStatusNone;
    const bool q0 = cudaStreamIsCapturing(ctx->stream, &c0) == cudaSuccess;
    const bool q1 = cudaStreamIsCapturing(next, &c1) == cudaSuccess;
    if (q0 && q1 && c0 == cudaStreamCaptureStatusNone && c1 == cudaStreamCaptureStatusNone) {
        if (cudaEventRecord(ctx->order_ev, ctx->stream) == cudaSuccess)
            cudaStreamWaitEvent(next, ctx->order_ev, 0);
    }
    cudaGetLastError();  // an old stream the caller has destroyed has nothing left to order after
    ctx->stream = next;
    return 0;
}

int64_t mind_b200_synchronize(void) {
    clear_error();
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    DevLock lock(ctx->mu);
    MB200_CUDA(cudaStreamSynchronize(ctx->stream));
    return Call::check_err_word(ctx);
}

int64_t mind_b200_device_count(void) { return usable_device_count(); }
int64_t mind_b200_kernel_launches(void) { return launches(); }

int64_t mind_b200_reserve(int64_t scratch_bytes, int64_t staging_bytes) {
    clear_error();
    if (scratch_bytes < 0 || staging_bytes < 0) return fail(MIND_B200_ERR_INVALID, "negative size");
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    DevLock lock(ctx->mu);
    MB200_TRY(arena_reserve(ctx, ctx->scratch, (size_t)scratch_bytes));
    MB200_TRY(arena_reserve(ctx, ctx->staging, (size_t)staging_bytes));
    return 0;
}

int64_t mind_b200_set_gemm_path(int64_t path) {
    clear_error();
    if (path < 0 || path > 14)
        return fail(MIND_B200_ERR_INVALID, "gemm path must be 0 (auto), 1 (CUDA cores), 2 / 3 (CTA pairs / single CTA), 4 / 5 (the same with B transposed first), 6 / 7 (Q16.16: FP64-pipe kernel alone / tensor-core hybrid), 8 / 9 (the hybrid with its halves in sequence / side by side) 10 / 11 (int8: the narrow-tile kernel always / never) 12 / 13 (int8: the 256 x 512-tile pair kernel always / never) or 14 (Q16.16: the hybrid with its floor term on the FP64 pipe)");
    Tuning& t = tuning();
    t.force_transpose = (path == 4 || path == 5) ? 1 : 0;
    t.q16_mode = path == 6 ? 6 : ((path >= 7 && path <= 9) || path == 14) ? 7 : 0;
    t.q16_floor = path == 14 ? 1 : 0;
    t.q16_fused = (path == 8 || path == 9 || path == 14) ? 0 : 1;
    t.q16_side_sms = path == 8 ? 0 : path == 9 ? 32 : -1;
    t.small_tile = path == 10 ? 1 : (path == 0 ? -1 : 0);
    t.wide_pair = path == 12 ? 1 : (path == 0 ? -1 : 0);
    t.gemm_path = path == 1 ? 1 : 0;
    t.pair_mode = (path == 2 || path == 4) ? 2 : (path == 3 || path == 5) ? 1 : 0;
    return 0;
}

int64_t mind_b200_set_tile_order(int64_t group_m, int64_t raster) {
    clear_error();
    if (group_m < 0 || group_m > 64 || raster < 0 || raster > 3) return fail(MIND_B200_ERR_INVALID, "bad tile order");
    // (raster 3 = default order, with the epilogue in its row-store form instead of TMA stores: a measurement knob)
    tuning().group_m = (int)group_m;
    tuning().raster = (int)raster;
    return 0;
}

int64_t mind_b200_set_devices(int64_t count) {
    clear_error();
    return multi_set_devices(count);
}

int64_t mind_b200_devices(void) { return multi_device_count(); }

int64_t mind_b200_shutdown(void) {
    clear_error();
    multi_shutdown();
    stager_shutdown();
    destroy_all_contexts();
    return 0;
}

int64_t mind_b200_selftest_wait_timeout(int64_t limit_ms) {
    clear_error();
    if (limit_ms < 1 || limit_ms > 1000) return fail(MIND_B200_ERR_INVALID, "limit must be 1..1000 ms");
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    DevLock lock(ctx->mu);
    MB200_TRY(launch_wait_selftest(ctx, limit_ms));
    MB200_CUDA(cudaStreamSynchronize(ctx->stream));
    return Call::check_err_word(ctx);
}

int64_t mind_b200_profile(int64_t enable) {
    clear_error();
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    DevLock lock(ctx->mu);
    ctx->profile = enable != 0;
    ctx->prof_count = 0;
    return 0;
}

int64_t mind_b200_profile_read(int64_t* launches_out, double* total_ms_out) {
    clear_error();
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    DevLock lock(ctx->mu);
    MB200_CUDA(cudaStreamSynchronize(ctx->stream));
    double total = 0.0;
    for (int i = 0; i < ctx->prof_count; ++i) {
        float ms = 0.f;
        MB200_CUDA(cudaEventElapsedTime(&ms, ctx->prof_ev[2 * i], ctx->prof_ev[2 * i + 1]));
        total += ms;
    }
    if (launches_out) *launches_out = ctx->prof_count;
    if (total_ms_out) *total_ms_out = total;
    ctx->prof_count = 0;
    return 0;
}

int64_t mind_b200_set_q16_split(int64_t side_sms) {
    clear_error();
    if (side_sms < -1 || side_sms > 1024) return fail(MIND_B200_ERR_INVALID, "bad SM count");
    tuning().q16_side_sms = (int)side_sms;
    return 0;
}

int64_t mind_b200_fp32_fma_peak(double* fma_per_s_out, double* sm_mhz_out) {
    clear_error();
    if (!fma_per_s_out) return fail(MIND_B200_ERR_INVALID, "null output");
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    DevLock lock(ctx->mu);
    return measure_fp32_fma_peak(ctx, fma_per_s_out, sm_mhz_out);
}

int64_t mind_b200_fp64_fma_peak(double* fma_per_s_out, double* sm_mhz_out) {
    clear_error();
    if (!fma_per_s_out) return fail(MIND_B200_ERR_INVALID, "null output");
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    DevLock lock(ctx->mu);
    return measure_fp64_fma_peak(ctx, fma_per_s_out, sm_mhz_out);
}

int64_t mind_b200_lcg_fill(int64_t dst, int64_t n, int64_t kind, int64_t seed, int64_t offset, int64_t shift) {
    clear_error();
    if (n < 0 || kind < 0 || kind > 2 || shift < 0 || shift > 31) return fail(MIND_B200_ERR_INVALID, "bad argument");
    if (n == 0) return 0;
    if (!dst) return fail(MIND_B200_ERR_INVALID, "null destination");
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    DevLock lock(ctx->mu);
    const size_t es = kind == 0 ? 4 : (kind == 1 ? 1 : 2);
    Call call(ctx);
    const int id = call.add((void*)dst, (size_t)n * es, true);
    MB200_TRY(call.begin());
    MB200_TRY(launch_lcg_fill(ctx, call.dev<void>(id), n, (int)kind, (uint64_t)seed, (uint64_t)offset, (int)shift));
    return call.end();
}

int64_t mind_b200_matvec_wrap(int64_t mat, int64_t elem_bytes, int64_t rows, int64_t cols, int64_t v, int64_t out) {
    clear_error();
    if (rows < 0 || cols < 0) return fail(MIND_B200_ERR_INVALID, "negative dimension");
    if (rows == 0) return 0;
    if (!out || (cols > 0 && (!mat || !v))) return fail(MIND_B200_ERR_INVALID, "null operand");
    if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4) return fail(MIND_B200_ERR_INVALID, "elem_bytes must be 1, 2 or 4");
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    DevLock lock(ctx->mu);
    Call call(ctx);
    const int im = call.add((void*)mat, (size_t)rows * cols * elem_bytes, false);
    const int iv = call.add((void*)v, (size_t)cols * 4, false);
    const int io = call.add((void*)out, (size_t)rows * 4, true);
    MB200_TRY(call.begin());
    MB200_TRY(launch_matvec_wrap(ctx, call.dev<void>(im), (int)elem_bytes, rows, cols, call.dev<int32_t>(iv), call.dev<int32_t>(io)));
    return call.end();
}

}  // extern "C"
