// Pageable host operands: host threads that move them through pinned slots.
//
// The reference's callers pass ordinary heap buffers (a Rust Vec, benches/det_matmul_i8.rs:282-297).
// cudaMemcpyAsync on such memory is staged by the driver in the calling thread, one chunk at a
// time, and returns only when the chunk is on its way: a large call then runs at the speed of one
// core's memcpy and nothing overlaps.  Here a small team of host threads does the staging: each
// thread copies a chunk into a pinned slot of its own and queues the DMA itself (uploads), or
// queues the DMA into its slot, waits for it and copies the chunk out to the caller's buffer
// (downloads).  Two teams, one per direction, so that downloads of finished rows run beside the
// uploads still to come.  A group of chunks can name an action for whichever thread finishes it
// last (recording the CUDA event that the kernels wait for), and the submitting thread can wait
// on the host until that has happened.
//
// The slots are pinned once (first pageable call) and freed at shutdown.  Upload slots are
// write-combined (the host only writes them; measured 41.5 - 42.9 ms against 44.5 - 46.4 ms for the
// 16384^3 int8 call with pageable operands, same host, alternating runs); download slots are not
// (the host reads them).
#include <condition_variable>
#include <deque>
#include <stdlib.h>
#include <string.h>
#include <thread>

#include "common.h"

namespace mb200 {
namespace {

constexpr size_t SLOT_BYTES = (size_t)4 << 20;
constexpr int SLOTS_PER_THREAD = 2;
constexpr int MAX_THREADS_PER_TEAM = 16;

// Threads per direction: MINDB200_STAGE_THREADS (1..16); default half the host's cores, at most 8
// (measured on a 16-core host, 1 GiB through 4 MiB slots: 4 threads 25 GB/s up / 28 down,
// 8 threads 41 / 36, 16 threads 47 / 39; the driver's own staging of a pageable
// cudaMemcpyAsync stays at 11 / 18 GB/s however many threads issue the copies).
int threads_per_team() {
    const char* e = getenv("MINDB200_STAGE_THREADS");
    long v = e && *e ? strtol(e, nullptr, 10) : 0;
    if (v <= 0) {
        v = (long)std::thread::hardware_concurrency() / 2;
        if (v > 8) v = 8;
    }
    return v < 1 ? 1 : v > MAX_THREADS_PER_TEAM ? MAX_THREADS_PER_TEAM : (int)v;
}

constexpr int MAX_DEV = 64;

struct Slot {
    char* ptr = nullptr;
    // One event per device (an event can only be recorded on a stream of the device it was made
    // on), made on first use; `last` names the one recorded after the slot's latest DMA.
    cudaEvent_t ev[MAX_DEV] = {};
    int last = -1;
    // With `device` current: the event to record behind a DMA that uses this slot.
    cudaEvent_t event_for(int device) {
        if (!ev[device] && cudaEventCreateWithFlags(&ev[device], cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        last = device;
        return ev[device];
    }
};

class Team {
public:
    // task(slot): runs on a team thread; must leave slot.ev recorded behind any DMA it queued on the slot
    void submit(std::function<void(Slot&)> task) {
        {
            std::lock_guard<std::mutex> lk(mu_);
            queue_.push_back(std::move(task));
            ++open_;
        }
        cv_.notify_one();
    }
    void drain() {
        std::unique_lock<std::mutex> lk(mu_);
        idle_.wait(lk, [&] { return open_ == 0; });
    }
    // write_combined: for slots the CPU only WRITES (uploads): streaming stores on the host side,
    // no cache snoops on the DMA side.  Never for slots the CPU reads.
    bool start(bool write_combined = false) {
        std::lock_guard<std::mutex> lk(mu_);
        if (started_) return ok_;
        started_ = true;
        ok_ = true;
        n_threads_ = threads_per_team();
        for (int t = 0; t < n_threads_ && ok_; ++t)
            for (int s = 0; s < SLOTS_PER_THREAD; ++s) {
                Slot& sl = slots_[t][s];
                if (cudaHostAlloc(&sl.ptr, SLOT_BYTES,
                                  cudaHostAllocPortable | (write_combined ? cudaHostAllocWriteCombined : 0)) != cudaSuccess) {
                    cudaGetLastError();
                    ok_ = false;
                    break;
                }
            }
        if (ok_) {
            stop_ = false;
            for (int t = 0; t < n_threads_; ++t) threads_[t] = std::thread([this, t] { run(t); });
        }
        return ok_;
    }
    void stop() {
        {
            std::lock_guard<std::mutex> lk(mu_);
            if (!started_) return;
            stop_ = true;
        }
        cv_.notify_all();
        for (auto& th : threads_)
            if (th.joinable()) th.join();
        for (auto& per_thread : slots_)
            for (Slot& sl : per_thread) {
                if (sl.ptr) cudaFreeHost(sl.ptr);
                for (cudaEvent_t e : sl.ev)
                    if (e) cudaEventDestroy(e);
                sl = Slot();
            }
        cudaGetLastError();
        std::lock_guard<std::mutex> lk(mu_);
        started_ = false;
    }

private:
    void run(int t) {
        int use = 0;
        for (;;) {
            std::function<void(Slot&)> task;
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return stop_ || !queue_.empty(); });
                if (queue_.empty()) return;  // stop_ and nothing left
                task = std::move(queue_.front());
                queue_.pop_front();
            }
            Slot& sl = slots_[t][use++ % SLOTS_PER_THREAD];
            if (sl.last >= 0) cudaEventSynchronize(sl.ev[sl.last]);  // the slot's previous DMA
            task(sl);
            {
                std::lock_guard<std::mutex> lk(mu_);
                if (--open_ == 0) idle_.notify_all();
            }
        }
    }
    std::mutex mu_;
    std::condition_variable cv_, idle_;
    std::deque<std::function<void(Slot&)>> queue_;
    std::thread threads_[MAX_THREADS_PER_TEAM];
    Slot slots_[MAX_THREADS_PER_TEAM][SLOTS_PER_THREAD];
    int n_threads_ = 0;
    int open_ = 0;
    bool started_ = false, ok_ = false, stop_ = false;
};

// Heap objects that no static destructor touches (the library's own destructor stops them).
Team& up_team() {
    static Team* t = new Team;
    return *t;
}
Team& down_team() {
    static Team* t = new Team;
    return *t;
}

}  // namespace

void StageGroup::arm(int chunks, std::function<void()> on_last) {
    std::lock_guard<std::mutex> lk(mu);
    left = chunks;
    done = chunks == 0;
    last = std::move(on_last);
    if (done && last) last();
}

void StageGroup::finish_one() {
    std::function<void()> fire;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (--left != 0) return;
        fire = std::move(last);
    }
    if (fire) fire();
    {
        std::lock_guard<std::mutex> lk(mu);
        done = true;
    }
    cv.notify_all();
}

void StageGroup::wait() {
    std::unique_lock<std::mutex> lk(mu);
    cv.wait(lk, [&] { return done; });
}

bool stager_start() { return up_team().start(true) && down_team().start(false); }

size_t stager_slot_bytes() { return SLOT_BYTES; }

void stager_shutdown() {
    up_team().stop();
    down_team().stop();
}

void stager_drain() {
    up_team().drain();
    down_team().drain();
}

bool host_pointer_is_pageable(const void* p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return true;
    }
    return at.type == cudaMemoryTypeUnregistered;
}

// rows x width bytes from pageable src (row pitch spitch) to device dst (row pitch dpitch >= width).
// Returns at once; `group` fires when every chunk's DMA has been queued on `stream`.
void stage_upload(int device, char* dst, size_t dpitch, const char* src, size_t spitch, size_t width, size_t rows,
                  cudaStream_t stream, StageGroup* group, std::function<void()> on_last, StageStatus* status) {
    const size_t rows_per = SLOT_BYTES / dpitch ? SLOT_BYTES / dpitch : 1;
    const int chunks = (int)((rows + rows_per - 1) / rows_per);
    group->arm(chunks, std::move(on_last));
    for (size_t r0 = 0; r0 < rows; r0 += rows_per) {
        const size_t nr = rows - r0 < rows_per ? rows - r0 : rows_per;
        up_team().submit([=](Slot& sl) {
            if (cudaSetDevice(device) != cudaSuccess) status->fail("cudaSetDevice");
            if (dpitch == spitch && spitch == width) {
                memcpy(sl.ptr, src + r0 * spitch, nr * width);
            } else {
                for (size_t r = 0; r < nr; ++r) memcpy(sl.ptr + r * dpitch, src + (r0 + r) * spitch, width);
            }
            const size_t bytes = (nr - 1) * dpitch + width;  // the last row's pad is not copied
            cudaEvent_t ev = sl.event_for(device);
            if (!ev || cudaMemcpyAsync(dst + r0 * dpitch, sl.ptr, bytes, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
                cudaEventRecord(ev, stream) != cudaSuccess)
                status->fail("staged upload");
            group->finish_one();
        });
    }
}

// `bytes` contiguous bytes from device src to pageable dst.  The DMAs are queued on `stream` (order
// it behind the producer first); `group` fires when the last DMA has been QUEUED (the device source
// may be reused once what is queued on `stream` so far has run); the copy out to dst completes later
// (stager_drain).
void stage_download(int device, char* dst, const char* src, size_t bytes, cudaStream_t stream, StageGroup* group,
                    std::function<void()> on_last, StageStatus* status) {
    const int chunks = (int)((bytes + SLOT_BYTES - 1) / SLOT_BYTES);
    group->arm(chunks, std::move(on_last));
    for (size_t off = 0; off < bytes; off += SLOT_BYTES) {
        const size_t nb = bytes - off < SLOT_BYTES ? bytes - off : SLOT_BYTES;
        down_team().submit([=](Slot& sl) {
            if (cudaSetDevice(device) != cudaSuccess) status->fail("cudaSetDevice");
            cudaEvent_t ev = sl.event_for(device);
            const bool ok = ev && cudaMemcpyAsync(sl.ptr, src + off, nb, cudaMemcpyDeviceToHost, stream) == cudaSuccess &&
                            cudaEventRecord(ev, stream) == cudaSuccess;
            group->finish_one();
            if (!ok || cudaEventSynchronize(ev) != cudaSuccess) {
                status->fail("staged download");
                return;
            }
            memcpy(dst + off, sl.ptr, nb);
        });
    }
}

}  // namespace mb200
