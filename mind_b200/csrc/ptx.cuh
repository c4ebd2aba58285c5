// Thin inline-PTX wrappers for the sm_100a features the GEMM kernels use:
// mbarrier, TMA (cp.async.bulk.tensor, never with cluster multicast), and the
// tcgen05 family (TMEM allocation, MMA, commit, TMEM loads, fences).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mb200 {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// Arrive on the barrier at the same offset in CTA `cta` of this cluster.  Relaxed: the
// arrival orders nothing but itself (callers fence tcgen05 traffic explicitly), so it
// does not wait for this thread's global stores to drain.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t cta) {
    asm volatile(
        "{\n\t.reg .b32 r;\n\t"
        "mapa.shared::cluster.u32 r, %0, %1;\n\t"
        "mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [r];\n\t}" ::"r"(bar),
        "r"(cta)
        : "memory");
}
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
    return r;
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wait on an mbarrier phase, bounded in time.  When the limit runs out the waiter raises the
// CTA's abort flag and records `code` in the device error word (first failure wins); every other
// waiter of the CTA sees the flag within 64 polls and gives up too.  Returns false on giving up.
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_s,
                                             int* err_g, int code,
                                             unsigned long long limit_ns = WAIT_LIMIT_NS) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63u) == 0u) {
            if (*abort_s) return false;
            if (globaltimer_ns() - t0 > limit_ns) {
                *abort_s = 1;
                atomicCAS(err_g, 0, code);
                return false;
            }
        }
    }
}

// The same wait for a thread that goes on to READ, with ordinary loads, the shared memory the
// barrier guards.  Returns `one` (any non-zero value the compiler cannot know: a kernel parameter)
// on success and 0 on giving up; the caller folds (result - one) into the address of those loads,
// which makes them data-dependent on the outcome of the wait.  The acquire of try_wait orders
// them already; the dependency keeps that order out of the instruction scheduler's hands (on the
// release side of the same pipeline an order left to it was seen to fail: gemm_q16_fused.cu).
__device__ __forceinline__ uint32_t mbar_try_wait_dep(uint32_t bar, uint32_t parity, uint32_t one) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, %3, 0, p;\n\t}"
        : "=r"(r)
        : "r"(bar), "r"(parity), "r"(one)
        : "memory");
    return r;
}
__device__ __forceinline__ uint32_t wait_bounded_dep(uint32_t bar, uint32_t parity, volatile int* abort_s, int* err_g,
                                                     int code, uint32_t one,
                                                     unsigned long long limit_ns = WAIT_LIMIT_NS) {
    uint32_t r = mbar_try_wait_dep(bar, parity, one);
    if (r) return r;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        r = mbar_try_wait_dep(bar, parity, one);
        if (r) return r;
        if ((++spins & 63u) == 0u) {
            if (*abort_s) return 0u;
            if (globaltimer_ns() - t0 > limit_ns) {
                *abort_s = 1;
                atomicCAS(err_g, 0, code);
                return 0u;
            }
        }
    }
}

// Registers per thread of the calling warpgroup (four consecutive warps, all of which must
// execute this together): give some back to the CTA's pool, or take more from it (waits until
// the pool has them).  N is a multiple of 8.
template <int N>
__device__ __forceinline__ void regs_release() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void regs_take() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// ----------------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tensormap(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// 2-D tiled load, global -> this CTA's shared memory; completion bytes land on `bar`.
// `policy` is an L2 eviction policy made by l2_policy().
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int32_t x,
                                            int32_t y, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%3, %4}], [%2], %5;" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "l"(policy)
        : "memory");
}
// L2 eviction policy for a whole operand: 0 = normal, 1 = keep (evict last), 2 = stream (evict first).
__device__ __forceinline__ uint64_t l2_policy(int kind) {
    uint64_t pol;
    if (kind == 1)
        asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    else if (kind == 2)
        asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    else
        asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
// Same, issued from either CTA of a pair; `bar` is a shared::cluster address and
// may name the barrier of the peer CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tmap, uint32_t bar,
                                                 int32_t x, int32_t y, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%3, %4}], [%2], %5;" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "l"(policy)
        : "memory");
}

// 2-D tiled store, this CTA's shared memory -> global (rows and columns outside the tensor are
// clipped by the hardware).  Completion is tracked by the issuing thread's bulk async-group.
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(src), "r"(x), "r"(y)
                 : "memory");
}
// The same, adding the tile onto what global memory holds (element type from the tensor map;
// the additions are performed in L2, atomically per element).
__device__ __forceinline__ void tma_reduce_add_2d(const void* tmap, uint32_t src, int32_t x, int32_t y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(src), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until at most N of this thread's bulk groups still have to READ their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Until at most N of this thread's bulk groups are still in flight at all.
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Makes this thread's earlier shared-memory writes visible to the TMA engine (async proxy).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// ------------------------------------------------- programmatic dependent launch
// No-ops unless the kernel was launched with the programmatic-stream-serialization attribute.
// launch_dependents: the next kernel in the stream may start (and run up to its own wait).
// wait: blocks until the previous kernel has completed and its writes are visible.
__device__ __forceinline__ void griddep_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void griddep_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ------------------------------------------------------------------- cluster
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ------------------------------------------------------------------- tcgen05
template <int CTAS>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    if constexpr (CTAS == 1)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
                     "r"(ncols)
                     : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
                     "r"(ncols)
                     : "memory");
}
template <int CTAS>
__device__ __forceinline__ void tmem_relinquish() {
    if constexpr (CTAS == 1)
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    else
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CTAS>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    if constexpr (CTAS == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                     : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                     : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] . B[smem desc], 8-bit integer operands, s32 accumulate.
template <int CTAS>
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
    if constexpr (CTAS == 1)
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
}

// Arrive once on `bar` (this CTA) when every MMA this thread issued so far is done.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
// Pair form: arrive on the barrier at this offset in every CTA named by `cta_mask`.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
        "[%0], %1;" ::"r"(bar),
        "h"(cta_mask)
        : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns: thread t of the warp gets lane
// (base lane + t), registers v[0..15] = columns col..col+15.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
          "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile whose rows are
// 128 bytes long and stored with the 128-byte swizzle (what a TMA box of
// {128 bytes, rows} with SWIZZLE_128B writes): groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);        // start address
    d |= static_cast<uint64_t>(1) << 16;                             // leading offset: unused here
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                     // 8-row group stride
    d |= static_cast<uint64_t>(1) << 46;                             // descriptor version (sm_100)
    d |= static_cast<uint64_t>(2) << 61;                             // layout: 128-byte swizzle
    return d;
}

// Shared-memory matrix descriptor for an MN-major operand tile (N contiguous): rows of
// K, each 128 bytes of N, stored with the 128-byte swizzle (a TMA box of {128 bytes of N,
// rows of K}).  Groups of 8 K-rows are 1024 bytes apart; the next 128 columns of N start
// `n_atom_stride` bytes further on.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t smem_addr, uint32_t n_atom_stride) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((n_atom_stride >> 4) & 0x3FFFu) << 16;  // leading offset: next N atom
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                       // stride offset: next 8 K-rows
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// The same for a tile of 64 bytes of N per K-row, stored with the 64-byte swizzle (a TMA box
// of {64 bytes of N, rows of K} with SWIZZLE_64B): groups of 8 K-rows are 512 bytes apart.
// The tile is a single atom in N, so the leading offset is not used.
__device__ __forceinline__ uint64_t smem_desc_mn_sw64(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;                               // leading offset: unused here
    d |= static_cast<uint64_t>(512 >> 4) << 32;                        // stride offset: next 8 K-rows
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(4) << 61;                               // layout: 64-byte swizzle
    return d;
}

// Instruction descriptor of tcgen05.mma kind::i8: s32 accumulator, A K-major, B K-major
// or (b_mn) MN-major, no saturation.  a_signed / b_signed pick s8 or u8.
__host__ __device__ constexpr uint32_t idesc_i8(int m, int n, bool a_signed, bool b_signed,
                                                bool b_mn = false) {
    return (2u << 4)                          // accumulator format: S32
           | ((a_signed ? 1u : 0u) << 7)      // A: 1 = signed 8-bit, 0 = unsigned
           | ((b_signed ? 1u : 0u) << 10)     // B
           | ((b_mn ? 1u : 0u) << 16)         // B major: 0 = K, 1 = MN
           | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

}  // namespace ptx
}  // namespace mb200
