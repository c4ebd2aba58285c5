// Q16.16 GEMM in one kernel: the limb products on the tensor cores and the per-product floor on
// the FP32 pipe, at the same time, on the same SM, for the same output tile.
//
//   C[i,j] = (i32) sum_k ((i64)A[i,k] * (i64)B[k,j]) >> 16
//          = sum_k a * bh + ah * bl  (mod 2^32: eleven 8-bit limb products, tcgen05 kind::i8)
//          + sum_k floor(al * bl / 65536)   (one fma.rm.f32 per product, see gemm_q16_f32.cu)
//
// The two-kernel hybrid runs those halves one after the other (or on disjoint SMs): the tensor
// pipe idles while the FP32 pipe works and the other way round.  The floor term needs 128 x 128 x
// 128 FMAs per 128 of K on a tile, about 19 000 cycles of the FP32 pipe; the limb products of the
// same block are 44 MMAs, under 3 000 cycles of the tensor pipe.  Here a CTA does both for its
// tile: the tensor-core work hides entirely behind the FMAs, and C is written once.
//
// Roles (384 threads, three warpgroups; registers move from the third to the first two):
//   warps 0..7  compute: the 8 x 8 register tile of gemm_q16_f32.cu per thread, operands from
//               shared-memory stages filled by TMA from pre-converted binary32 planes
//               (al transposed to [K][M], bl * 2^-16 as [K][N]); at the end of a run they drain
//               the four TMEM accumulators into a shared tile, add their own sums in place, and
//               the tile leaves as sixteen tensor stores (or tensor reductions, see below).
//   warp 8      lane 0 feeds the FP32 stages (TMA; two stages of 32 of K: fewer, longer stages
//               beat three of 16 by 4 % - a stage boundary is a vote, an arrive, a wait and a
//               first shared-memory load that nothing hides).
//   warp 9      lane 0 feeds and drives the tensor cores: one shared-memory stage of six byte
//               planes (a0..a3, two of b); per 128 of K a first pass with the planes of b >> 16
//               (seven MMAs per 32 of K) and a second with those of b & 0xffff (four, on a2 / a3).
//               One stage is enough: the tensor pipe has six times the time it needs.
//   warps 10, 11  idle (a warpgroup is four warps).
//
// Work is dealt out stream-K fashion in units of 32 of K of one tile, block b takes units
// [b U / G, (b + 1) U / G); a run that covers its tile's whole K stores its tile, the others add
// theirs onto a zeroed C with cp.reduce.async.bulk.tensor (.add, performed in L2; sums mod 2^32
// commute).  Per-element red.global.add from the register tiles cost 9 of the kernel's 65 us at
// 1024^3 (two runs per CTA, 16 384 scattered 4-byte reductions each).  A C that a tensor map
// cannot address (N % 4 != 0 or a base off 16 bytes) is written by the warps from the same tile.
//
// Every wait is an mbarrier wait bounded in time; when one runs out the CTA's roles leave their
// loops, the error word is set and the kernel ends normally.
#include <type_traits>

#include "common.h"
#include "ptx.cuh"

namespace mb200 {
using namespace ptx;

namespace {

constexpr int UT = 128;                      // output tile (rows and columns)
constexpr int UNIT_K = 32;                   // stream-K granule = one MMA's K
constexpr int TCB_K = 128;                   // K per tensor-core stage
constexpr int FSTEP = 32;                    // K per FP32 stage
constexpr int FSTAGES = 2;
constexpr int FLUSH_FSTEPS = 128 / FSTEP;    // a chain holds 128 products
constexpr int PLANE_BYTES = UT * TCB_K;      // one byte plane of a stage
constexpr int TC_STAGE_BYTES = 6 * PLANE_BYTES;
constexpr int F_HALF_BYTES = FSTEP * UT * 4;  // A or B part of an FP32 stage
constexpr int F_STAGE_BYTES = 2 * F_HALF_BYTES;
constexpr int T_BOX = 32;                    // the output tile is kept as 4 x 4 boxes of 32 x 32 words,
constexpr int T_BOX_BYTES = T_BOX * T_BOX * 4;  // each 32 rows of 128 bytes in the 128-byte swizzle (what a tensor store reads)
constexpr int T_BYTES = (UT / T_BOX) * (UT / T_BOX) * T_BOX_BYTES;
constexpr int FUSED_THREADS = 384;
constexpr int COMPUTE_WARPS = 8;
constexpr int FUSED_SMEM = 1024 + TC_STAGE_BYTES + FSTAGES * F_STAGE_BYTES + T_BYTES + 256;
static_assert(FUSED_SMEM <= 232448, "shared memory budget");

constexpr uint32_t TWO23_BITS = Q16_TWO23_BITS;
constexpr uint64_t CHAIN_START = ((uint64_t)TWO23_BITS << 32) | TWO23_BITS;

__device__ __forceinline__ uint64_t fma2_rm(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rm.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

struct FusedParams {
    int32_t* c;         // used only when the tile cannot leave through the tensor map (tma_c == 0)
    int tma_c;          // C is 16-byte aligned with N % 4 == 0: tensor stores / reductions
    int m, n;           // extents of C (the tensor maps carry the rest)
    int n_tiles;
    int k_units;        // ceil(k / 32)
    long long units;    // tiles * k_units
    int* err;
    uint32_t one;       // 1; a value the compiler cannot know (see wait_bounded_dep)
};

// The run of units [u, u_end) that lies in one tile: tile index and unit range inside it.
struct Run {
    int tile, ku0, ku1;
};
__device__ __forceinline__ Run next_run(long long& u, long long u_end, int k_units) {
    Run r;
    r.tile = (int)(u / k_units);
    r.ku0 = (int)(u % k_units);
    const long long left = u_end - u;
    r.ku1 = left < (long long)(k_units - r.ku0) ? r.ku0 + (int)left : k_units;
    u += r.ku1 - r.ku0;
    return r;
}

// EDGE: the product has tiles whose second half (rows or columns 64..127) is all padding, and many
// of them (a narrow N or M): those tiles skip the padding's loads and FMAs.  A build of its own,
// because the extra paths cost the whole-tile loop 4 % through a different instruction schedule.
template <bool EDGE>
__global__ void __launch_bounds__(FUSED_THREADS, 1)
gemm_q16_fused_kernel(const __grid_constant__ CUtensorMap tm_a0, const __grid_constant__ CUtensorMap tm_a1,
                      const __grid_constant__ CUtensorMap tm_a2, const __grid_constant__ CUtensorMap tm_a3,
                      const __grid_constant__ CUtensorMap tm_bh0, const __grid_constant__ CUtensorMap tm_bh1,
                      const __grid_constant__ CUtensorMap tm_bl0, const __grid_constant__ CUtensorMap tm_bl1,
                      const __grid_constant__ CUtensorMap tm_af, const __grid_constant__ CUtensorMap tm_bf,
                      const __grid_constant__ CUtensorMap tm_c, const FusedParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tc0 = (raw + 1023u) & ~1023u;            // six byte planes, 1024-byte aligned (swizzled)
    const uint32_t f0 = tc0 + TC_STAGE_BYTES;               // FP32 stages: [A part | B part] each
    const uint32_t t0 = f0 + FSTAGES * F_STAGE_BYTES;       // the tile the accumulators are drained into
    const uint32_t bars = t0 + T_BYTES;
    const uint32_t tc_full = bars, tc_empty = bars + 8;
    const uint32_t f_full0 = bars + 16, f_empty0 = f_full0 + 8 * FSTAGES;
    const uint32_t tmem_full = f_empty0 + 8 * FSTAGES, tmem_empty = tmem_full + 8;
    const uint32_t t_ready = tmem_empty + 8, t_free = t_ready + 8, t_done = t_free + 8;
    const uint32_t tmem_slot = t_done + 8;
    int* const misc = reinterpret_cast<int*>(smem_raw + (tmem_slot - raw));
    volatile int* const abort_s = misc + 1;
    const float* const f_tile = reinterpret_cast<const float*>(smem_raw + (f0 - raw));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(tc_full, 1);
        mbar_init(tc_empty, 1);
        for (int s = 0; s < FSTAGES; ++s) {
            mbar_init(f_full0 + 8 * s, 1);
            mbar_init(f_empty0 + 8 * s, COMPUTE_WARPS);
        }
        mbar_init(tmem_full, 1);
        mbar_init(tmem_empty, COMPUTE_WARPS);
        mbar_init(t_ready, COMPUTE_WARPS);
        mbar_init(t_free, COMPUTE_WARPS);
        mbar_init(t_done, COMPUTE_WARPS);
        misc[1] = 0;
        fence_mbar_init();
        prefetch_tensormap(&tm_a0); prefetch_tensormap(&tm_a1); prefetch_tensormap(&tm_a2); prefetch_tensormap(&tm_a3);
        prefetch_tensormap(&tm_bh0); prefetch_tensormap(&tm_bh1); prefetch_tensormap(&tm_bl0); prefetch_tensormap(&tm_bl1);
        prefetch_tensormap(&tm_af); prefetch_tensormap(&tm_bf); prefetch_tensormap(&tm_c);
    }
    if (warp == 9) {
        tmem_alloc<1>(tmem_slot, 512);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(misc);
    // from here on global memory is read and written: the kernel before this one (the operand
    // split, which also zeroes C where tiles are shared) must be done
    griddep_wait();

    // 384 threads start with 168 registers each; the third warpgroup keeps 56 and the two
    // compute warpgroups take 224 (256 * 224 + 128 * 56 = 384 * 168: the launcher checks that the
    // kernel was built with exactly 168, or the request could never be met).  Each role's code
    // follows its own request directly, which is what lets the compiler allocate to the new limit.
    const long long u_end = p.units * (blockIdx.x + 1) / gridDim.x;
    long long u = p.units * blockIdx.x / gridDim.x;

    if (warp >= 8) {
        regs_release<56>();
    if (warp == 8) {
        // ------------------------------------------------ FP32 stages: TMA producer
        if (lane == 0) {
            const uint64_t pol = l2_policy(0);
            uint32_t it = 0;
            bool ok = true;
            while (ok && u < u_end) {
                const Run r = next_run(u, u_end, p.k_units);
                const int row0 = (r.tile / p.n_tiles) * UT, col0 = (r.tile % p.n_tiles) * UT;
                const int fsteps = (r.ku1 - r.ku0) * (UNIT_K / FSTEP);
                for (int fs = 0; fs < fsteps; ++fs, ++it) {
                    const uint32_t s = it % FSTAGES, ph = (it / FSTAGES) & 1u;
                    if (!wait_bounded(f_empty0 + 8 * s, ph ^ 1u, abort_s, p.err, 11)) {
                        ok = false;
                        break;
                    }
                    const uint32_t bar = f_full0 + 8 * s, dst = f0 + s * F_STAGE_BYTES;
                    const int k0 = r.ku0 * UNIT_K + fs * FSTEP;
                    mbar_arrive_expect_tx(bar, F_STAGE_BYTES);
                    tma_load_2d(dst, &tm_af, bar, row0, k0, pol);
                    tma_load_2d(dst + F_HALF_BYTES, &tm_bf, bar, col0, k0, pol);
                }
            }
        }
    } else if (warp == 9) {
        // ------------------------------------------------ tensor cores: TMA producer and MMA issuer in one thread
        if (lane == 0) {
            constexpr uint32_t ID_SU = idesc_i8(UT, UT, true, false, true);
            constexpr uint32_t ID_US = idesc_i8(UT, UT, false, true, true);
            constexpr uint32_t ID_UU = idesc_i8(UT, UT, false, false, true);
            constexpr uint64_t B_KSTEP = (UNIT_K * UT) >> 4;  // 32 K-rows of 128 bytes, in units of 16 bytes
            const uint64_t pol_a = l2_policy(1), pol_b = l2_policy(0);
            const uint32_t sa = tc0, sb = tc0 + 4 * PLANE_BYTES;
            uint32_t it = 0, rc = 0;
            bool ok = true;
            while (ok && u < u_end) {
                const Run r = next_run(u, u_end, p.k_units);
                const int row0 = (r.tile / p.n_tiles) * UT, col0 = (r.tile % p.n_tiles) * UT;
                if (!wait_bounded(tmem_empty, (rc & 1u) ^ 1u, abort_s, p.err, 12)) break;
                tc_fence_after();
                for (int ku = r.ku0; ok && ku < r.ku1; ku += TCB_K / UNIT_K) {
                    const int kx = ku * UNIT_K;
                    const int steps = min(TCB_K / UNIT_K, r.ku1 - ku);
                    for (int pass = 0; pass < 2; ++pass, ++it) {
                        if (!wait_bounded(tc_empty, (it & 1u) ^ 1u, abort_s, p.err, 13)) {
                            ok = false;
                            break;
                        }
                        if (pass == 0) {
                            mbar_arrive_expect_tx(tc_full, 6 * PLANE_BYTES);
                            tma_load_2d(sa, &tm_a0, tc_full, kx, row0, pol_a);
                            tma_load_2d(sa + PLANE_BYTES, &tm_a1, tc_full, kx, row0, pol_a);
                            tma_load_2d(sa + 2 * PLANE_BYTES, &tm_a2, tc_full, kx, row0, pol_a);
                            tma_load_2d(sa + 3 * PLANE_BYTES, &tm_a3, tc_full, kx, row0, pol_a);
                            tma_load_2d(sb, &tm_bh0, tc_full, col0, kx, pol_b);
                            tma_load_2d(sb + PLANE_BYTES, &tm_bh1, tc_full, col0, kx, pol_b);
                        } else {
                            mbar_arrive_expect_tx(tc_full, 2 * PLANE_BYTES);
                            tma_load_2d(sb, &tm_bl0, tc_full, col0, kx, pol_b);
                            tma_load_2d(sb + PLANE_BYTES, &tm_bl1, tc_full, col0, kx, pol_b);
                        }
                        if (!wait_bounded(tc_full, it & 1u, abort_s, p.err, 14)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        for (int ks = 0; ks < steps; ++ks) {
                            const uint64_t koff = (uint64_t)((ks * UNIT_K) >> 4), kb_off = (uint64_t)ks * B_KSTEP;
                            const uint64_t a0d = smem_desc_k_sw128(sa) + koff;
                            const uint64_t a1d = smem_desc_k_sw128(sa + PLANE_BYTES) + koff;
                            const uint64_t a2d = smem_desc_k_sw128(sa + 2 * PLANE_BYTES) + koff;
                            const uint64_t a3d = smem_desc_k_sw128(sa + 3 * PLANE_BYTES) + koff;
                            const uint64_t b0d = smem_desc_mn_sw128(sb, PLANE_BYTES) + kb_off;
                            const uint64_t b1d = smem_desc_mn_sw128(sb + PLANE_BYTES, PLANE_BYTES) + kb_off;
                            const uint32_t d0 = tmem_base;
                            if (pass == 0) {
                                // a = a3*2^24 + a2*2^16 + a1*2^8 + a0 (a3 signed), bh = bh1*256 + bh0 (bh1
                                // signed); accumulator s collects the limb products of weight 2^(8s)
                                const uint32_t acc = (ku != r.ku0 || ks != 0) ? 1u : 0u;
                                mma_i8<1>(d0, a0d, b0d, ID_UU, acc);            // a0.bh0 -> s0
                                mma_i8<1>(d0 + UT, a0d, b1d, ID_US, acc);       // a0.bh1 -> s1
                                mma_i8<1>(d0 + UT, a1d, b0d, ID_UU, 1u);        // a1.bh0 -> s1
                                mma_i8<1>(d0 + 2 * UT, a1d, b1d, ID_US, acc);   // a1.bh1 -> s2
                                mma_i8<1>(d0 + 2 * UT, a2d, b0d, ID_UU, 1u);    // a2.bh0 -> s2
                                mma_i8<1>(d0 + 3 * UT, a2d, b1d, ID_US, acc);   // a2.bh1 -> s3
                                mma_i8<1>(d0 + 3 * UT, a3d, b0d, ID_SU, 1u);    // a3.bh0 -> s3
                            } else {
                                // ah * bl, ah = a3*256 + a2, bl = bl1*256 + bl0 (both unsigned)
                                mma_i8<1>(d0, a2d, b0d, ID_UU, 1u);             // a2.bl0 -> s0
                                mma_i8<1>(d0 + UT, a3d, b0d, ID_SU, 1u);        // a3.bl0 -> s1
                                mma_i8<1>(d0 + UT, a2d, b1d, ID_UU, 1u);        // a2.bl1 -> s1
                                mma_i8<1>(d0 + 2 * UT, a3d, b1d, ID_SU, 1u);    // a3.bl1 -> s2
                            }
                        }
                        mma_commit(tc_empty);
                    }
                }
                if (!ok) break;
                mma_commit(tmem_full);
                ++rc;
            }
        }
    }
    } else {
        regs_take<224>();
        // ------------------------------------------------ compute warps: the floor term, then the epilogue
        // 16 x 16 threads; a warp is 8 (x) by 4 (y) of them with every four consecutive lanes 2 x 2
        // (the lane order under which a 16-byte shared load takes two wavefronts, not four)
        const int lx = (lane & 1) | ((lane >> 1) & 6), ly = ((lane >> 1) & 1) | ((lane >> 3) & 2);
        const int tx = (warp & 1) * 8 + lx, ty = (warp >> 1) * 4 + ly;
        const int q = warp & 3, half = warp >> 2;  // TMEM lane quadrant and column half this warp drains
        uint32_t it = 0, rc = 0;
        bool ok = true;
        while (ok && u < u_end) {
            const Run r = next_run(u, u_end, p.k_units);
            const int row0 = (r.tile / p.n_tiles) * UT, col0 = (r.tile % p.n_tiles) * UT;

            uint64_t chain[8][4];  // chain[i][jp]: outputs (row i, columns 2 jp and 2 jp + 1) of the register tile
            uint32_t sum[8][8];    // what the chains have been emptied into (plus 2^23's bits per emptying)
#pragma unroll
            for (int i = 0; i < 8; ++i) {
#pragma unroll
                for (int jp = 0; jp < 4; ++jp) chain[i][jp] = CHAIN_START;
#pragma unroll
                for (int j = 0; j < 8; ++j) sum[i][j] = 0u;
            }
            uint32_t emptied = 0;
            auto empty_chains = [&]() {
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int jp = 0; jp < 4; ++jp) {
                        sum[i][2 * jp] += (uint32_t)chain[i][jp];
                        sum[i][2 * jp + 1] += (uint32_t)(chain[i][jp] >> 32);
                        chain[i][jp] = CHAIN_START;
                    }
                ++emptied;
            };

            const int fsteps = (r.ku1 - r.ku0) * (UNIT_K / FSTEP);
            const bool half_m = EDGE && row0 + 64 >= p.m, half_n = EDGE && col0 + 64 >= p.n;  // the second half is all padding
            int since = 0;
            for (int fs = 0; fs < fsteps; ++fs, ++it) {
                const uint32_t s = it % FSTAGES, ph = (it / FSTAGES) & 1u;
                const uint32_t landed = wait_bounded_dep(f_full0 + 8 * s, ph, abort_s, p.err, 15, p.one);
                if (!landed) {
                    ok = false;
                    break;
                }
                // (landed - one = 0: the stage's address depends on the outcome of the wait)
                const float* const fa_s = f_tile + s * (F_STAGE_BYTES / 4) + (landed - p.one);
                const float* const fb_s = fa_s + F_HALF_BYTES / 4;
                // One stage of FSTEP K steps.  Fragments of step kk + 1 are fetched while those of step kk
                // are multiplied.  MG / NG: how many of the register tile's two row / column groups
                // (rows +0..63 / +64..127 of the tile, likewise columns) lie inside C: a tile on the
                // edge of a narrow product (64 batched queries against a catalogue: N = 64) skips the
                // loads and the FMAs of the half that is padding.
                auto stage_fmas = [&](auto mg_tag, auto ng_tag) {
                    constexpr int MG = decltype(mg_tag)::value, NG = decltype(ng_tag)::value;
                    uint4 fa[2][2], fb[2][2];
                    auto fetch = [&](int kk, int slot) {
#pragma unroll
                        for (int g = 0; g < 2; ++g) {
                            if (g < MG) fa[slot][g] = *reinterpret_cast<const uint4*>(fa_s + kk * UT + g * 64 + ty * 4);
                            if (g < NG) fb[slot][g] = *reinterpret_cast<const uint4*>(fb_s + kk * UT + g * 64 + tx * 4);
                        }
                    };
                    fetch(0, 0);
#pragma unroll
                    for (int kk = 0; kk < FSTEP; ++kk) {
                        if (kk + 1 < FSTEP) fetch(kk + 1, (kk + 1) & 1);
                        uint64_t a2[8], b2[4];
#pragma unroll
                        for (int g = 0; g < 2; ++g) {
                            if (g < MG) {
                                const uint4 v = fa[kk & 1][g];
                                a2[4 * g] = ((uint64_t)v.x << 32) | v.x; a2[4 * g + 1] = ((uint64_t)v.y << 32) | v.y;
                                a2[4 * g + 2] = ((uint64_t)v.z << 32) | v.z; a2[4 * g + 3] = ((uint64_t)v.w << 32) | v.w;
                            }
                            if (g < NG) {
                                const uint4 w = fb[kk & 1][g];
                                b2[2 * g] = ((uint64_t)w.y << 32) | w.x; b2[2 * g + 1] = ((uint64_t)w.w << 32) | w.z;
                            }
                        }
                        // B pair outermost (in the order 0, 2, 1, 3: consecutive pairs come from different
                        // loads), rows walked forwards and backwards in turn, so that every FMA shares an
                        // operand register with the one before it.  Kernel at 4096^3: 2.51 ms; rows outermost
                        // 2.58 ms, pairs in order 2.52 ms, without the serpentine 2.55 ms.
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj)
#pragma unroll
                            for (int ii = 0; ii < 8; ++ii) {
                                const int jp = ((jj & 1) << 1) | (jj >> 1);
                                const int i = (jj & 1) ? 7 - ii : ii;
                                if (jp < 2 * NG && i < 4 * MG) chain[i][jp] = fma2_rm(a2[i], b2[jp], chain[i][jp]);
                            }
                    }
                };
                using one_t = std::integral_constant<int, 1>;
                using two_t = std::integral_constant<int, 2>;
                if (!EDGE || (!half_m && !half_n)) {
                    // (the whole tile, written out on its own)
                    uint4 fa[2][2], fb[2][2];
                    auto fetch = [&](int kk, int slot) {
#pragma unroll
                        for (int g = 0; g < 2; ++g) {
                            fa[slot][g] = *reinterpret_cast<const uint4*>(fa_s + kk * UT + g * 64 + ty * 4);
                            fb[slot][g] = *reinterpret_cast<const uint4*>(fb_s + kk * UT + g * 64 + tx * 4);
                        }
                    };
                    fetch(0, 0);
#pragma unroll
                    for (int kk = 0; kk < FSTEP; ++kk) {
                        if (kk + 1 < FSTEP) fetch(kk + 1, (kk + 1) & 1);
                        uint64_t a2[8], b2[4];
#pragma unroll
                        for (int g = 0; g < 2; ++g) {
                            const uint4 v = fa[kk & 1][g], w = fb[kk & 1][g];
                            a2[4 * g] = ((uint64_t)v.x << 32) | v.x; a2[4 * g + 1] = ((uint64_t)v.y << 32) | v.y;
                            a2[4 * g + 2] = ((uint64_t)v.z << 32) | v.z; a2[4 * g + 3] = ((uint64_t)v.w << 32) | v.w;
                            b2[2 * g] = ((uint64_t)w.y << 32) | w.x; b2[2 * g + 1] = ((uint64_t)w.w << 32) | w.z;
                        }
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj)
#pragma unroll
                            for (int ii = 0; ii < 8; ++ii) {
                                const int jp = ((jj & 1) << 1) | (jj >> 1);
                                const int i = (jj & 1) ? 7 - ii : ii;
                                chain[i][jp] = fma2_rm(a2[i], b2[jp], chain[i][jp]);
                            }
                    }
                } else if (!half_m) {
                    stage_fmas(two_t{}, one_t{});
                } else if (!half_n) {
                    stage_fmas(one_t{}, two_t{});
                } else {
                    stage_fmas(one_t{}, one_t{});
                }
                // Release the stage only once every lane's last fragments have been USED.  With a plain
                // __syncwarp() before lane 0's arrive, the last A fragment of a stage (its last K step)
                // was now and then read AFTER the producer had refilled the stage (with three stages of 16
                // it came back as the element 48 further on in K: what the next fill puts there), always
                // in the warp that shares a scheduler with a producer warp, i.e. the one whose arrival is
                // last and triggers the refill: one tile in thirty at 2048^3.  The vote below reads one
                // chain per operand register of the last K step, and the arrive is predicated on its
                // result, so neither a load of this stage nor an FMA waiting for one can follow the
                // release in any instruction order.
                uint64_t used = chain[0][1] ^ chain[0][2] ^ chain[0][3];
#pragma unroll
                for (int i = 0; i < 8; ++i) used ^= chain[i][0];
                const uint32_t all_used = __ballot_sync(0xffffffffu, used != 0x7ff8dead7ff8deadull);
                if (lane == 0 && all_used != 0u) mbar_arrive(f_empty0 + 8 * s);  // (always true: chains hold no NaN)
                if (++since == FLUSH_FSTEPS) {
                    empty_chains();
                    since = 0;
                }
            }
            if (!ok) break;
            empty_chains();

            // The accumulators of this run.  The output tile lives in shared memory as 4 x 4 boxes of
            // 32 x 32 words, each in the layout a tensor store reads (32 rows of 128 bytes, 16-byte
            // chunk j of row l at position j ^ (l & 7)).  (1) Lane 0 makes sure its tensor stores of
            // the previous run have read the tile, and all eight warps meet (t_free).  (2) After the
            // last MMA each warp drains its 32 rows x 64 columns of the four accumulators into the
            // tile as s0 + (s1 << 8) + (s2 << 16) + (s3 << 24) (lane = row) and frees TMEM for the
            // next run.  (3) When all have written, every thread adds its own 8 x 8 floor sums in
            // place.  (4) When all have done that, lane 0 of warp w sends boxes 2 w and 2 w + 1: a
            // tensor store if this run covers the tile's whole K, a tensor reduction (add) otherwise.
            if (lane == 0) {
                bulk_wait_group_read<0>();
                mbar_arrive(t_free);
            }
            if (!wait_bounded(tmem_full, rc & 1u, abort_s, p.err, 16)) break;
            tc_fence_after();
            if (!wait_bounded(t_free, rc & 1u, abort_s, p.err, 17)) break;
            {
                const uint32_t tsrc = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(half * 64);
#pragma unroll
                for (int c0 = 0; c0 < 64; c0 += 16) {
                    uint32_t s0[16], s1[16], s2[16], s3[16];
                    tmem_ld16(tsrc + c0, s0);
                    tmem_ld16(tsrc + UT + c0, s1);
                    tmem_ld16(tsrc + 2 * UT + c0, s2);
                    tmem_ld16(tsrc + 3 * UT + c0, s3);
                    tmem_ld_wait();
                    // box (q, 2 half + c0 / 32), chunks (c0 % 32) / 4 .. + 3 of row `lane`
                    const uint32_t brow = t0 + (uint32_t)((q * 4 + 2 * half + c0 / 32) * T_BOX_BYTES + lane * 128);
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        uint32_t v[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            v[e] = s0[j + e] + (s1[j + e] << 8) + (s2[j + e] << 16) + (s3[j + e] << 24);
                        st_shared_v4(brow + (uint32_t)((((c0 % 32) + j) / 4) ^ (lane & 7)) * 16u, v[0], v[1], v[2], v[3]);
                    }
                }
            }
            tc_fence_before();
            __threadfence_block();  // this warp's part of the tile is written before the arrive below, in any order of issue
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(tmem_empty);
                mbar_arrive(t_ready);
            }
            const uint32_t written = wait_bounded_dep(t_ready, rc & 1u, abort_s, p.err, 18, p.one);
            if (!written) break;
            const uint32_t t_rd = t0 + (written - p.one);  // the accesses below depend on the wait

            const uint32_t bias = emptied * TWO23_BITS;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int rl = (i / 4) * 64 + ty * 4 + (i % 4);
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const int cl = g * 64 + tx * 4;
                    const uint32_t at = t_rd + (uint32_t)(((rl / T_BOX) * 4 + cl / T_BOX) * T_BOX_BYTES + (rl % T_BOX) * 128 +
                                                          ((((cl % T_BOX) / 4) ^ (rl & 7)) << 4));
                    const uint4 lin = ld_shared_v4(at);
                    st_shared_v4(at, sum[i][4 * g] - bias + lin.x, sum[i][4 * g + 1] - bias + lin.y,
                                 sum[i][4 * g + 2] - bias + lin.z, sum[i][4 * g + 3] - bias + lin.w);
                }
            }
            fence_proxy_async_smem();  // these writes are read by the tensor stores below (another proxy)
            __threadfence_block();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(t_done);
                if (!wait_bounded(t_done, rc & 1u, abort_s, p.err, 19)) {
                    ok = false;
                } else if (p.tma_c) {
                    const bool owns = r.ku0 == 0 && r.ku1 == p.k_units;
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int box = 2 * warp + e, y = row0 + (box / 4) * T_BOX, x = col0 + (box % 4) * T_BOX;
                        if (y >= p.m || x >= p.n) continue;  // (a box partly outside is clipped by the hardware)
                        if (owns)
                            tma_store_2d(&tm_c, t0 + (uint32_t)box * T_BOX_BYTES, x, y);
                        else
                            tma_reduce_add_2d(&tm_c, t0 + (uint32_t)box * T_BOX_BYTES, x, y);
                    }
                    bulk_commit_group();
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            if (!p.tma_c) {
                // C with an odd pitch or base: the warp writes its two boxes itself, lane = column
                // (a row of a box is 128 contiguous bytes of C), stores or red.global.add
                const bool owns = r.ku0 == 0 && r.ku1 == p.k_units;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int box = 2 * warp + e, y = row0 + (box / 4) * T_BOX, x = col0 + (box % 4) * T_BOX + lane;
                    if (y >= p.m || x >= p.n) continue;
                    const uint32_t src = t0 + (uint32_t)box * T_BOX_BYTES + (uint32_t)(lane & 3) * 4u;
                    unsigned int* dst = reinterpret_cast<unsigned int*>(p.c) + (size_t)y * p.n + x;
                    for (int rr = 0; rr < T_BOX && y + rr < p.m; ++rr, dst += p.n) {
                        uint32_t v;
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(src + (uint32_t)(rr * 128 + (((lane >> 2) ^ (rr & 7)) << 4))) : "memory");
                        if (owns)
                            *dst = v;
                        else
                            atomicAdd(dst, v);
                    }
                }
                __threadfence_block();  // the tile has been read before it is handed back (t_free, next run)
            }
            ++rc;
        }
    }

    // ------------------------------------------------------------------ teardown
    if (warp < COMPUTE_WARPS && lane == 0) bulk_wait_group<0>();  // this warp's tensor stores have landed
    __syncwarp();
    if (*abort_s) __nanosleep(200000);  // let copies / MMAs still in flight land before freeing
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc<1>(tmem_base, 512);
    }
}

}  // namespace

// Map over a binary32 plane [k][inner] (row pitch in bytes): boxes of 128 along the inner
// dimension by 16 rows of K, no swizzle.  Reads past either extent return zeros.
static int64_t make_tmap_f32(CUtensorMap* tm, const float* base, int64_t inner, int64_t k, int64_t pitch_bytes) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(MIND_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)k};
    cuuint64_t strides[1] = {(cuuint64_t)pitch_bytes};
    cuuint32_t box[2] = {(cuuint32_t)UT, (cuuint32_t)FSTEP};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(MIND_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed for a binary32 plane with CUresult %d (inner=%lld k=%lld)",
                    (int)r, (long long)inner, (long long)k);
    return 0;
}

// The kernel moves registers between its warpgroups on the assumption that it was built with 168
// per thread (see the kernel); with any other count it must not run.
bool gemm_q16_fused_usable(DeviceCtx* ctx) {
    static thread_local int asked_dev = -1;
    static thread_local bool usable = false;
    if (asked_dev != ctx->device) {
        cudaFuncAttributes fa;
        usable = true;
        for (int edge = 0; edge < 2 && usable; ++edge) {
            const void* kern = edge ? (const void*)gemm_q16_fused_kernel<true> : (const void*)gemm_q16_fused_kernel<false>;
            usable = cudaFuncGetAttributes(&fa, kern) == cudaSuccess && fa.numRegs == 168 &&
                     cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FUSED_SMEM) == cudaSuccess;
        }
        cudaGetLastError();
        asked_dev = ctx->device;
    }
    return usable;
}

// A tile shared by several blocks is added to with red.global.add: C must start from zero then
// (the operand split does that).  Same partition rule as the kernel's.
bool gemm_q16_fused_shares_tiles(DeviceCtx* ctx, int64_t m, int64_t n, int64_t k) {
    const int64_t tiles = ((m + UT - 1) / UT) * ((n + UT - 1) / UT), k_units = (k + UNIT_K - 1) / UNIT_K;
    const int64_t units = tiles * k_units, grid = units < ctx->sm_count ? units : ctx->sm_count;
    for (int64_t b = 1; b < grid; ++b)
        if ((units * b / grid) % k_units != 0) return true;
    return false;
}

// c = the whole Q16.16 product.  a_limb[0..3]: byte planes of a ([m][kp_a], a_limb[3] signed);
// b_limb[0..1]: bytes of b >> 16, b_limb[2..3]: bytes of b & 0xffff ([k][pitch_b]); a_low_t:
// (a & 0xffff) as binary32, transposed, [k][mp]; b_low: (b & 0xffff) * 2^-16 as binary32, [k][np].
// Any m, n, k and any 4-byte aligned c (the planes carry their own padded pitches).
int64_t launch_gemm_q16_fused(DeviceCtx* ctx, const uint8_t* const a_limb[4], const uint8_t* const b_limb[4],
                              const float* a_low_t, const float* b_low, int32_t* c, int64_t m, int64_t n, int64_t k,
                              int64_t kp_a, int64_t pitch_b, int64_t mp, int64_t np) {
    if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff)
        return fail(MIND_B200_ERR_TOO_LARGE, "GEMM dimension above 2^31-1");
    CUtensorMap ta[4], tb[4], taf, tbf;
    for (int i = 0; i < 4; ++i) MB200_TRY(make_tmap_u8(&ta[i], a_limb[i], k, m, kp_a, UT, 128));
    for (int i = 0; i < 4; ++i) MB200_TRY(make_tmap_u8(&tb[i], b_limb[i], n, k, pitch_b, TCB_K, 128));
    MB200_TRY(make_tmap_f32(&taf, a_low_t, m, k, mp * 4));
    MB200_TRY(make_tmap_f32(&tbf, b_low, n, k, np * 4));
    // C through a tensor map where the hardware can address it (16-byte base and pitch)
    const bool tma_c = n % 4 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0;
    CUtensorMap tc = taf;
    if (tma_c) MB200_TRY(make_tmap_c32(&tc, c, n, m));
    const int64_t m_tiles = (m + UT - 1) / UT, n_tiles = (n + UT - 1) / UT;
    if (m_tiles * n_tiles > 0x7fffffff) return fail(MIND_B200_ERR_TOO_LARGE, "too many output tiles");
    FusedParams p;
    p.c = c;
    p.tma_c = tma_c ? 1 : 0;
    p.m = (int)m;
    p.n = (int)n;
    p.n_tiles = (int)n_tiles;
    p.k_units = (int)((k + UNIT_K - 1) / UNIT_K);
    p.units = m_tiles * n_tiles * p.k_units;
    p.err = ctx->err_word;
    p.one = 1u;
    const unsigned grid = (unsigned)(p.units < ctx->sm_count ? p.units : ctx->sm_count);
    // Launched so that it may start while the kernel before it (the operand split) still runs: its
    // set-up (barriers, TMEM, tensor-map prefetch, the register hand-over) touches no global memory,
    // and every role waits for that kernel before its first global access.
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(grid, 1, 1);
    lc.blockDim = dim3(FUSED_THREADS, 1, 1);
    lc.dynamicSmemBytes = FUSED_SMEM;
    lc.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at;
    lc.numAttrs = 1;
    prof_begin(ctx);
    // tiles whose second half is padding: worth the EDGE build when they are a quarter of all tiles or more
    const int64_t half_rows = (m - 1) % UT < 64 ? n_tiles : 0, half_cols = (n - 1) % UT < 64 ? m_tiles : 0;
    const bool edge = 4 * (half_rows + half_cols) >= m_tiles * n_tiles;
    if (edge)
        MB200_CUDA(cudaLaunchKernelEx(&lc, gemm_q16_fused_kernel<true>, ta[0], ta[1], ta[2], ta[3], tb[0], tb[1], tb[2],
                                      tb[3], taf, tbf, tc, p));
    else
        MB200_CUDA(cudaLaunchKernelEx(&lc, gemm_q16_fused_kernel<false>, ta[0], ta[1], ta[2], ta[3], tb[0], tb[1], tb[2],
                                      tb[3], taf, tbf, tc, p));
    prof_end(ctx);
    count_launch();
    return check_launch("gemm_q16_fused_kernel");
}

}  // namespace mb200
