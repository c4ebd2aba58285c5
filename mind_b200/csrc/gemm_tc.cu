// Tensor-core integer GEMM for sm_100a: C[M,N] (s32, wrap) = A[M,K] . Bt[N,K]^T.
//
// One persistent, warp-specialised kernel, written against tcgen05 directly:
//   warp 0     : TMA producer  - cp.async.bulk.tensor tiles (128-byte swizzle) into a
//                ring of shared-memory stages, completion on a "full" mbarrier;
//   warp 1     : MMA issuer    - one thread issues tcgen05.mma kind::i8 from shared-
//                memory descriptors into TMEM accumulators, tcgen05.commit frees the
//                stage ("empty" mbarrier) and finally publishes the accumulator;
//   warps 2..5 : epilogue      - tcgen05.ld the accumulator (each warp its 32 TMEM
//                lanes = 32 output rows), combine, transpose 32 x 32 blocks through a
//                shared-memory patch and store int32 rows to global, 128 bytes at a time.
//                The modes with four accumulators per tile (int16, Q16.16 linear part) fill
//                all of TMEM, so their epilogue cannot overlap the next main loop: they run
//                eight epilogue warps (warps 2..9, two per lane quadrant, half the columns
//                each) to halve that exposed time.
// Tiles are 128 rows of A by BLOCK_N rows of Bt by 128 bytes of K per stage.
// MODE 0 (int8):  one s8 x s8 product, BLOCK_N = 256, two accumulator stages so the
//                 epilogue of tile t overlaps the main loop of tile t + 1.
// MODE 1 (int16): operands arrive as 8-bit limb planes, a = 256*hi + lo with hi signed
//                 and lo unsigned, b = 256*hi + (lo' + 128) with both planes signed.
//                 B's planes lie side by side in the stage, so two MMAs of N = 256
//                 per 32 of K give [hi.hi | hi.lo'] and [lo.hi | lo.lo'] in two
//                 accumulators, and the epilogue forms
//                 (HH << 16) + ((HL' + LH) << 8) + LL' + 128 * rowsum(a) with 32-bit
//                 wrap, which equals the exact sum truncated to 32 bits.  Wrap inside
//                 an accumulator is harmless (the tensor core does not saturate:
//                 descriptor bit 3 is 0).  One CTA per tile.
// MODE 3 (int8, narrow tiles): the same product with BLOCK_N = 64 and four small accumulator
//                 stages, for shapes whose 128 x 256 tiles would leave most SMs idle (256^3 is
//                 two such tiles but eight narrow ones, each with a quarter of the epilogue).
//                 A B that is read in place arrives as TMA boxes of 64 bytes of N by 128 rows of
//                 K with the 64-byte swizzle, the canonical MN-major layout of a 64-wide operand.
// MODE 5 (int8, CTA pair, 256 x 512 tiles): two MMAs of N = 256 per 32 of K read the same A
//                 slab, so a pair moves 48 KB per 128 of K for twice the work of MODE 0's 32 KB:
//                 a quarter less L2 -> shared-memory traffic per product, and the same bytes in
//                 flight cover a third more latency.  The 512 columns fill TMEM, so the epilogue
//                 (eight warps) does not overlap the next main loop: for long K only.
// The PAIR = 2 variant (int8) runs one tile on a pair of CTAs (a 2-CTA cluster,
// tcgen05 cta_group::2): 256 rows of A (128 per CTA) by BLOCK_N rows of Bt, of which
// each CTA stages only its half, which halves the shared-memory traffic per MMA.
// Out-of-range rows / K tails are zero-filled by TMA; stores are predicated.
// Every wait is bounded in time: when it runs out the kernel records a code in
// the device error word, all roles leave their loops, and the kernel exits cleanly.
#include "common.h"
#include "ptx.cuh"

namespace mb200 {
using namespace ptx;

namespace {

constexpr int BLOCK_M = 128;            // rows of A per CTA
constexpr int BLOCK_K = 128;            // bytes (= 8-bit elements) of K per stage
constexpr int UMMA_K = 32;              // K of one tcgen05.mma kind::i8
constexpr int TC_THREADS = 192;  // TMA warp + MMA warp + four epilogue warps (see epi_warps)
constexpr int A_TILE_BYTES = BLOCK_M * BLOCK_K;
constexpr int EPI_PATCH_WORDS = 32 * 32;  // per epilogue warp: a 32 x 32 block of outputs (4 KiB, 1024-byte aligned)

template <int MODE, int PAIR>
struct Cfg;
template <>
struct Cfg<0, 1> {
    static constexpr int BLOCK_N = 256, NA = 1, NB = 1, NACC = 1, ACC_STAGES = 2, STAGES = 4, TMEM_COLS = 512, NSUB = 1, EPI_PATCHES = 2;
};
template <>
struct Cfg<1, 1> {  // int16: two accumulators of 2 x BLOCK_N columns (A high / A low times [B high | B low])
    static constexpr int BLOCK_N = 128, NA = 2, NB = 2, NACC = 4, ACC_STAGES = 1, STAGES = 3, TMEM_COLS = 512, NSUB = 1, EPI_PATCHES = 1;
};
template <>
struct Cfg<0, 2> {
    static constexpr int BLOCK_N = 256, NA = 1, NB = 1, NACC = 1, ACC_STAGES = 2, STAGES = 6, TMEM_COLS = 512, NSUB = 1, EPI_PATCHES = 2;
};

template <>
struct Cfg<2, 1> {  // linear part of the Q16.16 product: a (4 limbs) x bh (2 limbs), 4 accumulators
    static constexpr int BLOCK_N = 128, NA = 4, NB = 2, NACC = 4, ACC_STAGES = 1, STAGES = 2, TMEM_COLS = 512, NSUB = 1, EPI_PATCHES = 1;
};
template <>
struct Cfg<4, 1> {  // the same with 64-column tiles: twice the CTAs for mid-sized products, two accumulator stages
    static constexpr int BLOCK_N = 64, NA = 4, NB = 2, NACC = 4, ACC_STAGES = 2, STAGES = 2, TMEM_COLS = 512, NSUB = 1, EPI_PATCHES = 2;
};
template <>
struct Cfg<3, 1> {  // int8, narrow tiles
    static constexpr int BLOCK_N = 64, NA = 1, NB = 1, NACC = 1, ACC_STAGES = 4, STAGES = 3, TMEM_COLS = 256, NSUB = 1, EPI_PATCHES = 2;
};
template <>
struct Cfg<5, 2> {  // int8, 256 x 512 tiles on a CTA pair: two MMAs of N = 256 share every A slab
    static constexpr int BLOCK_N = 512, NA = 1, NB = 1, NACC = 1, ACC_STAGES = 1, STAGES = 3, TMEM_COLS = 512, NSUB = 2, EPI_PATCHES = 2;
};

// Epilogue warps of a mode: four, or eight where a tile has four accumulators to drain.
template <int MODE, int PAIR>
__host__ __device__ constexpr int epi_warps() {
    return (Cfg<MODE, PAIR>::NACC == 4 || Cfg<MODE, PAIR>::BLOCK_N == 512) ? 8 : 4;
}
template <int MODE, int PAIR>
__host__ __device__ constexpr int tc_threads() { return 64 + 32 * epi_warps<MODE, PAIR>(); }

struct TcParams {
    int32_t* c;
    int m, n, k;
    int m_tiles, n_tiles;  // tile grid; an m-tile is PAIR * 128 rows
    int group_m;           // m-tiles walked together before moving on in n (L2 reuse of A panels)
    int raster;            // 1: odd groups walk n backwards, so a group starts on the B panels the last one ended on
    int hint_a, hint_b;    // L2 eviction policy per operand (see l2_policy)
    const int32_t* row_sums;  // int16 mode: sum of every row of A
    int accumulate;           // add onto C with red.global.add (C shared with a kernel running beside this one)
    int k_splits;             // > 1: every tile's K range is cut into this many work items (accumulate is set, C zeroed)
    int q16_low;              // Q16.16 linear mode: a second pass over K adds (a >> 16) * (b & 0xffff)
    int tma_store;            // the epilogue hands its 32 x 32 blocks to TMA stores (C 16-byte aligned, N % 4 == 0, no accumulate)
    int* err;
};

__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int group_m, int raster,
                                            int& tm, int& tn) {
    const int per_group = group_m * n_tiles;
    const int g = tile / per_group;
    const int r = tile - g * per_group;
    const int gm0 = g * group_m;
    const int gsize = min(group_m, m_tiles - gm0);
    tm = gm0 + r % gsize;
    tn = r / gsize;
    if (raster == 1 && (g & 1)) tn = n_tiles - 1 - tn;
}

// BMN = false: B is given transposed (Bt[N][K], K contiguous).  BMN = true: B is used as the
// caller has it (B[K][N], N contiguous = "MN-major"); its tiles are TMA boxes of 128 bytes of N
// by 128 rows of K, and the MMA reads them through an MN-major descriptor - no transpose pass.
template <int MODE, int PAIR, bool BMN>
__global__ void __launch_bounds__(tc_threads<MODE, PAIR>(), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a0, const __grid_constant__ CUtensorMap tm_a1,
               const __grid_constant__ CUtensorMap tm_a2, const __grid_constant__ CUtensorMap tm_a3,
               const __grid_constant__ CUtensorMap tm_b0, const __grid_constant__ CUtensorMap tm_b1,
               const __grid_constant__ CUtensorMap tm_b2, const __grid_constant__ CUtensorMap tm_b3,
               const __grid_constant__ CUtensorMap tm_c, const TcParams p) {
    constexpr bool Q16LIN = MODE == 2 || MODE == 4;  // linear part of the Q16.16 product (wide / narrow tiles)
    static_assert(!Q16LIN || (PAIR == 1 && BMN), "the Q16.16 linear-part mode is single-CTA, B in place");
    static_assert(MODE != 1 || PAIR == 1, "the int16 mode is single-CTA");
    static_assert(MODE != 3 || PAIR == 1, "the narrow-tile mode is single-CTA");
    static_assert(MODE != 5 || PAIR == 2, "the 256 x 512 mode runs on a CTA pair");
    using cfg = Cfg<MODE, PAIR>;
    constexpr int BLOCK_N = cfg::BLOCK_N;
    constexpr int B_ROWS = BLOCK_N / PAIR;  // columns of the output (rows of Bt) this CTA stages
    constexpr int B_TILE_BYTES = B_ROWS * BLOCK_K;
    // An MN-major B tile is made of boxes of BOX_N columns x 128 rows of K: 128 columns with the
    // 128-byte swizzle, or the whole 64-column tile with the 64-byte swizzle.
    constexpr int BOX_N = B_ROWS < 128 ? B_ROWS : 128;
    static_assert(!BMN || B_ROWS % BOX_N == 0, "an MN-major B tile is made of whole boxes");
    static_assert(BOX_N == 128 || BOX_N == 64, "box width = swizzle width");
    constexpr int B_BOX_BYTES = BOX_N * BLOCK_K;  // one MN-major box
    // N sub-tiles of a stage (one MMA each per 32 of K, all reading the same A slab); a sub-tile
    // is UMMA_N columns of the output, of which this CTA stages SUB_ROWS.
    constexpr int NSUB = cfg::NSUB;
    constexpr int UMMA_N = BLOCK_N / NSUB;
    constexpr int SUB_ROWS = B_ROWS / NSUB;
    constexpr int SUB_TILE_BYTES = SUB_ROWS * BLOCK_K;
    static_assert(NSUB == 1 || (PAIR == 2 && SUB_ROWS == 128), "sub-tiles are single 128-column boxes of a CTA pair");
    constexpr int STAGE_BYTES = cfg::NA * A_TILE_BYTES + cfg::NB * B_TILE_BYTES;
    constexpr int STAGES = cfg::STAGES;
    constexpr int ACC_STAGES = cfg::ACC_STAGES;
    constexpr int ACC_COLS = cfg::NACC * BLOCK_N;  // TMEM columns per accumulator stage
    constexpr int TMEM_COLS = cfg::TMEM_COLS;
    static_assert(ACC_COLS * ACC_STAGES <= TMEM_COLS, "TMEM overflow");
    constexpr int UMMA_M = BLOCK_M * PAIR;
    constexpr int EPI_WARPS = epi_warps<MODE, PAIR>();
    constexpr int EPI_GROUPS = EPI_WARPS / 4;         // warps per TMEM lane quadrant
    constexpr int EPI_COLS = BLOCK_N / EPI_GROUPS;    // output columns each of them drains
    static_assert(EPI_COLS % 32 == 0, "an epilogue warp drains whole 32-column blocks");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles0 = (raw + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
    const uint32_t bars = tiles0 + STAGES * STAGE_BYTES;
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES;
    const uint32_t tfull0 = bars + 16 * STAGES, tempty0 = tfull0 + 8 * ACC_STAGES;
    const uint32_t tmem_slot = tempty0 + 8 * ACC_STAGES;
    int* const misc = reinterpret_cast<int*>(smem_raw + (tmem_slot - raw));
    const uint32_t patches0 = bars + 1024;  // one 32 x 32-word patch per epilogue warp, 1024-byte aligned
    volatile int* const abort_s = misc + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = PAIR == 2 ? cluster_ctarank() : 0u;
    const bool leader = cta == 0;

    // The narrow-tile kernel serves launch-bound shapes: it is launched so that the next kernel
    // in the stream may start while this one runs, and its own set-up (barriers, TMEM, tensor-map
    // prefetch: nothing that touches global memory) overlaps the tail of the kernel before it.
    if (MODE == 3) griddep_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);     // one arrive.expect_tx (by the leader, for both CTAs' bytes)
            mbar_init(empty0 + 8 * s, 1);    // one tcgen05.commit
        }
        for (int s = 0; s < ACC_STAGES; ++s) {
            mbar_init(tfull0 + 8 * s, 1);           // one tcgen05.commit
            mbar_init(tempty0 + 8 * s, EPI_WARPS * PAIR);   // one arrive per epilogue warp (of both CTAs)
        }
        misc[1] = 0;
        fence_mbar_init();
        prefetch_tensormap(&tm_a0);
        prefetch_tensormap(&tm_b0);
        if (cfg::NA >= 2) prefetch_tensormap(&tm_a1);
        if (cfg::NA == 4) {
            prefetch_tensormap(&tm_a2);
            prefetch_tensormap(&tm_a3);
        }
        if (cfg::NB == 2) prefetch_tensormap(&tm_b1);
        if (Q16LIN && p.q16_low) {
            prefetch_tensormap(&tm_b2);
            prefetch_tensormap(&tm_b3);
        }
    }
    if (warp == 1) {
        tmem_alloc<PAIR>(tmem_slot, TMEM_COLS);
        tmem_relinquish<PAIR>();
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR == 2) {
        cluster_arrive();
        cluster_wait();
    }
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(misc);
    // from here on global memory is read and written: the kernel before this one must be done
    // (int16: that kernel is the limb split, whose tail this kernel's set-up overlaps)
    if (MODE == 3 || MODE == 1) griddep_wait();

    // Work items: (tile, split) with the split index fastest; a split is a contiguous range of
    // k-blocks, never empty (the launcher sees to that).
    const int total_tiles = p.m_tiles * p.n_tiles * p.k_splits;
    const int k_blocks = (p.k + BLOCK_K - 1) / BLOCK_K;
    const int kb_per_split = (k_blocks + p.k_splits - 1) / p.k_splits;
    const int tile_step = gridDim.x / PAIR;
    const int tile_first = blockIdx.x / PAIR;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            const uint64_t pol_a = l2_policy(p.hint_a), pol_b = l2_policy(p.hint_b);
            for (int item = tile_first; ok && item < total_tiles; item += tile_step) {
                int tm, tn;
                tile_coords(item / p.k_splits, p.m_tiles, p.n_tiles, p.group_m, p.raster, tm, tn);
                const int row_a = (tm * PAIR + (int)cta) * BLOCK_M;
                const int row_b = tn * BLOCK_N + (int)cta * B_ROWS;
                const int kb0 = (item % p.k_splits) * kb_per_split;
                const int kb1 = min(k_blocks, kb0 + kb_per_split);
                // Q16.16 with the low-half term: a second pass over the same K range, in which a
                // stage holds only the two high planes of a and the two planes of b & 0xffff
                const int passes = (Q16LIN && p.q16_low) ? 2 : 1;
                for (int pass = 0; ok && pass < passes; ++pass)
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                    if (!wait_bounded(empty0 + 8 * s, ph ^ 1u, abort_s, p.err, 1)) {
                        ok = false;
                        break;
                    }
                    const uint32_t dst = tiles0 + s * STAGE_BYTES;
                    const int kx = kb * BLOCK_K;
                    if (Q16LIN && pass == 1) {
                        const uint32_t bar = full0 + 8 * s;
                        mbar_arrive_expect_tx(bar, 2 * A_TILE_BYTES + 2 * B_TILE_BYTES);
                        tma_load_2d(dst + 2 * A_TILE_BYTES, &tm_a2, bar, kx, row_a, pol_a);
                        tma_load_2d(dst + 3 * A_TILE_BYTES, &tm_a3, bar, kx, row_a, pol_a);
                        const uint32_t db = dst + cfg::NA * A_TILE_BYTES;
#pragma unroll
                        for (int j = 0; j < B_ROWS / BOX_N; ++j) {
                            tma_load_2d(db + j * B_BOX_BYTES, &tm_b2, bar, row_b + BOX_N * j, kx, pol_b);
                            tma_load_2d(db + B_TILE_BYTES + j * B_BOX_BYTES, &tm_b3, bar, row_b + BOX_N * j, kx, pol_b);
                        }
                    } else if (PAIR == 1) {
                        const uint32_t bar = full0 + 8 * s;
                        mbar_arrive_expect_tx(bar, STAGE_BYTES);
                        tma_load_2d(dst, &tm_a0, bar, kx, row_a, pol_a);
                        if (cfg::NA >= 2) tma_load_2d(dst + A_TILE_BYTES, &tm_a1, bar, kx, row_a, pol_a);
                        if (cfg::NA == 4) {
                            tma_load_2d(dst + 2 * A_TILE_BYTES, &tm_a2, bar, kx, row_a, pol_a);
                            tma_load_2d(dst + 3 * A_TILE_BYTES, &tm_a3, bar, kx, row_a, pol_a);
                        }
                        const uint32_t db = dst + cfg::NA * A_TILE_BYTES;
                        if (!BMN) {
                            tma_load_2d(db, &tm_b0, bar, kx, row_b, pol_b);
                            if (cfg::NB == 2) tma_load_2d(db + B_TILE_BYTES, &tm_b1, bar, kx, row_b, pol_b);
                        } else {
#pragma unroll
                            for (int j = 0; j < B_ROWS / BOX_N; ++j) {
                                tma_load_2d(db + j * B_BOX_BYTES, &tm_b0, bar, row_b + BOX_N * j, kx, pol_b);
                                if (cfg::NB == 2)
                                    tma_load_2d(db + B_TILE_BYTES + j * B_BOX_BYTES, &tm_b1, bar, row_b + BOX_N * j, kx, pol_b);
                            }
                        }
                    } else if (BMN) {
                        const uint32_t bar = mapa(full0 + 8 * s, 0);
                        if (leader) mbar_arrive_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
                        tma_load_2d_pair(dst, &tm_a0, bar, kx, row_a, pol_a);
                        if (cfg::NA == 2) tma_load_2d_pair(dst + A_TILE_BYTES, &tm_a1, bar, kx, row_a, pol_a);
                        const uint32_t db = dst + cfg::NA * A_TILE_BYTES;
#pragma unroll
                        for (int j = 0; j < B_ROWS / 128; ++j) {
                            // with sub-tiles, box j is this CTA's 128 columns of sub-tile j
                            const int col = NSUB == 1 ? row_b + 128 * j : tn * BLOCK_N + j * UMMA_N + (int)cta * SUB_ROWS;
                            tma_load_2d_pair(db + j * B_BOX_BYTES, &tm_b0, bar, col, kx, pol_b);
                            if (cfg::NB == 2)
                                tma_load_2d_pair(db + B_TILE_BYTES + j * B_BOX_BYTES, &tm_b1, bar, col, kx, pol_b);
                        }
                    } else if (NSUB == 2) {
                        const uint32_t bar = mapa(full0 + 8 * s, 0);
                        if (leader) mbar_arrive_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
                        tma_load_2d_pair(dst, &tm_a0, bar, kx, row_a, pol_a);
                        const uint32_t db = dst + cfg::NA * A_TILE_BYTES;
#pragma unroll
                        for (int j = 0; j < NSUB; ++j)
                            tma_load_2d_pair(db + j * SUB_TILE_BYTES, &tm_b0, bar, kx,
                                             tn * BLOCK_N + j * UMMA_N + (int)cta * SUB_ROWS, pol_b);
                    } else {
                        // Both CTAs' copies complete on the LEADER's full barrier (it alone issues
                        // MMAs).  Only the leader arrives, expecting the bytes of both; the peer's
                        // bytes may land first, which a transaction count allows.  No remote
                        // arrive: its release fence would drain the copies in flight every stage.
                        const uint32_t bar = mapa(full0 + 8 * s, 0);
                        if (leader) mbar_arrive_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
                        tma_load_2d_pair(dst, &tm_a0, bar, kx, row_a, pol_a);
                        if (cfg::NA == 2) tma_load_2d_pair(dst + A_TILE_BYTES, &tm_a1, bar, kx, row_a, pol_a);
                        const uint32_t db = dst + cfg::NA * A_TILE_BYTES;
                        tma_load_2d_pair(db, &tm_b0, bar, kx, row_b, pol_b);
                        if (cfg::NB == 2) tma_load_2d_pair(db + B_TILE_BYTES, &tm_b1, bar, kx, row_b, pol_b);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0 && leader) {
            constexpr uint32_t ID_SS = idesc_i8(UMMA_M, UMMA_N, true, true, BMN);
            constexpr uint32_t ID_SU = idesc_i8(UMMA_M, UMMA_N, true, false, BMN);
            constexpr uint32_t ID_US = idesc_i8(UMMA_M, UMMA_N, false, true, BMN);
            constexpr uint32_t ID_UU = idesc_i8(UMMA_M, UMMA_N, false, false, BMN);
            // Descriptor step per MMA (32 of K): 32 bytes along a K-major row, or 32 K-rows of
            // 128 bytes in an MN-major tile; in units of 16 bytes.
            constexpr uint64_t B_KSTEP = BMN ? (UMMA_K * BOX_N) >> 4 : UMMA_K >> 4;
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int item = tile_first; ok && item < total_tiles; item += tile_step, ++tcount) {
                const uint32_t as = tcount % ACC_STAGES, aph = (tcount / ACC_STAGES) & 1u;
                if (!wait_bounded(tempty0 + 8 * as, aph ^ 1u, abort_s, p.err, 2)) break;
                tc_fence_after();
                const uint32_t d0 = tmem_base + as * ACC_COLS;
                const int kb0 = (item % p.k_splits) * kb_per_split;
                const int kb1 = min(k_blocks, kb0 + kb_per_split);
                const int passes = (Q16LIN && p.q16_low) ? 2 : 1;
                for (int pass = 0; ok && pass < passes; ++pass)
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                    if (!wait_bounded(full0 + 8 * s, ph, abort_s, p.err, 3)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = tiles0 + s * STAGE_BYTES;
                    const uint32_t sb = sa + cfg::NA * A_TILE_BYTES;
                    const uint64_t da0 = smem_desc_k_sw128(sa);
                    const uint64_t db0 = !BMN ? smem_desc_k_sw128(sb)
                                         : BOX_N == 128 ? smem_desc_mn_sw128(sb, B_BOX_BYTES) : smem_desc_mn_sw64(sb);
#pragma unroll
                    for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks) {
                        const uint32_t acc = (kb != kb0 || ks != 0 || pass != 0) ? 1u : 0u;
                        const uint64_t koff = (uint64_t)((ks * UMMA_K) >> 4);
                        const uint64_t kb_off = (uint64_t)ks * B_KSTEP;
                        if (MODE == 5) {
#pragma unroll
                            for (int j = 0; j < NSUB; ++j) {
                                const uint32_t sbj = sb + j * SUB_TILE_BYTES;
                                const uint64_t dbj = BMN ? smem_desc_mn_sw128(sbj, B_BOX_BYTES) : smem_desc_k_sw128(sbj);
                                mma_i8<PAIR>(d0 + j * UMMA_N, da0 + koff, dbj + kb_off, ID_SS, acc);
                            }
                        } else if (MODE == 0 || MODE == 3) {
                            mma_i8<PAIR>(d0, da0 + koff, db0 + kb_off, ID_SS, acc);
                        } else if (Q16LIN) {
                            // a = a3*2^24 + a2*2^16 + a1*2^8 + a0 (a3 signed), bh = bh1*256 + bh0 (bh1
                            // signed); accumulator s collects the limb products of weight 2^(8s).
                            const uint64_t a0d = da0 + koff;
                            const uint64_t a1d = smem_desc_k_sw128(sa + A_TILE_BYTES) + koff;
                            const uint64_t a2d = smem_desc_k_sw128(sa + 2 * A_TILE_BYTES) + koff;
                            const uint64_t a3d = smem_desc_k_sw128(sa + 3 * A_TILE_BYTES) + koff;
                            const uint64_t b0d = db0 + kb_off;
                            const uint64_t b1d = (BOX_N == 128 ? smem_desc_mn_sw128(sb + B_TILE_BYTES, B_BOX_BYTES)
                                                               : smem_desc_mn_sw64(sb + B_TILE_BYTES)) + kb_off;
                            if (pass == 1) {
                                // ah * bl, ah = a3*256 + a2 (a3 signed), bl = bl1*256 + bl0 (both unsigned):
                                // the stage's B planes are bl0 and bl1 in this pass
                                mma_i8<PAIR>(d0, a2d, b0d, ID_UU, 1u);                   // a2.bl0      -> s0
                                mma_i8<PAIR>(d0 + BLOCK_N, a3d, b0d, ID_SU, 1u);         // a3.bl0      -> s1
                                mma_i8<PAIR>(d0 + BLOCK_N, a2d, b1d, ID_UU, 1u);         // a2.bl1      -> s1
                                mma_i8<PAIR>(d0 + 2 * BLOCK_N, a3d, b1d, ID_SU, 1u);     // a3.bl1      -> s2
                                continue;
                            }
                            mma_i8<PAIR>(d0, a0d, b0d, ID_UU, acc);                  // a0.bh0      -> s0
                            mma_i8<PAIR>(d0 + BLOCK_N, a0d, b1d, ID_US, acc);        // a0.bh1      -> s1
                            mma_i8<PAIR>(d0 + BLOCK_N, a1d, b0d, ID_UU, 1u);         // a1.bh0      -> s1
                            mma_i8<PAIR>(d0 + 2 * BLOCK_N, a1d, b1d, ID_US, acc);    // a1.bh1      -> s2
                            mma_i8<PAIR>(d0 + 2 * BLOCK_N, a2d, b0d, ID_UU, 1u);     // a2.bh0      -> s2
                            mma_i8<PAIR>(d0 + 3 * BLOCK_N, a2d, b1d, ID_US, acc);    // a2.bh1      -> s3
                            mma_i8<PAIR>(d0 + 3 * BLOCK_N, a3d, b0d, ID_SU, 1u);     // a3.bh0      -> s3
                        } else {
                            // The two planes of B lie side by side in the stage (high, then low
                            // minus 128: both signed), exactly like a 2 x BLOCK_N wide int8 tile, so
                            // one MMA of N = 2 x BLOCK_N forms [hi.hi | hi.lo'] and a second one
                            // [lo.hi | lo.lo']: A is read from shared memory twice per 32 of K
                            // instead of four times (the kernel is bound by shared-memory reads).
                            static_assert(MODE != 1 || B_TILE_BYTES == B_BOX_BYTES, "planes must be adjacent boxes");
                            constexpr uint32_t ID2_SS = idesc_i8(UMMA_M, 2 * BLOCK_N, true, true, BMN);
                            constexpr uint32_t ID2_US = idesc_i8(UMMA_M, 2 * BLOCK_N, false, true, BMN);
                            const uint64_t da1 = smem_desc_k_sw128(sa + A_TILE_BYTES) + koff;
                            mma_i8<PAIR>(d0, da0 + koff, db0 + kb_off, ID2_SS, acc);               // hi.[hi | lo']
                            mma_i8<PAIR>(d0 + 2 * BLOCK_N, da1, db0 + kb_off, ID2_US, acc);        // lo.[hi | lo']
                        }
                    }
                    if (PAIR == 1)
                        mma_commit(empty0 + 8 * s);
                    else
                        mma_commit_pair(empty0 + 8 * s, 3);
                }
                if (!ok) break;
                if (PAIR == 1)
                    mma_commit(tfull0 + 8 * as);
                else
                    mma_commit_pair(tfull0 + 8 * as, 3);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int q = warp & 3;  // TMEM lane quadrant this warp may read
        const int c_first = ((warp - 2) / 4) * EPI_COLS;  // its share of the tile's columns
        // each epilogue warp owns EPI_PATCHES patches of 4 KiB (two where shared memory allows: a
        // block is written while the tensor store of the one before still reads its patch)
        constexpr int EPI_PATCHES = cfg::EPI_PATCHES;
        uint32_t* const patch = reinterpret_cast<uint32_t*>(smem_raw + (patches0 - raw)) + (warp - 2) * EPI_PATCHES * EPI_PATCH_WORDS;
        const uint32_t patch_first = patches0 + (uint32_t)(warp - 2) * (EPI_PATCHES * EPI_PATCH_WORDS * 4);
        uint32_t blocks_stored = 0;
        uint32_t tcount = 0;
        for (int item = tile_first; item < total_tiles; item += tile_step, ++tcount) {
            int tm, tn;
            tile_coords(item / p.k_splits, p.m_tiles, p.n_tiles, p.group_m, p.raster, tm, tn);
            const bool first_split = item % p.k_splits == 0;  // the int16 offset term goes in once
            (void)first_split;
            const uint32_t as = tcount % ACC_STAGES, aph = (tcount / ACC_STAGES) & 1u;
            const int row = (tm * PAIR + (int)cta) * BLOCK_M + q * 32 + lane;
            // int16: 128 * (row sum of A) puts back the 128 taken off B's low plane.  Fetched before
            // the wait for the accumulator, so that the load's latency hides behind the main loop.
            uint32_t back = 0u;
            if (MODE == 1 && row < p.m && first_split) back = 128u * (uint32_t)__ldg(p.row_sums + row);
            if (!wait_bounded(tfull0 + 8 * as, aph, abort_s, p.err, 4)) break;
            tc_fence_after();
            const int col_tile = tn * BLOCK_N;
            const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + as * ACC_COLS;
            for (int c0 = c_first; c0 < c_first + EPI_COLS; c0 += 32) {
                if (col_tile + c0 >= p.n) break;  // warp-uniform
                uint32_t v[32];
                if (MODE == 0 || MODE == 3 || MODE == 5) {
                    tmem_ld32(t0 + c0, v);
                    tmem_ld_wait();
                } else if (Q16LIN) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint32_t s0[16], s1[16], s2[16], s3[16];
                        tmem_ld16(t0 + c0 + 16 * h, s0);
                        tmem_ld16(t0 + BLOCK_N + c0 + 16 * h, s1);
                        tmem_ld16(t0 + 2 * BLOCK_N + c0 + 16 * h, s2);
                        tmem_ld16(t0 + 3 * BLOCK_N + c0 + 16 * h, s3);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            v[16 * h + j] = s0[j] + (s1[j] << 8) + (s2[j] << 16) + (s3[j] << 24);
                    }
                } else {
                    // columns [0, N) hi.hi, [N, 2N) hi.lo', [2N, 3N) lo.hi, [3N, 4N) lo.lo' with
                    // lo' = lo - 128: `back` puts the 128 back (all mod 2^32)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint32_t hh[16], hl[16], lh[16], ll[16];
                        tmem_ld16(t0 + c0 + 16 * h, hh);
                        tmem_ld16(t0 + BLOCK_N + c0 + 16 * h, hl);
                        tmem_ld16(t0 + 2 * BLOCK_N + c0 + 16 * h, lh);
                        tmem_ld16(t0 + 3 * BLOCK_N + c0 + 16 * h, ll);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            v[16 * h + j] = (hh[j] << 16) + ((hl[j] + lh[j]) << 8) + ll[j] + back;
                    }
                }
                if (p.tma_store && row - lane < p.m) {  // (a block wholly below the matrix has nothing to store)
                    // The block goes to this warp's patch as 32 rows of 128 bytes in the 128-byte
                    // swizzle (lane = row; its eight 16-byte pieces land on eight different bank
                    // groups), and ONE bulk tensor store writes it out: nine instructions per block
                    // instead of ninety-six, and rows / columns past the matrix edge are clipped by
                    // the hardware.  The patch is reused once the previous store has read it.
                    if (lane == 0) bulk_wait_group_read<EPI_PATCHES - 1>();
                    __syncwarp();
                    const uint32_t patch_addr = patch_first + (blocks_stored++ % EPI_PATCHES) * (EPI_PATCH_WORDS * 4);
                    const uint32_t prow = patch_addr + (uint32_t)lane * 128u;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        st_shared_v4(prow + (uint32_t)((j ^ (lane & 7)) << 4), v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tm_c, patch_addr, col_tile + c0, row - lane);
                        bulk_commit_group();
                    }
                    continue;
                }
                if (p.tma_store) continue;
                // Lane = row in TMEM, but a store wants lane = column: the 32 x 32 block goes through
                // this warp's shared-memory patch (word j of row l at l * 32 + (j ^ l): no bank
                // conflicts either way), and every store / atomic instruction then covers one
                // 128-byte line of a row.  Straight from registers each lane wrote 16 bytes of a
                // different row, which held output-bound shapes (short K) to a third of the write
                // bandwidth.
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 32; ++j) patch[lane * 32 + (j ^ lane)] = v[j];
                __syncwarp();
                const int col = col_tile + c0 + lane;
                const int row_first = row - lane;
                if (col < p.n) {
                    int32_t* dst = p.c + (size_t)row_first * (size_t)p.n + col;
#pragma unroll 8
                    for (int r = 0; r < 32; ++r) {
                        if (row_first + r >= p.m) break;  // warp-uniform
                        const uint32_t x = patch[r * 32 + (lane ^ r)];
                        if (p.accumulate)
                            atomicAdd(reinterpret_cast<unsigned int*>(dst), x);
                        else
                            *dst = (int32_t)x;
                        dst += p.n;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR == 1)
                    mbar_arrive(tempty0 + 8 * as);
                else
                    mbar_arrive_cluster(tempty0 + 8 * as, 0);
            }
        }
        if (lane == 0) bulk_wait_group<0>();  // this warp's tensor stores have left shared memory and landed
    }

    // ------------------------------------------------------------------ teardown
    __syncwarp();
    if (*abort_s) __nanosleep(200000);  // let copies / MMAs still in flight land before freeing
    tc_fence_before();
    __syncthreads();
    if (PAIR == 2) {
        cluster_arrive();
        cluster_wait();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<PAIR>(tmem_base, TMEM_COLS);
    }
}

// A wait that nothing will ever satisfy, with a short limit: exercises the give-up path of
// wait_bounded (error word written, kernel returns, context stays usable).
__global__ void wait_selftest_kernel(int* err, unsigned long long limit_ns) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) wait_bounded(smem_u32(&bar), 0, &abort_flag, err, 9, limit_ns);
}

// 2-D map over a row-major 8-bit matrix [rows][k] with row pitch `pitch` bytes; the
// box is 128 bytes of K by `box_rows` rows, written to shared memory with the
// 128-byte swizzle.  Reads past `k` or `rows` return zeros.
// box_bytes = 64 makes boxes of 64 bytes with the 64-byte swizzle instead (narrow MN-major B tiles).
// A tensor map is a pure function of these arguments, so the last few are kept per thread:
// launch-bound callers repeat the same operands, and an encode costs about as much as a launch.
struct TmapKey {
    const void* base;
    int64_t k, rows, pitch;
    int box_rows, box_bytes;
    bool operator==(const TmapKey& o) const {
        return base == o.base && k == o.k && rows == o.rows && pitch == o.pitch && box_rows == o.box_rows &&
               box_bytes == o.box_bytes;
    }
};
struct TmapCache {
    static constexpr int N = 8;
    TmapKey key[N];
    CUtensorMap map[N];
    int used = 0, next = 0;
};

// Map over the int32 output C[m][n] for the epilogue's stores: boxes of 32 columns (128 bytes) by
// 32 rows, read from shared memory in the 128-byte swizzle.  Needs a 16-byte aligned base and
// N % 4 == 0 (the caller checks).
int64_t make_tmap_c(CUtensorMap* tm, int32_t* c, int64_t n, int64_t m) {
    static thread_local TmapCache cache;
    const TmapKey want{c, n, m, n * 4, 32, -32};
    for (int i = 0; i < cache.used; ++i)
        if (cache.key[i] == want) {
            *tm = cache.map[i];
            return 0;
        }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(MIND_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)m};
    cuuint64_t strides[1] = {(cuuint64_t)n * 4};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, c, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(MIND_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed for the output with CUresult %d (n=%lld m=%lld)",
                    (int)r, (long long)n, (long long)m);
    cache.key[cache.next] = want;
    cache.map[cache.next] = *tm;
    cache.next = (cache.next + 1) % TmapCache::N;
    if (cache.used < TmapCache::N) ++cache.used;
    return 0;
}

int64_t make_tmap(CUtensorMap* tm, const void* base, int64_t k, int64_t rows, int64_t pitch,
                  int box_rows, int box_bytes = BLOCK_K) {
    static thread_local TmapCache cache;
    const TmapKey want{base, k, rows, pitch, box_rows, box_bytes};
    for (int i = 0; i < cache.used; ++i)
        if (cache.key[i] == want) {
            *tm = cache.map[i];
            return 0;
        }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(MIND_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch};
    cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                     estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     box_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(MIND_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (k=%lld rows=%lld pitch=%lld)",
                    (int)r, (long long)k, (long long)rows, (long long)pitch);
    cache.key[cache.next] = want;
    cache.map[cache.next] = *tm;
    cache.next = (cache.next + 1) % TmapCache::N;
    if (cache.used < TmapCache::N) ++cache.used;
    return 0;
}

// kp_b: row pitch of the B operand(s) in bytes: of Bt[N][K] rows (BMN = false) or of
// B[K][N] rows (BMN = true).
template <int MODE, int PAIR, bool BMN>
int64_t launch_tc(DeviceCtx* ctx, const void* a0, const void* a1, const void* b0, const void* b1,
                  int32_t* c, int64_t m, int64_t n, int64_t k, int64_t kp_a, int64_t kp_b,
                  const void* a2 = nullptr, const void* a3 = nullptr, const int32_t* row_sums = nullptr,
                  bool accumulate = false, int max_ctas = 0, const void* b2 = nullptr, const void* b3 = nullptr) {
    using cfg = Cfg<MODE, PAIR>;
    constexpr int B_ROWS = cfg::BLOCK_N / PAIR;
    constexpr int BOX_N = B_ROWS < 128 ? B_ROWS : 128;  // width of an MN-major box = its swizzle width
    constexpr int STAGE_BYTES = cfg::NA * A_TILE_BYTES + cfg::NB * B_ROWS * BLOCK_K;
    constexpr int SMEM = cfg::STAGES * STAGE_BYTES + 1024 + 1024 + epi_warps<MODE, PAIR>() * cfg::EPI_PATCHES * EPI_PATCH_WORDS * 4;
    static_assert(SMEM <= 232448, "shared memory budget");
    if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff)
        return fail(MIND_B200_ERR_TOO_LARGE, "GEMM dimension above 2^31-1");
    CUtensorMap ta0, ta1, tb0, tb1;
    MB200_TRY(make_tmap(&ta0, a0, k, m, kp_a, BLOCK_M));
    if (BMN)
        MB200_TRY(make_tmap(&tb0, b0, n, k, kp_b, BLOCK_K, BOX_N));  // boxes of BOX_N columns x 128 rows of K
    else
        MB200_TRY(make_tmap(&tb0, b0, k, n, kp_b, B_ROWS / cfg::NSUB));
    ta1 = ta0;
    tb1 = tb0;
    CUtensorMap ta2 = ta0, ta3 = ta0;
    if (cfg::NA >= 2) MB200_TRY(make_tmap(&ta1, a1, k, m, kp_a, BLOCK_M));
    if (cfg::NA == 4) {
        MB200_TRY(make_tmap(&ta2, a2, k, m, kp_a, BLOCK_M));
        MB200_TRY(make_tmap(&ta3, a3, k, m, kp_a, BLOCK_M));
    }
    if (cfg::NB == 2) {
        if (BMN)
            MB200_TRY(make_tmap(&tb1, b1, n, k, kp_b, BLOCK_K, BOX_N));
        else
            MB200_TRY(make_tmap(&tb1, b1, k, n, kp_b, B_ROWS));
    }
    CUtensorMap tb2 = tb0, tb3 = tb0;
    if (b2 && b3) {  // Q16.16: the planes of b & 0xffff, for the second pass
        MB200_TRY(make_tmap(&tb2, b2, n, k, kp_b, BLOCK_K, BOX_N));
        MB200_TRY(make_tmap(&tb3, b3, n, k, kp_b, BLOCK_K, BOX_N));
    }
    TcParams p;
    p.q16_low = (b2 && b3) ? 1 : 0;
    p.c = c;
    p.m = (int)m;
    p.n = (int)n;
    p.k = (int)k;
    p.m_tiles = (int)((m + BLOCK_M * PAIR - 1) / (BLOCK_M * PAIR));
    p.n_tiles = (int)((n + cfg::BLOCK_N - 1) / cfg::BLOCK_N);
    p.row_sums = row_sums;
    p.accumulate = accumulate ? 1 : 0;
    p.err = ctx->err_word;
    // Tile order and L2 policy, measured at 16384^3 (DRAM reads were 16x the operand bytes with
    // 16 m-tiles per group and no hints): groups of 8 m-tiles keep the group's A panels
    // (8 x 256 rows x K) L2-resident across successive waves; A is marked evict-last, B is left
    // at the normal policy (marking it evict-first throws away panels a wave still shares).
    // Odd groups walk N backwards (a group starts on the B panels the last one ended on): 6 % fewer
    // DRAM reads again at 16384^3 (ncu, one launch each: 6.16 -> 5.77 GB; groups of 4 / 6 / 12 / 16
    // m-tiles read 7.7 - 8.8 / 6.3 - 6.9 / 6.1 - 6.2 / 6.1 GB).
    const int knob_group = tuning().group_m.load(), knob_raster = tuning().raster.load();
    p.group_m = knob_group > 0 ? knob_group : 8;
    p.raster = knob_raster == 2 ? 0 : 1;  // 0 = default (1), 2 = every group forwards, 3 = default order (see direct_store)
    p.hint_a = 1;
    p.hint_b = 0;
    const long long total = (long long)p.m_tiles * p.n_tiles;
    if (total > 0x7fffffff) return fail(MIND_B200_ERR_TOO_LARGE, "too many output tiles");
    auto kern = gemm_tc_kernel<MODE, PAIR, BMN>;
    static thread_local int done_for = -1;  // one per template instance
    if (done_for != ctx->device) {
        MB200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        done_for = ctx->device;
    }
    int units = ctx->sm_count / PAIR;  // CTAs (or CTA pairs) resident at once
    // Fewer tiles than a quarter of the SMs and a long K: cut every tile's K range into splits, one work
    // item each, all adding onto a zeroed C with red.global.add (sums mod 2^32 commute), so that a
    // tall-and-skinny product (64 x 16384 x 64 is one tile) still uses the whole GPU.
    int splits = 1;
    const int64_t k_blocks = (k + BLOCK_K - 1) / BLOCK_K;
    if (total * 4 <= units && k_blocks >= 16) {
        int64_t want = units / total;
        if (want > k_blocks / 4) want = k_blocks / 4;
        if (want > 32) want = 32;
        // below four splits the zeroing of C and the atomics cost what the split saves (1024^3)
        if (want >= 4) {
            const int64_t per = (k_blocks + want - 1) / want;
            splits = (int)((k_blocks + per - 1) / per);  // no empty split
        }
    }
    p.k_splits = splits;
    if (splits > 1 && !p.accumulate) {
        MB200_CUDA(cudaMemsetAsync(c, 0, (size_t)m * (size_t)n * 4, ctx->stream));
        p.accumulate = 1;
    }
    // Epilogue through TMA stores where the hardware can address C (16-byte base and pitch) and
    // nothing else adds onto it meanwhile; otherwise plain row stores / atomics.
    p.tma_store = (!p.accumulate && n % 4 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0 &&
                   tuning().raster.load() != 3) ? 1 : 0;
    CUtensorMap tc = ta0;
    if (p.tma_store) MB200_TRY(make_tmap_c(&tc, c, n, m));
    const long long items = total * splits;
    if (items < units) units = (int)items;
    if (max_ctas > 0 && PAIR == 1 && units > max_ctas) units = max_ctas;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)(units * PAIR), 1, 1);
    lc.blockDim = dim3(tc_threads<MODE, PAIR>(), 1, 1);
    lc.dynamicSmemBytes = SMEM;
    lc.stream = ctx->stream;
    cudaLaunchAttribute at[2];
    int n_at = 0;
    if (PAIR == 2) {
        at[n_at].id = cudaLaunchAttributeClusterDimension;
        at[n_at].val.clusterDim.x = PAIR;
        at[n_at].val.clusterDim.y = 1;
        at[n_at].val.clusterDim.z = 1;
        ++n_at;
    }
    if (MODE == 3 || MODE == 1) {  // see griddep_launch_dependents / griddep_wait in the kernel
        at[n_at].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[n_at].val.programmaticStreamSerializationAllowed = 1;
        ++n_at;
    }
    lc.attrs = at;
    lc.numAttrs = n_at;
    if (PAIR == 2) {
        // Not every SM need be pairable; a pair that is not resident would only start
        // after another one ends, so size the persistent grid to what fits at once.
        static thread_local int fit_dev = -1, fit = 0;  // per template instance; asked once per device
        if (fit_dev != ctx->device) {
            lc.gridDim = dim3((unsigned)(ctx->sm_count / PAIR * PAIR), 1, 1);
            if (cudaOccupancyMaxActiveClusters(&fit, kern, &lc) != cudaSuccess) {
                cudaGetLastError();
                fit = 0;
            }
            fit_dev = ctx->device;
            lc.gridDim = dim3((unsigned)(units * PAIR), 1, 1);
        }
        if (fit > 0 && fit < units) {
            units = fit;
            lc.gridDim = dim3((unsigned)(units * PAIR), 1, 1);
        }
    }
    prof_begin(ctx);
    MB200_CUDA(cudaLaunchKernelEx(&lc, kern, ta0, ta1, ta2, ta3, tb0, tb1, tb2, tb3, tc, p));
    prof_end(ctx);
    count_launch();
    return check_launch("gemm_tc_kernel");
}

}  // namespace

int64_t make_tmap_c32(CUtensorMap* tm, int32_t* c, int64_t n, int64_t m) { return make_tmap_c(tm, c, n, m); }

int64_t make_tmap_u8(CUtensorMap* tm, const void* base, int64_t k, int64_t rows, int64_t pitch, int box_rows,
                     int box_bytes) {
    return make_tmap(tm, base, k, rows, pitch, box_rows, box_bytes);
}

int64_t launch_wait_selftest(DeviceCtx* ctx, int64_t limit_ms) {
    wait_selftest_kernel<<<1, 32, 0, ctx->stream>>>(ctx->err_word, (unsigned long long)limit_ms * 1000000ull);
    count_launch();
    return check_launch("wait_selftest_kernel");
}

// Measured on B200: the CTA-pair kernel is the faster int8 kernel once there is more than one
// 128 x 256 tile per SM (3072^3 and up: +6 % to +17 %); below that one CTA per tile is as fast
// or slightly faster and needs no cluster launch.
static bool pair_pays(const DeviceCtx* ctx, int64_t m, int64_t n) {
    return m > 128 && ((m + 127) / 128) * ((n + 255) / 256) > ctx->sm_count;
}

// Few wide tiles and a K too short to split: 128 x 64 tiles spread the product over four times
// as many SMs, each with a quarter of the epilogue (256^3: 2 CTAs -> 8).
static bool narrow_pays(const DeviceCtx* ctx, int64_t m, int64_t n, int64_t k) {
    const int knob = tuning().small_tile.load();
    if (knob >= 0) return knob == 1;
    if (tuning().pair_mode.load() != 0) return false;  // a kernel was asked for by name
    const int64_t wide_tiles = ((m + 127) / 128) * ((n + 255) / 256);
    return wide_tiles * 4 <= ctx->sm_count && (k + BLOCK_K - 1) / BLOCK_K < 16;
}

// 256 x 512 tiles on CTA pairs: their epilogue is not overlapped, so only where a tile's main
// loop is long (K) and there are tiles enough to keep every pair busy for several rounds.
static bool wide_pair_pays(const DeviceCtx* ctx, int64_t m, int64_t n, int64_t k) {
    const int knob = tuning().wide_pair.load();
    if (knob >= 0) return knob == 1;
    if (tuning().pair_mode.load() != 0) return false;
    return k >= 16384 && ((m + 255) / 256) * ((n + 511) / 512) >= 4 * (ctx->sm_count / 2);
}

int64_t launch_gemm_i8_tc(DeviceCtx* ctx, const int8_t* a, const int8_t* bt, int32_t* c, int64_t m,
                          int64_t n, int64_t k, int64_t kp_a, int64_t kp_b) {
    if (narrow_pays(ctx, m, n, k)) return launch_tc<3, 1, false>(ctx, a, nullptr, bt, nullptr, c, m, n, k, kp_a, kp_b);
    if (wide_pair_pays(ctx, m, n, k)) return launch_tc<5, 2, false>(ctx, a, nullptr, bt, nullptr, c, m, n, k, kp_a, kp_b);
    const int pair_mode = tuning().pair_mode.load();
    const bool pair = pair_mode == 2 || (pair_mode == 0 && pair_pays(ctx, m, n));
    if (pair) return launch_tc<0, 2, false>(ctx, a, nullptr, bt, nullptr, c, m, n, k, kp_a, kp_b);
    return launch_tc<0, 1, false>(ctx, a, nullptr, bt, nullptr, c, m, n, k, kp_a, kp_b);
}

int64_t launch_gemm_i8_tc_bmn(DeviceCtx* ctx, const int8_t* a, const int8_t* b, int32_t* c, int64_t m,
                              int64_t n, int64_t k, int64_t kp_a, int64_t pitch_b) {
    if (narrow_pays(ctx, m, n, k)) return launch_tc<3, 1, true>(ctx, a, nullptr, b, nullptr, c, m, n, k, kp_a, pitch_b);
    if (wide_pair_pays(ctx, m, n, k)) return launch_tc<5, 2, true>(ctx, a, nullptr, b, nullptr, c, m, n, k, kp_a, pitch_b);
    const int pair_mode = tuning().pair_mode.load();
    const bool pair = pair_mode == 2 || (pair_mode == 0 && pair_pays(ctx, m, n));
    if (pair) return launch_tc<0, 2, true>(ctx, a, nullptr, b, nullptr, c, m, n, k, kp_a, pitch_b);
    return launch_tc<0, 1, true>(ctx, a, nullptr, b, nullptr, c, m, n, k, kp_a, pitch_b);
}

bool tc_pair_forced() { return tuning().pair_mode.load() == 2; }

// Linear part of the Q16.16 GEMM on tensor cores, mod 2^32, from byte planes: a_limb[0..3] the
// bytes of a (a_limb[3] signed), b_limb[0..1] the bytes of bh = b >> 16 (b_limb[1] signed) and,
// when given, b_limb[2..3] the bytes of bl = b & 0xffff; B planes in B's own orientation
// ([K][pitch_b]).  Without bl planes P = sum_k a * bh (seven limb products); with them
// P = sum_k a * bh + (a >> 16) * bl (four more, in a second pass over K).
// accumulate: add onto p_out (red.global.add) instead of storing; max_ctas > 0 caps the persistent
// grid, for running beside another kernel that holds the other SMs.
int64_t launch_gemm_q16_linear_tc(DeviceCtx* ctx, const uint8_t* const a_limb[4], const uint8_t* const b_limb[4],
                                  int32_t* p_out, int64_t m, int64_t n, int64_t k, int64_t kp_a,
                                  int64_t pitch_b, bool accumulate, int max_ctas) {
    // fewer 128 x 128 tiles than SMs: 64-column tiles put twice as many CTAs on a latency-bound product
    if (max_ctas <= 0 && ((m + 127) / 128) * ((n + 127) / 128) < ctx->sm_count)
        return launch_tc<4, 1, true>(ctx, a_limb[0], a_limb[1], b_limb[0], b_limb[1], p_out, m, n, k, kp_a,
                                     pitch_b, a_limb[2], a_limb[3], nullptr, accumulate, max_ctas, b_limb[2], b_limb[3]);
    return launch_tc<2, 1, true>(ctx, a_limb[0], a_limb[1], b_limb[0], b_limb[1], p_out, m, n, k, kp_a,
                                 pitch_b, a_limb[2], a_limb[3], nullptr, accumulate, max_ctas, b_limb[2], b_limb[3]);
}

int64_t launch_gemm_i16_tc_bmn(DeviceCtx* ctx, const int8_t* a_hi, const uint8_t* a_lo,
                               const int8_t* b_hi, const uint8_t* b_lo, const int32_t* a_row_sums,
                               int32_t* c, int64_t m, int64_t n, int64_t k, int64_t kp_a, int64_t pitch_b) {
    return launch_tc<1, 1, true>(ctx, a_hi, a_lo, b_hi, b_lo, c, m, n, k, kp_a, pitch_b, nullptr, nullptr,
                                 a_row_sums);
}

int64_t launch_gemm_i16_tc(DeviceCtx* ctx, const int8_t* a_hi, const uint8_t* a_lo,
                           const int8_t* bt_hi, const uint8_t* bt_lo, const int32_t* a_row_sums,
                           int32_t* c, int64_t m, int64_t n, int64_t k, int64_t kp) {
    return launch_tc<1, 1, false>(ctx, a_hi, a_lo, bt_hi, bt_lo, c, m, n, k, kp, kp, nullptr, nullptr,
                                  a_row_sums);
}

}  // namespace mb200
