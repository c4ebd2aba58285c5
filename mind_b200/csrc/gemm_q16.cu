// Q16.16 GEMM with the per-product floor on the FP64 pipe.
//
//   C[i,j] = (i32) sum_k ((i64)A[i,k] * (i64)B[k,j]) >> 16        (shift per product)
//
// With bl = b & 0xffff (unsigned) and bh = b >> 16 (arithmetic):
//     (a * b) >> 16 = a * bh + floor(a * bl / 65536).
// The all-integer kernel (gemm_simt.cu) spends a mad.lo and a mad.hi per product and is bound by
// the 32-bit integer multiplier (mad.hi issues at a quarter of the FP32 rate; measured ~11 Top/s
// at 4096^3 with every tile size).  Here the floor term moves to the FP64 pipe:
//     |a * bl| < 2^47, so a * (bl * 2^-16) is exact in binary64, and
//     fma.rm.f64(a, bl * 2^-16, t) = t + floor(a * bl / 65536)  exactly
// whenever t is an integer-valued binary64 in [2^52, 2^53) (one rounding, toward minus
// infinity, at unit weight).  Every term is below 2^31 in magnitude, so starting from
// t = 1.5 * 2^52 the chain accumulates sum_k floor(a * bl / 65536) exactly for 2^20 products,
// and the low mantissa word of t is that sum mod 2^32.  The launcher cuts a longer K into slices
// of 2^20 (c accumulates across them).
//
// One kernel, two forms:
//   FULL   everything on the CUDA cores: a * bh with mad.lo.s32 beside the fma.rm.f64 chain
//          (8 x 4 outputs per thread, 128 x 64 per block).  Small and mid-sized calls.
//   floor  only the floor term, added onto the linear part a * bh that the tensor cores have
//          already written to c (the hybrid, large calls).  What bounds it is the FP64 pipe's
//          operand traffic through the register file, not shared memory (measured: the same
//          rate with half and with a quarter of the shared-memory bytes), so the register tile
//          is the largest that fits: 8 x 8 outputs per thread, 128 x 128 per block.
//
// bl * 2^-16 has at most 16 significant bits, so the low word of its binary64 form is zero:
// shared memory holds only the HIGH word (4 bytes per element) and the register pair is
// completed with a zero.  A is converted to binary64 once per element on its way to shared
// memory (converting in the inner loop made the conversion unit the bottleneck).
//
// Work is dealt out stream-K fashion: the units are (output tile, 16-deep K step) pairs in
// tile-major order, block b takes units [b * U / G, (b + 1) * U / G), and every run of units
// inside one tile ends with red.global.add.u32 onto c (zeroed first in the FULL form).  Sums
// mod 2^32 commute, so the result does not depend on which block adds first, and every SM gets
// the same number of K steps whatever the tile count (8 tiles at 256^3, 64 at 1024^3).
//
// Shared memory is double buffered: the tile for step t + 1 is written while step t is read, one
// barrier per step.  Needs 16-byte aligned operands with K % 4 == 0 and N % 4 == 0; other calls
// use the integer kernel.
#include "common.h"

namespace mb200 {
namespace {

constexpr int QBM = 128, QBK = 16;
constexpr int QTHREADS = 256;

__device__ __forceinline__ uint32_t mad_lo_u(int32_t a, int32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.lo.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ double fma_rm(double a, double b, double c) {
    double d;
    asm("fma.rm.f64 %0, %1, %2, %3;" : "=d"(d) : "d"(a), "d"(b), "d"(c));
    return d;
}
// high word of the binary64 value (v & 0xffff) * 2^-16: the exponent drops by 16, zero stays zero
__device__ __forceinline__ int32_t q16_low_hi_word(int32_t v) {
    const int32_t bl = v & 0xffff;
    return bl ? __double2hiint(__int2double_rn(bl)) - (16 << 20) : 0;
}

template <int BN, bool FULL>
struct Q16Smem {
    double ad[2][QBK][QBM + 2];                          // A as binary64
    int32_t bw[2][QBK][BN];                              // high words of (b & 0xffff) * 2^-16
    int32_t as[FULL ? 2 : 1][FULL ? QBK : 1][QBM + 4];   // A as int32 (FULL only)
    int32_t bh[FULL ? 2 : 1][FULL ? QBK : 1][BN];        // b >> 16 (FULL only)
};

template <int BN, bool FULL>
__global__ void __launch_bounds__(QTHREADS, 1)
gemm_q16_fp64_kernel(const int32_t* __restrict__ a, const int32_t* __restrict__ b, int32_t* __restrict__ c,
                     int m, int k, int n, int lda, int n_tiles, int k_steps, long long units, int exclusive) {
    constexpr int TM = QBM / 16, TN = BN / 16;
    static_assert(TM % 4 == 0 && TN % 4 == 0, "register tile is built from 4-wide groups");
    extern __shared__ __align__(16) unsigned char q16_smem[];
    Q16Smem<BN, FULL>& sm = *reinterpret_cast<Q16Smem<BN, FULL>*>(q16_smem);

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    constexpr int A_VEC = QBM * QBK / 4 / QTHREADS;  // 16-byte vectors per thread
    constexpr int B_VEC = BN * QBK / 4 / QTHREADS;
    int4 ra[A_VEC], rb[B_VEC];
    int row0 = 0, col0 = 0;

    auto load_tiles = [&](int k0) {
#pragma unroll
        for (int i = 0; i < A_VEC; ++i) {
            const int r = (tid >> 2) + 64 * i, kk = k0 + (tid & 3) * 4;
            ra[i] = make_int4(0, 0, 0, 0);
            if (row0 + r < m && kk < k) ra[i] = *reinterpret_cast<const int4*>(a + (size_t)(row0 + r) * lda + kk);
        }
#pragma unroll
        for (int i = 0; i < B_VEC; ++i) {
            const int e = tid + QTHREADS * i;
            const int kk = k0 + e / (BN / 4), cc = (e % (BN / 4)) * 4;
            rb[i] = make_int4(0, 0, 0, 0);
            if (kk < k && col0 + cc < n) rb[i] = *reinterpret_cast<const int4*>(b + (size_t)kk * n + col0 + cc);
        }
    };
    auto store_tiles = [&](int buf) {
#pragma unroll
        for (int i = 0; i < A_VEC; ++i) {
            const int r = (tid >> 2) + 64 * i, kq = (tid & 3) * 4;
            if (FULL) {
                sm.as[buf][kq][r] = ra[i].x; sm.as[buf][kq + 1][r] = ra[i].y;
                sm.as[buf][kq + 2][r] = ra[i].z; sm.as[buf][kq + 3][r] = ra[i].w;
            }
            sm.ad[buf][kq][r] = __int2double_rn(ra[i].x); sm.ad[buf][kq + 1][r] = __int2double_rn(ra[i].y);
            sm.ad[buf][kq + 2][r] = __int2double_rn(ra[i].z); sm.ad[buf][kq + 3][r] = __int2double_rn(ra[i].w);
        }
#pragma unroll
        for (int i = 0; i < B_VEC; ++i) {
            const int e = tid + QTHREADS * i;
            const int kq = e / (BN / 4), cc = (e % (BN / 4)) * 4;
            if (FULL)
                *reinterpret_cast<int4*>(&sm.bh[buf][kq][cc]) =
                    make_int4(rb[i].x >> 16, rb[i].y >> 16, rb[i].z >> 16, rb[i].w >> 16);
            *reinterpret_cast<int4*>(&sm.bw[buf][kq][cc]) = make_int4(
                q16_low_hi_word(rb[i].x), q16_low_hi_word(rb[i].y), q16_low_hi_word(rb[i].z), q16_low_hi_word(rb[i].w));
        }
    };

    const double MAGIC = 6755399441055744.0;  // 1.5 * 2^52: unit weight in the last place
    const long long u_end = units * (blockIdx.x + 1) / gridDim.x;
    long long u = units * blockIdx.x / gridDim.x;
    while (u < u_end) {
        // one run: the units of this block that lie in one output tile
        const int tile = (int)(u / k_steps), s_begin = (int)(u % k_steps);
        const long long left = u_end - u;
        const int s_end = left < (long long)(k_steps - s_begin) ? s_begin + (int)left : k_steps;
        u += s_end - s_begin;
        row0 = (tile / n_tiles) * QBM;
        col0 = (tile % n_tiles) * BN;

        uint32_t acc[FULL ? TM : 1][FULL ? TN : 1];
        double facc[TM][TN];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                facc[i][j] = MAGIC;
                if (FULL) acc[i][j] = 0u;
            }

        __syncthreads();  // the previous run's last reads of buffer 0
        load_tiles(s_begin * QBK);
        store_tiles(0);
        if (s_begin + 1 < s_end) load_tiles((s_begin + 1) * QBK);
        __syncthreads();
        for (int s = s_begin; s < s_end; ++s) {
            const int buf = (s - s_begin) & 1;
            if (s + 1 < s_end) {
                store_tiles(buf ^ 1);  // read last in step s - 1, which every warp has left
                if (s + 2 < s_end) load_tiles((s + 2) * QBK);
            }
#pragma unroll 4
            for (int kk = 0; kk < QBK; ++kk) {
                int32_t av[FULL ? TM : 1], bh[FULL ? TN : 1];
                double ad[TM], bd[TN];
#pragma unroll
                for (int g = 0; g < TM / 4; ++g) {
                    const double2 d0 = *reinterpret_cast<const double2*>(&sm.ad[buf][kk][g * 64 + ty * 4]);
                    const double2 d1 = *reinterpret_cast<const double2*>(&sm.ad[buf][kk][g * 64 + ty * 4 + 2]);
                    ad[4 * g] = d0.x; ad[4 * g + 1] = d0.y; ad[4 * g + 2] = d1.x; ad[4 * g + 3] = d1.y;
                    if (FULL) {
                        const int4 v = *reinterpret_cast<const int4*>(&sm.as[buf][kk][g * 64 + ty * 4]);
                        av[4 * g] = v.x; av[4 * g + 1] = v.y; av[4 * g + 2] = v.z; av[4 * g + 3] = v.w;
                    }
                }
#pragma unroll
                for (int g = 0; g < TN / 4; ++g) {
                    const int4 w = *reinterpret_cast<const int4*>(&sm.bw[buf][kk][g * 64 + tx * 4]);
                    bd[4 * g] = __hiloint2double(w.x, 0); bd[4 * g + 1] = __hiloint2double(w.y, 0);
                    bd[4 * g + 2] = __hiloint2double(w.z, 0); bd[4 * g + 3] = __hiloint2double(w.w, 0);
                    if (FULL) {
                        const int4 v = *reinterpret_cast<const int4*>(&sm.bh[buf][kk][g * 64 + tx * 4]);
                        bh[4 * g] = v.x; bh[4 * g + 1] = v.y; bh[4 * g + 2] = v.z; bh[4 * g + 3] = v.w;
                    }
                }
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) {
                        if (FULL) acc[i][j] = mad_lo_u(av[i], bh[j], acc[i][j]);
                        facc[i][j] = fma_rm(ad[i], bd[j], facc[i][j]);
                    }
            }
            __syncthreads();
        }

        // A run that covers the tile's whole K, with no other kernel adding to c meanwhile, owns its
        // outputs: plain 16-byte stores (FULL) or load-add-store (floor form).  Everything else adds
        // with red.global.add.  With a short K nearly every run is of the first kind, and the
        // scattered 4-byte atomics would otherwise cost several times the arithmetic.
        const bool owns = exclusive && s_begin == 0 && s_end == k_steps;
        const bool c_vec = (n % 4 == 0) && (reinterpret_cast<uintptr_t>(c) % 16 == 0);
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int r = row0 + (i / 4) * 64 + ty * 4 + (i % 4);
            if (r >= m) continue;
#pragma unroll
            for (int g = 0; g < TN / 4; ++g) {
                const int cc = col0 + g * 64 + tx * 4;
                uint32_t part[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    part[j] = (uint32_t)__double2loint(facc[i][4 * g + j]) + (FULL ? acc[i][4 * g + j] : 0u);
                unsigned int* dst = reinterpret_cast<unsigned int*>(c) + (size_t)r * n + cc;
                if (owns && c_vec && cc + 3 < n) {
                    uint4 o = make_uint4(part[0], part[1], part[2], part[3]);
                    if (!FULL) {
                        const uint4 old = *reinterpret_cast<const uint4*>(dst);
                        o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                    }
                    *reinterpret_cast<uint4*>(dst) = o;
                } else if (owns) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (cc + j < n) dst[j] = FULL ? part[j] : dst[j] + part[j];
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (cc + j < n) atomicAdd(dst + j, part[j]);
                }
            }
        }
    }
}

template <int BN, bool FULL>
int64_t launch_q16_streamk(DeviceCtx* ctx, const int32_t* a, const int32_t* b, int32_t* c, int64_t m, int64_t k,
                           int64_t n, int max_blocks, bool exclusive) {
    if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff)
        return fail(MIND_B200_ERR_TOO_LARGE, "GEMM dimension above 2^31-1");
    constexpr int SMEM = (int)sizeof(Q16Smem<BN, FULL>);
    static thread_local int attr_dev = -1;
    if (attr_dev != ctx->device) {
        MB200_CUDA(cudaFuncSetAttribute(gemm_q16_fp64_kernel<BN, FULL>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        attr_dev = ctx->device;
    }
    const int64_t m_tiles = (m + QBM - 1) / QBM, n_tiles = (n + BN - 1) / BN;
    if (m_tiles * n_tiles > 0x7fffffff) return fail(MIND_B200_ERR_TOO_LARGE, "too many output tiles");
    if (FULL) MB200_CUDA(cudaMemsetAsync(c, 0, (size_t)m * n * 4, ctx->stream));
    constexpr int64_t K_SLICE = 1 << 20;
    for (int64_t k0 = 0; k0 < k; k0 += K_SLICE) {
        const int64_t kc = k - k0 < K_SLICE ? k - k0 : K_SLICE;
        const int64_t k_steps = (kc + QBK - 1) / QBK, units = m_tiles * n_tiles * k_steps;
        const int64_t cap = max_blocks > 0 && max_blocks < ctx->sm_count ? max_blocks : ctx->sm_count;
        const unsigned grid = (unsigned)(units < cap ? units : cap);
        prof_begin(ctx);
        gemm_q16_fp64_kernel<BN, FULL><<<grid, QTHREADS, SMEM, ctx->stream>>>(
            a + k0, b + k0 * n, c, (int)m, (int)kc, (int)n, (int)k, (int)n_tiles, (int)k_steps, (long long)units,
            (exclusive && (FULL ? k0 == 0 : true)) ? 1 : 0);
        prof_end(ctx);
        count_launch();
        const int64_t rc = check_launch("gemm_q16_fp64_kernel");
        if (rc) return rc;
    }
    return 0;
}

}  // namespace

bool gemm_q16_fp64_usable(const int32_t* a, const int32_t* b, int64_t k, int64_t n) {
    return k % 4 == 0 && n % 4 == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0 &&
           reinterpret_cast<uintptr_t>(b) % 16 == 0;
}

// c = the whole product (c is zeroed here, then added to)
int64_t launch_gemm_q16_fp64(DeviceCtx* ctx, const int32_t* a, const int32_t* b, int32_t* c, int64_t m,
                             int64_t k, int64_t n) {
    return launch_q16_streamk<64, true>(ctx, a, b, c, m, k, n, 0, true);
}

// c += the floor half (c holds the linear half, or the linear half is being added beside this
// kernel); max_blocks > 0 leaves the other SMs to that kernel
int64_t launch_gemm_q16_floor_add(DeviceCtx* ctx, const int32_t* a, const int32_t* b, int32_t* c, int64_t m,
                                  int64_t k, int64_t n, int max_blocks) {
    // with max_blocks > 0 the tensor-core kernel adds onto c at the same time: atomics only
    return launch_q16_streamk<128, false>(ctx, a, b, c, m, k, n, max_blocks, max_blocks <= 0);
}

}  // namespace mb200
