// Q16.16 GEMM with the per-product floor on the FP64 pipe (alone, or as the floor half of the
// tensor-core hybrid: see HYBRID below).
//
//   C[i,j] = (i32) sum_k ((i64)A[i,k] * (i64)B[k,j]) >> 16        (shift per product)
//
// With bl = (int16)b and bh = (b - bl) >> 16:  (a*b) >> 16 = a*bh + floor(a*bl / 65536).
// The all-integer kernel (gemm_simt.cu) spends a mad.lo and a mad.hi per product and is
// bound by the 32-bit integer multiplier (measured: ~11 Top/s at 4096^3 with every tile size;
// this kernel: ~15 Top/s).  Here
// the floor term moves to the FP64 pipe:
//     |a * bl| < 2^47, so a * (bl * 2^-16) is exact in binary64, and
//     fma.rm.f64(a, bl * 2^-16, t) = t + floor(a*bl / 65536)  exactly
// whenever t is an integer-valued binary64 in [2^52, 2^53) (one rounding, toward minus
// infinity, at unit weight).  Starting from t = 1.5 * 2^52 the chain of fused multiply-adds
// therefore accumulates sum_k floor(a*bl / 65536) exactly for 2^21 products (each term is
// below 2^30 in magnitude), and the low mantissa word of t is that sum mod 2^32.  Per
// product: one mad.lo.s32 (integer multiplier) and one fma.rm.f64 (FP64 pipe), two
// independent accumulators per output, folded every 4096 steps of K - bit-identical to the
// integer form.
//
// Tiling as in gemm_simt.cu: 256 threads, BM x BN outputs per block, BK = 16, 8 x (BN/16)
// outputs per thread.  B goes to shared memory as bh (int32) and bl * 2^-16 (binary64, laid
// out so that a thread's 16-byte reads are contiguous across the warp); A as int32 and as
// binary64 (converted once per element on its way to shared memory: converting in the inner
// loop made the conversion unit the bottleneck).  Needs 16-byte aligned operands with K % 4 == 0 and N % 4 == 0;
// other calls use the integer kernel.
#include "common.h"

namespace mb200 {
namespace {

constexpr int QBK = 16;
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
__device__ __forceinline__ int32_t q16_hi_part(int32_t b) { return (b >> 16) + ((b >> 15) & 1); }
template <bool UNSIGNED_LOW>
__device__ __forceinline__ double q16_lo_scaled(int32_t b) {  // exact: a power-of-two scale
    return UNSIGNED_LOW ? (double)(b & 0xffff) * (1.0 / 65536.0)
                        : (double)(int32_t)(int16_t)(b & 0xffff) * (1.0 / 65536.0);
}

// HYBRID: only the floor term sum_k floor(a * (b & 0xffff) / 65536) is computed here (with the
// UNSIGNED low half, so that b >> 16 is the matching high part) and added onto the linear part
// sum_k a * (b >> 16), which the tensor cores have already written to c.
template <int BM, int BN, bool HYBRID>
__global__ void __launch_bounds__(QTHREADS)
gemm_q16_fp64_kernel(const int32_t* __restrict__ a, const int32_t* __restrict__ b, int32_t* __restrict__ c,
                     int m, int k, int n) {
    constexpr int TM = BM / 16, TN = BN / 16;
    static_assert(TM % 4 == 0 && TN % 4 == 0, "register tile is built from 4-wide groups");
    __shared__ __align__(16) int32_t As[HYBRID ? 1 : QBK][BM + 4];
    __shared__ __align__(16) double Ad[QBK][BM + 2];  // A as binary64: converted once per element
    __shared__ __align__(16) int32_t Bh[HYBRID ? 1 : QBK][BN];
    __shared__ __align__(16) double2 Bd[QBK][BN / 2];  // [kk][(group * 2 + half) * 16 + tx]

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
    constexpr int A_VEC = BM * QBK / 4 / QTHREADS;  // 16-byte vectors per thread
    constexpr int B_VEC = BN * QBK / 4 / QTHREADS;
    int4 ra[A_VEC], rb[B_VEC];

    auto load_tiles = [&](int k0) {
#pragma unroll
        for (int i = 0; i < A_VEC; ++i) {
            const int r = (tid >> 2) + 64 * i, kk = k0 + (tid & 3) * 4;
            ra[i] = make_int4(0, 0, 0, 0);
            if (row0 + r < m && kk < k) ra[i] = *reinterpret_cast<const int4*>(a + (size_t)(row0 + r) * k + kk);
        }
#pragma unroll
        for (int i = 0; i < B_VEC; ++i) {
            const int e = tid + QTHREADS * i;
            const int kk = k0 + e / (BN / 4), cc = (e % (BN / 4)) * 4;
            rb[i] = make_int4(0, 0, 0, 0);
            if (kk < k && col0 + cc < n) rb[i] = *reinterpret_cast<const int4*>(b + (size_t)kk * n + col0 + cc);
        }
    };
    auto store_tiles = [&]() {
#pragma unroll
        for (int i = 0; i < A_VEC; ++i) {
            const int r = (tid >> 2) + 64 * i, kq = (tid & 3) * 4;
            if (!HYBRID) {
                As[kq][r] = ra[i].x; As[kq + 1][r] = ra[i].y; As[kq + 2][r] = ra[i].z; As[kq + 3][r] = ra[i].w;
            }
            Ad[kq][r] = __int2double_rn(ra[i].x); Ad[kq + 1][r] = __int2double_rn(ra[i].y);
            Ad[kq + 2][r] = __int2double_rn(ra[i].z); Ad[kq + 3][r] = __int2double_rn(ra[i].w);
        }
#pragma unroll
        for (int i = 0; i < B_VEC; ++i) {
            const int e = tid + QTHREADS * i;
            const int kq = e / (BN / 4), cc = (e % (BN / 4)) * 4;
            if (!HYBRID)
                *reinterpret_cast<int4*>(&Bh[kq][cc]) = make_int4(q16_hi_part(rb[i].x), q16_hi_part(rb[i].y),
                                                                   q16_hi_part(rb[i].z), q16_hi_part(rb[i].w));
            const int g = cc / 64, t = (cc % 64) / 4;
            Bd[kq][(g * 2) * 16 + t] =
                make_double2(q16_lo_scaled<HYBRID>(rb[i].x), q16_lo_scaled<HYBRID>(rb[i].y));
            Bd[kq][(g * 2 + 1) * 16 + t] =
                make_double2(q16_lo_scaled<HYBRID>(rb[i].z), q16_lo_scaled<HYBRID>(rb[i].w));
        }
    };

    const double MAGIC = 6755399441055744.0;  // 1.5 * 2^52: unit weight in the last place
    uint32_t acc[TM][TN];
    double facc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            acc[i][j] = 0u;
            facc[i][j] = MAGIC;
        }

    load_tiles(0);
    for (int k0 = 0; k0 < k; k0 += QBK) {
        if ((k0 & 4095) == 0 && k0 != 0) {  // fold the floor sums long before they leave [2^52, 2^53)
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    acc[i][j] += (uint32_t)__double2loint(facc[i][j]);
                    facc[i][j] = MAGIC;
                }
        }
        __syncthreads();
        store_tiles();
        __syncthreads();
        if (k0 + QBK < k) load_tiles(k0 + QBK);
#pragma unroll
        for (int kk = 0; kk < QBK; ++kk) {
            int32_t av[TM], bh[TN];
            double ad[TM], bd[TN];
            if (!HYBRID) {
#pragma unroll
                for (int g = 0; g < TM / 4; ++g) {
                    const int4 v = *reinterpret_cast<const int4*>(&As[kk][g * 64 + ty * 4]);
                    av[4 * g] = v.x; av[4 * g + 1] = v.y; av[4 * g + 2] = v.z; av[4 * g + 3] = v.w;
                }
            }
#pragma unroll
            for (int g = 0; g < TM / 4; ++g) {
                const double2 d0 = *reinterpret_cast<const double2*>(&Ad[kk][g * 64 + ty * 4]);
                const double2 d1 = *reinterpret_cast<const double2*>(&Ad[kk][g * 64 + ty * 4 + 2]);
                ad[4 * g] = d0.x; ad[4 * g + 1] = d0.y; ad[4 * g + 2] = d1.x; ad[4 * g + 3] = d1.y;
            }
#pragma unroll
            for (int g = 0; g < TN / 4; ++g) {
                if (!HYBRID) {
                    const int4 v = *reinterpret_cast<const int4*>(&Bh[kk][g * 64 + tx * 4]);
                    bh[4 * g] = v.x; bh[4 * g + 1] = v.y; bh[4 * g + 2] = v.z; bh[4 * g + 3] = v.w;
                }
                const double2 d0 = Bd[kk][(g * 2) * 16 + tx], d1 = Bd[kk][(g * 2 + 1) * 16 + tx];
                bd[4 * g] = d0.x; bd[4 * g + 1] = d0.y; bd[4 * g + 2] = d1.x; bd[4 * g + 3] = d1.y;
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    if (!HYBRID) acc[i][j] = mad_lo_u(av[i], bh[j], acc[i][j]);
                    facc[i][j] = fma_rm(ad[i], bd[j], facc[i][j]);
                }
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] += (uint32_t)__double2loint(facc[i][j]);

    const bool c_vec = (n % 4 == 0) && (reinterpret_cast<uintptr_t>(c) % 16 == 0);
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = row0 + (i / 4) * 64 + ty * 4 + (i % 4);
        if (r >= m) continue;
#pragma unroll
        for (int g = 0; g < TN / 4; ++g) {
            const int cc = col0 + g * 64 + tx * 4;
            int32_t* dst = c + (size_t)r * n + cc;
            if (c_vec && cc + 3 < n) {
                uint4 o = make_uint4(acc[i][4 * g], acc[i][4 * g + 1], acc[i][4 * g + 2], acc[i][4 * g + 3]);
                if (HYBRID) {
                    const uint4 lin = *reinterpret_cast<const uint4*>(dst);
                    o.x += lin.x; o.y += lin.y; o.z += lin.z; o.w += lin.w;
                }
                *reinterpret_cast<uint4*>(dst) = o;
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (cc + j < n) dst[j] = (int32_t)(acc[i][4 * g + j] + (HYBRID ? (uint32_t)dst[j] : 0u));
            }
        }
    }
}

template <int BM, int BN, bool HYBRID>
int64_t launch_fp64_cfg(DeviceCtx* ctx, const int32_t* a, const int32_t* b, int32_t* c, int64_t m,
                        int64_t k, int64_t n) {
    dim3 grid((unsigned)((n + BN - 1) / BN), (unsigned)((m + BM - 1) / BM));
    if (grid.y > 65535) return fail(MIND_B200_ERR_TOO_LARGE, "M too large for the CUDA-core GEMM grid");
    prof_begin(ctx);
    gemm_q16_fp64_kernel<BM, BN, HYBRID><<<grid, QTHREADS, 0, ctx->stream>>>(a, b, c, (int)m, (int)k, (int)n);
    prof_end(ctx);
    count_launch();
    return check_launch("gemm_q16_fp64_kernel");
}

}  // namespace

bool gemm_q16_fp64_usable(const int32_t* a, const int32_t* b, int64_t k, int64_t n) {
    return k % 4 == 0 && n % 4 == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0 &&
           reinterpret_cast<uintptr_t>(b) % 16 == 0;
}

int64_t launch_gemm_q16_fp64(DeviceCtx* ctx, const int32_t* a, const int32_t* b, int32_t* c, int64_t m,
                             int64_t k, int64_t n) {
    if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff)
        return fail(MIND_B200_ERR_TOO_LARGE, "GEMM dimension above 2^31-1");
    const int64_t sms = ctx->sm_count;
    auto tiles = [&](int bm, int bn) { return ((m + bm - 1) / bm) * ((n + bn - 1) / bn); };
    // 8 x 4 outputs per thread is the largest register tile that holds both accumulator sets.
    if (tiles(128, 64) >= (sms * 3) / 4) return launch_fp64_cfg<128, 64, false>(ctx, a, b, c, m, k, n);
    return launch_fp64_cfg<64, 64, false>(ctx, a, b, c, m, k, n);
}

int64_t launch_gemm_q16_floor_add(DeviceCtx* ctx, const int32_t* a, const int32_t* b, int32_t* c, int64_t m,
                                  int64_t k, int64_t n) {
    const int64_t sms = ctx->sm_count;
    auto tiles = [&](int bm, int bn) { return ((m + bm - 1) / bm) * ((n + bn - 1) / bn); };
    if (tiles(128, 64) >= (sms * 3) / 4) return launch_fp64_cfg<128, 64, true>(ctx, a, b, c, m, k, n);
    return launch_fp64_cfg<64, 64, true>(ctx, a, b, c, m, k, n);
}

}  // namespace mb200
