// CUDA-core GEMMs.
//
// Q16.16 (the product path):  C[i,j] = (i32) sum_k ((i64)A[i,k] * (i64)B[k,j]) >> 16.
// The shift is applied to every product before the add, so the sum is not bilinear
// and cannot go through the tensor cores.  With bl = (int16)b (signed low half) and
// bh = (b - bl) >> 16, b = 65536*bh + bl exactly, hence
//     (a*b) >> 16  ==  a*bh + floor(a*bl / 65536)  ==  a*bh + mulhi_s32(a, bl << 16),
// and since only the low 32 bits of the sum are kept, each product costs two 32-bit
// multiply-adds (mad.lo.s32, mad.hi.s32) into one 32-bit accumulator.  B is split into
// the two planes (bh, bl << 16 == b << 16) once per tile on its way to shared memory.
//
// int8 / int16 (cross-check path): the same tiling with a single plane and one mad.lo
// per product; kept as an independent on-device check of the tensor-core kernels.
//
// Tiling: BM x BN outputs per 256-thread block, BK = 16 per step, (BM/16) x (BN/16)
// outputs per thread held in registers, operands staged in shared memory with the next
// step's global loads in flight during the current step's arithmetic.
#include "common.h"

namespace mb200 {
namespace {

constexpr int BK = 16;
constexpr int SIMT_THREADS = 256;

__device__ __forceinline__ uint32_t mad_lo(int32_t a, int32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.lo.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// c + high 32 bits of the 64-bit product a*b.  (A widening multiply followed by an add of
// the high word was measured 5 % slower than the fused form.)
__device__ __forceinline__ uint32_t mad_hi(int32_t a, int32_t b, uint32_t c) {
#ifndef MB200_Q16_MULWIDE
    uint32_t d;
    asm("mad.hi.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
#else
    uint32_t d;
    asm("{\n\t.reg .b64 p;\n\t.reg .b32 lo, hi;\n\t"
        "mul.wide.s32 p, %1, %2;\n\t"
        "mov.b64 {lo, hi}, p;\n\t"
        "add.s32 %0, hi, %3;\n\t}"
        : "=r"(d)
        : "r"(a), "r"(b), "r"(c));
    return d;
#endif
}
// bh of the split b = 65536*bh + (int16)b, without overflow for any b.
__device__ __forceinline__ int32_t q16_hi(int32_t b) { return (b >> 16) + ((b >> 15) & 1); }

template <typename T, bool Q16, int BM, int BN, bool VEC>
__global__ void __launch_bounds__(SIMT_THREADS)
gemm_simt_kernel(const T* __restrict__ a, const T* __restrict__ b, int32_t* __restrict__ c, int m,
                 int k, int n, int c_vec) {
    constexpr int TM = BM / 16, TN = BN / 16;
    static_assert(TM % 4 == 0 && TN % 4 == 0, "register tile is built from 4-wide groups");
    constexpr int NPL = Q16 ? 2 : 1;
    __shared__ __align__(16) int32_t As[BK][BM + 4];
    __shared__ __align__(16) int32_t Bs[NPL][BK][BN];

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;

    // global -> register staging
    constexpr int A_PER = BM * BK / SIMT_THREADS;  // elements per thread
    constexpr int B_PER = BN * BK / SIMT_THREADS;
    int32_t ra[A_PER], rb[B_PER];

    auto load_tiles = [&](int k0) {
        if (VEC) {
            // A: rows of 16 = 4 vectors; thread -> (row = tid/4 + 64*i, kvec = tid%4)
#pragma unroll
            for (int i = 0; i < A_PER / 4; ++i) {
                const int r = (tid >> 2) + 64 * i, kk = k0 + (tid & 3) * 4;
                int4 v = make_int4(0, 0, 0, 0);
                if (row0 + r < m && kk < k)  // k % 4 == 0 on this path
                    v = *reinterpret_cast<const int4*>(a + (size_t)(row0 + r) * k + kk);
                ra[4 * i] = v.x; ra[4 * i + 1] = v.y; ra[4 * i + 2] = v.z; ra[4 * i + 3] = v.w;
            }
            // B: rows of BN = BN/4 vectors
#pragma unroll
            for (int i = 0; i < B_PER / 4; ++i) {
                const int e = tid + SIMT_THREADS * i;
                const int kk = k0 + e / (BN / 4), cc = (e % (BN / 4)) * 4;
                int4 v = make_int4(0, 0, 0, 0);
                if (kk < k && col0 + cc < n)  // n % 4 == 0 on this path
                    v = *reinterpret_cast<const int4*>(b + (size_t)kk * n + col0 + cc);
                rb[4 * i] = v.x; rb[4 * i + 1] = v.y; rb[4 * i + 2] = v.z; rb[4 * i + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < A_PER; ++i) {
                const int e = tid + SIMT_THREADS * i;
                const int r = e / BK, kk = k0 + e % BK;
                ra[i] = (row0 + r < m && kk < k) ? (int32_t)a[(size_t)(row0 + r) * k + kk] : 0;
            }
#pragma unroll
            for (int i = 0; i < B_PER; ++i) {
                const int e = tid + SIMT_THREADS * i;
                const int kk = k0 + e / BN, cc = e % BN;
                rb[i] = (kk < k && col0 + cc < n) ? (int32_t)b[(size_t)kk * n + col0 + cc] : 0;
            }
        }
    };
    auto store_tiles = [&]() {
        if (VEC) {
#pragma unroll
            for (int i = 0; i < A_PER / 4; ++i) {
                const int r = (tid >> 2) + 64 * i, kq = (tid & 3) * 4;
#pragma unroll
                for (int j = 0; j < 4; ++j) As[kq + j][r] = ra[4 * i + j];
            }
#pragma unroll
            for (int i = 0; i < B_PER / 4; ++i) {
                const int e = tid + SIMT_THREADS * i;
                const int kq = e / (BN / 4), cc = (e % (BN / 4)) * 4;
                if (Q16) {
                    *reinterpret_cast<int4*>(&Bs[0][kq][cc]) = make_int4(
                        q16_hi(rb[4 * i]), q16_hi(rb[4 * i + 1]), q16_hi(rb[4 * i + 2]), q16_hi(rb[4 * i + 3]));
                    *reinterpret_cast<int4*>(&Bs[NPL - 1][kq][cc]) = make_int4(
                        rb[4 * i] << 16, rb[4 * i + 1] << 16, rb[4 * i + 2] << 16, rb[4 * i + 3] << 16);
                } else {
                    *reinterpret_cast<int4*>(&Bs[0][kq][cc]) =
                        make_int4(rb[4 * i], rb[4 * i + 1], rb[4 * i + 2], rb[4 * i + 3]);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < A_PER; ++i) {
                const int e = tid + SIMT_THREADS * i;
                As[e % BK][e / BK] = ra[i];
            }
#pragma unroll
            for (int i = 0; i < B_PER; ++i) {
                const int e = tid + SIMT_THREADS * i;
                if (Q16) {
                    Bs[0][e / BN][e % BN] = q16_hi(rb[i]);
                    Bs[NPL - 1][e / BN][e % BN] = (int32_t)((uint32_t)rb[i] << 16);
                } else {
                    Bs[0][e / BN][e % BN] = rb[i];
                }
            }
        }
    };

    uint32_t acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0u;

    load_tiles(0);
    for (int k0 = 0; k0 < k; k0 += BK) {
        __syncthreads();  // previous step's readers are done with shared memory
        store_tiles();
        __syncthreads();
        if (k0 + BK < k) load_tiles(k0 + BK);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            int32_t av[TM], bh[TN], bl[TN];
#pragma unroll
            for (int g = 0; g < TM / 4; ++g) {
                const int4 v = *reinterpret_cast<const int4*>(&As[kk][g * 64 + ty * 4]);
                av[4 * g] = v.x; av[4 * g + 1] = v.y; av[4 * g + 2] = v.z; av[4 * g + 3] = v.w;
            }
#pragma unroll
            for (int g = 0; g < TN / 4; ++g) {
                const int4 v = *reinterpret_cast<const int4*>(&Bs[0][kk][g * 64 + tx * 4]);
                bh[4 * g] = v.x; bh[4 * g + 1] = v.y; bh[4 * g + 2] = v.z; bh[4 * g + 3] = v.w;
                if (Q16) {
                    const int4 w = *reinterpret_cast<const int4*>(&Bs[NPL - 1][kk][g * 64 + tx * 4]);
                    bl[4 * g] = w.x; bl[4 * g + 1] = w.y; bl[4 * g + 2] = w.z; bl[4 * g + 3] = w.w;
                }
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    acc[i][j] = mad_lo(av[i], bh[j], acc[i][j]);
                    if (Q16) acc[i][j] = mad_hi(av[i], bl[j], acc[i][j]);
                }
        }
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = row0 + (i / 4) * 64 + ty * 4 + (i % 4);
        if (r >= m) continue;
#pragma unroll
        for (int g = 0; g < TN / 4; ++g) {
            const int cc = col0 + g * 64 + tx * 4;
            int32_t* dst = c + (size_t)r * n + cc;
            if (c_vec && cc + 3 < n) {
                *reinterpret_cast<uint4*>(dst) =
                    make_uint4(acc[i][4 * g], acc[i][4 * g + 1], acc[i][4 * g + 2], acc[i][4 * g + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (cc + j < n) dst[j] = (int32_t)acc[i][4 * g + j];
            }
        }
    }
}

template <typename T, bool Q16, int BM, int BN>
int64_t launch_cfg(DeviceCtx* ctx, const T* a, const T* b, int32_t* c, int64_t m, int64_t k,
                   int64_t n) {
    dim3 grid((unsigned)((n + BN - 1) / BN), (unsigned)((m + BM - 1) / BM));
    if (grid.y > 65535) return fail(MIND_B200_ERR_TOO_LARGE, "M too large for the CUDA-core GEMM grid");
    const int c_vec = (n % 4 == 0) && (reinterpret_cast<uintptr_t>(c) % 16 == 0);
    const bool vec = sizeof(T) == 4 && k % 4 == 0 && n % 4 == 0 &&
                     reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(b) % 16 == 0;
    prof_begin(ctx);
    if (vec)
        gemm_simt_kernel<T, Q16, BM, BN, true>
            <<<grid, SIMT_THREADS, 0, ctx->stream>>>(a, b, c, (int)m, (int)k, (int)n, c_vec);
    else
        gemm_simt_kernel<T, Q16, BM, BN, false>
            <<<grid, SIMT_THREADS, 0, ctx->stream>>>(a, b, c, (int)m, (int)k, (int)n, c_vec);
    prof_end(ctx);
    count_launch();
    return check_launch("gemm_simt_kernel");
}

template <typename T, bool Q16>
int64_t launch_simt(DeviceCtx* ctx, const T* a, const T* b, int32_t* c, int64_t m, int64_t k,
                    int64_t n) {
    if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff)
        return fail(MIND_B200_ERR_TOO_LARGE, "GEMM dimension above 2^31-1");
    // Largest tile that still gives every SM a block; small problems take the small tile.
    const int64_t sms = ctx->sm_count;
    auto tiles = [&](int bm, int bn) { return ((m + bm - 1) / bm) * ((n + bn - 1) / bn); };
    if (tiles(128, 128) >= sms) return launch_cfg<T, Q16, 128, 128>(ctx, a, b, c, m, k, n);
    if (tiles(128, 64) >= (sms * 3) / 4) return launch_cfg<T, Q16, 128, 64>(ctx, a, b, c, m, k, n);
    return launch_cfg<T, Q16, 64, 64>(ctx, a, b, c, m, k, n);
}

}  // namespace

int64_t launch_gemm_q16(DeviceCtx* ctx, const int32_t* a, const int32_t* b, int32_t* c, int64_t m,
                        int64_t k, int64_t n) {
    return launch_simt<int32_t, true>(ctx, a, b, c, m, k, n);
}
int64_t launch_gemm_i8_simt(DeviceCtx* ctx, const int8_t* a, const int8_t* b, int32_t* c, int64_t m,
                            int64_t k, int64_t n) {
    return launch_simt<int8_t, false>(ctx, a, b, c, m, k, n);
}
int64_t launch_gemm_i16_simt(DeviceCtx* ctx, const int16_t* a, const int16_t* b, int32_t* c,
                             int64_t m, int64_t k, int64_t n) {
    return launch_simt<int16_t, false>(ctx, a, b, c, m, k, n);
}

}  // namespace mb200
