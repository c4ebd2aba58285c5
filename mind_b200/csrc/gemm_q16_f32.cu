// Q16.16 GEMM: the one term that no linear kernel can form, on the FP32 pipe.
//
//   C[i,j] = (i32) sum_k ((i64)A[i,k] * (i64)B[k,j]) >> 16        (shift per product)
//
// With a = 65536 * ah + al and b = 65536 * bh + bl (al, bl the unsigned low halves, ah, bh the
// arithmetic high halves):
//     (a * b) >> 16 = a * bh + ah * bl + floor(al * bl / 65536).
// The first two terms are plain integer products: the tensor cores form them mod 2^32 from byte
// planes (gemm_tc.cu).  The last one has a rounding per product.  al * bl < 2^32, so al and
// bl * 2^-16 are exact binary32 values and their product is exact inside an FMA; with t an
// integer-valued binary32 in [2^23, 2^24) (unit weight in the last place),
//     fma.rm.f32(al, bl * 2^-16, t) = t + floor(al * bl / 65536)      exactly
// as long as the result stays below 2^24.  Every term is at most 65534, so a chain started at
// 2^23 holds 128 products; then its mantissa is added to an integer register and the chain starts
// again.  The FP32 pipe issues twice the FMAs of the FP64 pipe, and as the packed form
// fma.rm.f32x2 (two chains per instruction) it leaves half of the issue slots to the loads.
//
// Register tile 8 x 8 per thread (32 packed chains along N + 64 integer sums), 128 x 128 per block
// of 256 threads.  Shared memory holds al and bl * 2^-16 as binary32, converted once per element
// on the way in (or-ing the value into the mantissa of 2^23: no integer-to-float unit involved);
// the packed FMA wants the A operand in both halves of a register pair, which two moves make
// (measured against keeping (al, al) pairs in shared memory, and against pairing rows and
// swapping the B pair instead: 4 % and 1 % slower).  The fragments of K step kk + 1 are read from
// shared memory while step kk is multiplied (7 % faster than leaving the order to the compiler).
//
// Work is dealt out stream-K fashion, as in the FP64 kernel (gemm_q16.cu): units are (output tile,
// 16-deep K step) pairs in tile-major order, block b takes units [b * U / G, (b + 1) * U / G), and
// each run of units inside one tile ends by adding onto c, which already holds (or is being
// given, by the tensor-core kernel running beside this one) the linear terms.
#include "common.h"

namespace mb200 {
namespace {

constexpr int FBM = 128, FBN = 128, FBK = 16;
constexpr int FTHREADS = 256;
constexpr int FLUSH_STEPS = 128 / FBK;  // K steps one chain may run before it is emptied

__device__ __forceinline__ uint64_t fma2_rm(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rm.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

constexpr uint32_t TWO23_BITS = Q16_TWO23_BITS;
constexpr uint64_t CHAIN_START = ((uint64_t)TWO23_BITS << 32) | TWO23_BITS;

struct F32Smem {
    float ad[2][FBK][FBM + 4];  // al
    float bf[2][FBK][FBN];      // bl * 2^-16
};

__global__ void __launch_bounds__(FTHREADS, 1)
gemm_q16_f32_kernel(const int32_t* __restrict__ a, const int32_t* __restrict__ b, int32_t* __restrict__ c, int m,
                    int k, int n, int lda, int n_tiles, int k_steps, long long units, int exclusive) {
    extern __shared__ __align__(16) unsigned char q16f_smem[];
    F32Smem& sm = *reinterpret_cast<F32Smem*>(q16f_smem);

    // 16 x 16 threads; a warp is 8 (x) by 4 (y) of them, and every four consecutive lanes are 2 x 2.
    // A 16-byte shared load is served half a warp at a time, and in one pass only if no four
    // consecutive lanes ask for more than two different 16-byte groups (measured on B200: two
    // wavefronts per load with this lane order, four with lanes laid out row by row).  Here the
    // 16 lanes of a half read 128 contiguous bytes of B and two neighbouring groups of A.
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int lx = (lane & 1) | ((lane >> 1) & 6), ly = ((lane >> 1) & 1) | ((lane >> 3) & 2);
    const int tx = (warp & 1) * 8 + lx, ty = (warp >> 1) * 4 + ly;
    constexpr int A_VEC = FBM * FBK / 4 / FTHREADS;  // 16-byte vectors per thread
    constexpr int B_VEC = FBN * FBK / 4 / FTHREADS;
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
            const int e = tid + FTHREADS * i;
            const int kk = k0 + e / (FBN / 4), cc = (e % (FBN / 4)) * 4;
            rb[i] = make_int4(0, 0, 0, 0);
            if (kk < k && col0 + cc < n) rb[i] = *reinterpret_cast<const int4*>(b + (size_t)kk * n + col0 + cc);
        }
    };
    auto store_tiles = [&](int buf) {
#pragma unroll
        for (int i = 0; i < A_VEC; ++i) {
            const int r = (tid >> 2) + 64 * i, kq = (tid & 3) * 4;
            const float x = q16_low_half_f32(ra[i].x), y = q16_low_half_f32(ra[i].y), z = q16_low_half_f32(ra[i].z),
                        w = q16_low_half_f32(ra[i].w);
            sm.ad[buf][kq][r] = x;
            sm.ad[buf][kq + 1][r] = y;
            sm.ad[buf][kq + 2][r] = z;
            sm.ad[buf][kq + 3][r] = w;
        }
#pragma unroll
        for (int i = 0; i < B_VEC; ++i) {
            const int e = tid + FTHREADS * i;
            const int kq = e / (FBN / 4), cc = (e % (FBN / 4)) * 4;
            *reinterpret_cast<float4*>(&sm.bf[buf][kq][cc]) =
                make_float4(q16_low_half_scaled_f32(rb[i].x), q16_low_half_scaled_f32(rb[i].y), q16_low_half_scaled_f32(rb[i].z),
                            q16_low_half_scaled_f32(rb[i].w));
        }
    };

    const long long u_end = units * (blockIdx.x + 1) / gridDim.x;
    long long u = units * blockIdx.x / gridDim.x;
    while (u < u_end) {
        // one run: the units of this block that lie in one output tile
        const int tile = (int)(u / k_steps), s_begin = (int)(u % k_steps);
        const long long left = u_end - u;
        const int s_end = left < (long long)(k_steps - s_begin) ? s_begin + (int)left : k_steps;
        u += s_end - s_begin;
        row0 = (tile / n_tiles) * FBM;
        col0 = (tile % n_tiles) * FBN;

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

        __syncthreads();  // the previous run's last reads of buffer 0
        load_tiles(s_begin * FBK);
        store_tiles(0);
        if (s_begin + 1 < s_end) load_tiles((s_begin + 1) * FBK);
        __syncthreads();
        for (int s = s_begin; s < s_end; ++s) {
            const int buf = (s - s_begin) & 1;
            if (s + 1 < s_end) {
                store_tiles(buf ^ 1);  // read last in step s - 1, which every warp has left
                if (s + 2 < s_end) load_tiles((s + 2) * FBK);
            }
            // fragments of step kk + 1 are fetched while those of step kk are multiplied
            uint4 fa[2][2], fb[2][2];
            auto fetch = [&](int kk, int slot) {
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    fa[slot][g] = *reinterpret_cast<const uint4*>(&sm.ad[buf][kk][g * 64 + ty * 4]);
                    fb[slot][g] = *reinterpret_cast<const uint4*>(&sm.bf[buf][kk][g * 64 + tx * 4]);
                }
            };
            fetch(0, 0);
#pragma unroll
            for (int kk = 0; kk < FBK; ++kk) {
                if (kk + 1 < FBK) fetch(kk + 1, (kk + 1) & 1);
                uint64_t a2[8], b2[4];
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const uint4 v = fa[kk & 1][g], w = fb[kk & 1][g];
                    a2[4 * g] = ((uint64_t)v.x << 32) | v.x; a2[4 * g + 1] = ((uint64_t)v.y << 32) | v.y;
                    a2[4 * g + 2] = ((uint64_t)v.z << 32) | v.z; a2[4 * g + 3] = ((uint64_t)v.w << 32) | v.w;
                    b2[2 * g] = ((uint64_t)w.y << 32) | w.x; b2[2 * g + 1] = ((uint64_t)w.w << 32) | w.z;
                }
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int jp = 0; jp < 4; ++jp) chain[i][jp] = fma2_rm(a2[i], b2[jp], chain[i][jp]);
            }
            if (((s - s_begin) % FLUSH_STEPS) == FLUSH_STEPS - 1) empty_chains();
            __syncthreads();
        }
        empty_chains();

        // A run that covers the tile's whole K, with no other kernel adding to c meanwhile, owns its
        // outputs: 16-byte load-add-store.  Everything else adds with red.global.add.
        const bool owns = exclusive && s_begin == 0 && s_end == k_steps;
        const bool c_vec = (n % 4 == 0) && (reinterpret_cast<uintptr_t>(c) % 16 == 0);
        const uint32_t bias = emptied * TWO23_BITS;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = row0 + (i / 4) * 64 + ty * 4 + (i % 4);
            if (r >= m) continue;
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                const int cc = col0 + g * 64 + tx * 4;
                uint32_t part[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) part[j] = sum[i][4 * g + j] - bias;
                unsigned int* dst = reinterpret_cast<unsigned int*>(c) + (size_t)r * n + cc;
                if (owns && c_vec && cc + 3 < n) {
                    const uint4 old = *reinterpret_cast<const uint4*>(dst);
                    *reinterpret_cast<uint4*>(dst) =
                        make_uint4(old.x + part[0], old.y + part[1], old.z + part[2], old.w + part[3]);
                } else if (owns) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (cc + j < n) dst[j] += part[j];
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (cc + j < n) atomicAdd(dst + j, part[j]);
                }
            }
        }
    }
}

}  // namespace

// c += sum_k floor((a & 0xffff) * (b & 0xffff) / 65536) mod 2^32.  c holds the linear terms, or they
// are being added beside this kernel (max_blocks > 0 leaves the other SMs to that kernel; then
// every output is added with red.global.add).  Same operand rules as gemm_q16_fp64_usable.
int64_t launch_gemm_q16_floor_f32(DeviceCtx* ctx, const int32_t* a, const int32_t* b, int32_t* c, int64_t m,
                                  int64_t k, int64_t n, int max_blocks) {
    if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff)
        return fail(MIND_B200_ERR_TOO_LARGE, "GEMM dimension above 2^31-1");
    const int64_t m_tiles = (m + FBM - 1) / FBM, n_tiles = (n + FBN - 1) / FBN;
    if (m_tiles * n_tiles > 0x7fffffff) return fail(MIND_B200_ERR_TOO_LARGE, "too many output tiles");
    const int64_t k_steps = (k + FBK - 1) / FBK, units = m_tiles * n_tiles * k_steps;
    const int64_t cap = max_blocks > 0 && max_blocks < ctx->sm_count ? max_blocks : ctx->sm_count;
    const unsigned grid = (unsigned)(units < cap ? units : cap);
    static thread_local int attr_dev = -1;
    constexpr int SMEM = (int)sizeof(F32Smem);
    if (attr_dev != ctx->device) {
        MB200_CUDA(cudaFuncSetAttribute(gemm_q16_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        attr_dev = ctx->device;
    }
    prof_begin(ctx);
    gemm_q16_f32_kernel<<<grid, FTHREADS, SMEM, ctx->stream>>>(a, b, c, (int)m, (int)k, (int)n, (int)k, (int)n_tiles,
                                                               (int)k_steps, (long long)units, max_blocks <= 0 ? 1 : 0);
    prof_end(ctx);
    count_launch();
    return check_launch("gemm_q16_f32_kernel");
}

}  // namespace mb200
