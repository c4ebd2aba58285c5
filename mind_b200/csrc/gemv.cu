// Memory-bound row reductions: Q16.16 / int16 matrix x vector, dots, L1 distance.
//
//   Q16.16:  y[r] = (i32) sum_c (W[r,c] * x[c]) >> 16   (shift per product, then add)
//   int16 :  y[r] = (i32) sum_c  W[r,c] * x[c]
//   L1    :  out  = (i32) sum_c |a[c] - b[c]|
// Only the low 32 bits of the exact sum are kept, so 32-bit wrap-around
// accumulation in any order gives the reference's bits.  The Q16.16 product uses the
// split x = 65536*xh + (int16)x:  (w*x) >> 16 == w*xh + mulhi_s32(w, x << 16).
//
// The matrix is streamed exactly once with 128-bit loads that bypass L1
// (ld.global.nc.L1::no_allocate), the vector comes through the read-only cache;
// one warp owns a row (several warps share a long row; a whole block takes it when there
// are few long rows), eight 128-bit loads per lane are in flight, and partial sums are
// combined with warp shuffles and shared memory.
#include "common.h"

namespace mb200 {
namespace {

enum { OP_Q16 = 0, OP_I16 = 1, OP_L1 = 2 };

__device__ __forceinline__ int4 ld_stream(const void* p) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t mad_lo(int32_t a, int32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.lo.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t mad_hi(int32_t a, int32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.hi.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int32_t q16_hi(int32_t b) { return (b >> 16) + ((b >> 15) & 1); }

template <int OP>
__device__ __forceinline__ uint32_t fma_word(uint32_t acc, int32_t w, int32_t x) {
    if (OP == OP_Q16) {
        acc = mad_lo(w, q16_hi(x), acc);
        return mad_hi(w, (int32_t)((uint32_t)x << 16), acc);
    } else if (OP == OP_I16) {  // two int16 per word
        acc = mad_lo((int32_t)((uint32_t)w << 16) >> 16, (int32_t)((uint32_t)x << 16) >> 16, acc);
        return mad_lo(w >> 16, x >> 16, acc);
    } else {
        return acc + (w >= x ? (uint32_t)w - (uint32_t)x : (uint32_t)x - (uint32_t)w);
    }
}
// int16 rows: x = 256 * xh + xl (xh signed, xl unsigned bytes), so w . x = 256 * (w . xh) + w . xl,
// and dp2a multiplies two packed int16 of w by two bytes at once: eight dp2a and four byte
// permutes per eight elements, with no sign extension of w (the shift-and-multiply form left
// the kernel at 0.70 of the copy bandwidth).  lo collects w . xl, hi collects w . xh.
__device__ __forceinline__ void dp2a_word_pair(uint32_t& lo, uint32_t& hi, int32_t w0, int32_t w1, uint32_t xl,
                                               uint32_t xh) {
    asm("dp2a.lo.s32.u32 %0, %1, %2, %0;" : "+r"(lo) : "r"(w0), "r"(xl));
    asm("dp2a.hi.s32.u32 %0, %1, %2, %0;" : "+r"(lo) : "r"(w1), "r"(xl));
    asm("dp2a.lo.s32.s32 %0, %1, %2, %0;" : "+r"(hi) : "r"(w0), "r"(xh));
    asm("dp2a.hi.s32.s32 %0, %1, %2, %0;" : "+r"(hi) : "r"(w1), "r"(xh));
}
__device__ __forceinline__ void i16_vec(uint32_t& lo, uint32_t& hi, const int4& w, const int4& x) {
    // bytes of four consecutive x elements: low bytes 0x6420, high bytes 0x7531
    dp2a_word_pair(lo, hi, w.x, w.y, __byte_perm(x.x, x.y, 0x6420), __byte_perm(x.x, x.y, 0x7531));
    dp2a_word_pair(lo, hi, w.z, w.w, __byte_perm(x.z, x.w, 0x6420), __byte_perm(x.z, x.w, 0x7531));
}

template <int OP>
__device__ __forceinline__ uint32_t fma_vec(uint32_t acc, const int4& w, const int4& x) {
    acc = fma_word<OP>(acc, w.x, x.x);
    acc = fma_word<OP>(acc, w.y, x.y);
    acc = fma_word<OP>(acc, w.z, x.z);
    return fma_word<OP>(acc, w.w, x.w);
}

// Partial sum of one row for participant `tid` of `nthr`. `cols` counts ELEMENTS.
template <int OP, bool VEC>
__device__ __forceinline__ uint32_t row_partial(const void* wrow, const void* x, int64_t cols,
                                                int tid, int nthr) {
    uint32_t acc = 0;
    if (VEC) {
        constexpr int EPV = OP == OP_I16 ? 8 : 4;  // elements per 16-byte vector
        const int64_t nvec = cols / EPV;           // exact on this path
        const int4* wv = static_cast<const int4*>(wrow);
        const int4* xv = static_cast<const int4*>(x);
        int64_t i = tid;
        constexpr int U = 8;
        uint32_t hi = 0;  // int16 only: the sum of w . (high bytes of x)
        for (; i + (int64_t)(U - 1) * nthr < nvec; i += (int64_t)U * nthr) {
            int4 w[U];
#pragma unroll
            for (int u = 0; u < U; ++u) w[u] = ld_stream(wv + i + (int64_t)u * nthr);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (OP == OP_I16)
                    i16_vec(acc, hi, w[u], __ldg(xv + i + (int64_t)u * nthr));
                else
                    acc = fma_vec<OP>(acc, w[u], __ldg(xv + i + (int64_t)u * nthr));
            }
        }
        for (; i < nvec; i += nthr) {
            if (OP == OP_I16)
                i16_vec(acc, hi, ld_stream(wv + i), __ldg(xv + i));
            else
                acc = fma_vec<OP>(acc, ld_stream(wv + i), __ldg(xv + i));
        }
        if (OP == OP_I16) acc += hi << 8;
    } else if (OP == OP_I16) {
        const int16_t* w = static_cast<const int16_t*>(wrow);
        const int16_t* xs = static_cast<const int16_t*>(x);
        for (int64_t i = tid; i < cols; i += nthr) acc = mad_lo(w[i], __ldg(xs + i), acc);
    } else {
        const int32_t* w = static_cast<const int32_t*>(wrow);
        const int32_t* xs = static_cast<const int32_t*>(x);
        for (int64_t i = tid; i < cols; i += nthr) acc = fma_word<OP>(acc, w[i], __ldg(xs + i));
    }
    return acc;
}

__device__ __forceinline__ uint32_t warp_sum(uint32_t v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One warp per row, rows handed out grid-stride.
template <int OP, bool VEC>
__global__ void __launch_bounds__(512)
rows_warp_kernel(const char* __restrict__ w, const void* __restrict__ x, int32_t* __restrict__ y,
                 int64_t rows, int64_t cols, int64_t row_bytes) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = warp; r < rows; r += nwarps) {
        const uint32_t s = warp_sum(row_partial<OP, VEC>(w + r * row_bytes, x, cols, lane, 32));
        if (lane == 0) y[r] = (int32_t)s;
    }
}

// One block per row (few, long rows; also the dot products, rows == 1).
template <int OP, bool VEC>
__global__ void __launch_bounds__(512)
rows_block_kernel(const char* __restrict__ w, const void* __restrict__ x, int32_t* __restrict__ y,
                  int64_t rows, int64_t cols, int64_t row_bytes, int64_t x_period) {
    __shared__ uint32_t part[16];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        // x_period > 1: "row" r is piece r % x_period of a longer row, and meets that piece of x
        const char* xr = static_cast<const char*>(x) + (x_period > 1 ? (r % x_period) * row_bytes : 0);
        uint32_t s = warp_sum(row_partial<OP, VEC>(w + r * row_bytes, xr, cols, threadIdx.x, blockDim.x));
        if (lane == 0) part[wid] = s;
        __syncthreads();
        if (wid == 0) {
            s = lane < (int)(blockDim.x >> 5) ? part[lane] : 0u;
            s = warp_sum(s);
            if (lane == 0) y[r] = (int32_t)s;
        }
        __syncthreads();
    }
}

// y[r] = sum of the `parts` partial sums of row r (few, very long rows cut into pieces).
__global__ void sum_parts_kernel(const int32_t* __restrict__ partial, int32_t* __restrict__ y, int64_t rows,
                                 int parts) {
    const int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (r >= rows) return;
    uint32_t t = 0;
    for (int p = 0; p < parts; ++p) t += (uint32_t)partial[r * parts + p];
    y[r] = (int32_t)t;
}

// WPR warps share a row (interleaved 512-byte pieces), 16 / WPR rows per block per pass;
// persistent blocks walk the rows grid-stride.  Finer than one warp per row, so the
// last pass leaves fewer SMs idle when there are only a few rows per warp.
template <int OP, bool VEC, int WPR>
__global__ void __launch_bounds__(512)
rows_group_kernel(const char* __restrict__ w, const void* __restrict__ x, int32_t* __restrict__ y,
                  int64_t rows, int64_t cols, int64_t row_bytes) {
    constexpr int RPB = 16 / WPR;
    __shared__ uint32_t part[16];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int sub = wid % WPR, rslot = wid / WPR;
    for (int64_t r0 = (int64_t)blockIdx.x * RPB; r0 < rows; r0 += (int64_t)gridDim.x * RPB) {
        const int64_t r = r0 + rslot;
        uint32_t s = 0;
        if (r < rows)
            s = warp_sum(row_partial<OP, VEC>(w + r * row_bytes, x, cols, sub * 32 + lane, WPR * 32));
        if (lane == 0) part[wid] = s;
        __syncthreads();
        if (sub == 0 && lane == 0 && r < rows) {
            uint32_t t = 0;
#pragma unroll
            for (int j = 0; j < WPR; ++j) t += part[wid + j];
            y[r] = (int32_t)t;
        }
        __syncthreads();
    }
}

template <int OP>
int64_t launch_rows(DeviceCtx* ctx, const void* w, const void* x, int32_t* y, int64_t rows,
                    int64_t cols) {
    if (rows <= 0) return 0;
    constexpr int ES = OP == OP_I16 ? 2 : 4;
    constexpr int EPV = 16 / ES;
    const int64_t row_bytes = cols * ES;
    const bool vec = cols % EPV == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(x) % 16 == 0;
    const char* wc = static_cast<const char*>(w);
    const int sms = ctx->sm_count;
    const bool by_block = rows < (int64_t)sms * 4 && cols >= 2048;
    // Long rows: several warps per row, at least one full batch of eight 16-byte loads per
    // lane; one pass per block, so the hardware block scheduler evens out the tail
    // (measured on the 16384 x 16384 case: 86 % of the copy bandwidth with one warp per row
    // and a persistent grid, 100 % this way).
    const int64_t nvec = cols / EPV;
    const int wpr = nvec >= 4096 ? 8 : (nvec >= 2048 ? 4 : (nvec >= 1024 ? 2 : 1));
    // pieces per row for the few-long-rows case: a power of two that divides the row's vectors,
    // leaves at least 4096 vectors (one batch of eight per thread) per piece and fills ~2 blocks per SM
    int parts = 1;
    if (by_block && vec)
        while (parts < 256 && rows * parts * 2 <= (int64_t)sms * 2 && nvec % (parts * 2) == 0 &&
               nvec / (parts * 2) >= 4096)
            parts *= 2;
    int32_t* partial = nullptr;
    if (parts > 1) {
        MB200_TRY(arena_reserve(ctx, ctx->scratch, (size_t)rows * parts * 4 + 1024));
        partial = static_cast<int32_t*>(arena_take(ctx->scratch, (size_t)rows * parts * 4));
    }
    prof_begin(ctx);
    if (vec && !by_block && wpr > 1) {
        const int64_t rpb = 16 / wpr;
        int64_t blocks = (rows + rpb - 1) / rpb;
        if (blocks > (int64_t)sms * 64) blocks = (int64_t)sms * 64;
        if (wpr == 8)
            rows_group_kernel<OP, true, 8><<<(unsigned)blocks, 512, 0, ctx->stream>>>(wc, x, y, rows, cols, row_bytes);
        else if (wpr == 4)
            rows_group_kernel<OP, true, 4><<<(unsigned)blocks, 512, 0, ctx->stream>>>(wc, x, y, rows, cols, row_bytes);
        else
            rows_group_kernel<OP, true, 2><<<(unsigned)blocks, 512, 0, ctx->stream>>>(wc, x, y, rows, cols, row_bytes);
    } else if (by_block && parts > 1) {
        // Few, very long rows (a long dot product is one row): each row is cut into `parts` equal
        // pieces, one block per piece, and a second small kernel adds the pieces up in a fixed
        // order - a single block per row would leave the other SMs idle.
        const int64_t piece_cols = cols / parts;
        rows_block_kernel<OP, true><<<(unsigned)(rows * parts), 512, 0, ctx->stream>>>(
            wc, x, partial, rows * parts, piece_cols, piece_cols * ES, parts);
        count_launch();
        sum_parts_kernel<<<(unsigned)((rows + 127) / 128), 128, 0, ctx->stream>>>(partial, y, rows, parts);
    } else if (by_block) {
        const unsigned grid = (unsigned)rows;
        if (vec)
            rows_block_kernel<OP, true><<<grid, 512, 0, ctx->stream>>>(wc, x, y, rows, cols, row_bytes, 1);
        else
            rows_block_kernel<OP, false><<<grid, 512, 0, ctx->stream>>>(wc, x, y, rows, cols, row_bytes, 1);
    } else {
        int64_t blocks = (rows + 15) / 16;  // 16 warps per block, one row per warp, one pass
        if (blocks > (int64_t)sms * 64) blocks = (int64_t)sms * 64;
        if (vec)
            rows_warp_kernel<OP, true><<<(unsigned)blocks, 512, 0, ctx->stream>>>(wc, x, y, rows, cols, row_bytes);
        else
            rows_warp_kernel<OP, false><<<(unsigned)blocks, 512, 0, ctx->stream>>>(wc, x, y, rows, cols, row_bytes);
    }
    prof_end(ctx);
    count_launch();
    return check_launch("row reduction kernel");
}

}  // namespace

int64_t launch_gemv_q16(DeviceCtx* ctx, const int32_t* w, const int32_t* x, int32_t* y,
                        int64_t rows, int64_t cols) {
    return launch_rows<OP_Q16>(ctx, w, x, y, rows, cols);
}
int64_t launch_gemv_i16(DeviceCtx* ctx, const int16_t* w, const int16_t* x, int32_t* y,
                        int64_t rows, int64_t cols) {
    return launch_rows<OP_I16>(ctx, w, x, y, rows, cols);
}
int64_t launch_dist_l1_q16(DeviceCtx* ctx, const int32_t* a, const int32_t* b, int32_t* out,
                           int64_t len) {
    return launch_rows<OP_L1>(ctx, a, b, out, 1, len);
}

}  // namespace mb200
