// Device-side seeded input generator (the reference's LCG with jump-ahead) and
// the wrap-around matrix x vector used for exact large-shape checks.
#include "common.h"

namespace mb200 {
namespace {

constexpr uint64_t LCG_A = 1664525ull, LCG_C = 1013904223ull;
constexpr int LCG_CHUNK = 16;  // consecutive elements per thread

// State after `steps` steps from s0: the affine map x -> a*x + c raised to `steps`.
__device__ __forceinline__ uint64_t lcg_jump(uint64_t s0, uint64_t steps) {
    uint64_t a = 1, c = 0, ca = LCG_A, cc = LCG_C;
    while (steps) {
        if (steps & 1) {
            a = ca * a;
            c = ca * c + cc;
        }
        cc = (ca + 1) * cc;
        ca = ca * ca;
        steps >>= 1;
    }
    return a * s0 + c;
}

template <int KIND>
__global__ void lcg_fill_kernel(void* __restrict__ dst, int64_t n, uint64_t seed, uint64_t offset,
                                int shift) {
    const int64_t chunks = (n + LCG_CHUNK - 1) / LCG_CHUNK;
    for (int64_t ch = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; ch < chunks;
         ch += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i0 = ch * LCG_CHUNK;
        uint64_t s = lcg_jump(seed, offset + (uint64_t)i0);
        const int64_t i1 = i0 + LCG_CHUNK < n ? i0 + LCG_CHUNK : n;
        for (int64_t i = i0; i < i1; ++i) {
            s = s * LCG_A + LCG_C;
            const uint32_t u = (uint32_t)(s >> 16);
            if (KIND == 0)
                static_cast<int32_t*>(dst)[i] = (int32_t)u >> shift;
            else if (KIND == 1)
                static_cast<int8_t*>(dst)[i] = (int8_t)(u >> 16);
            else
                static_cast<int16_t*>(dst)[i] = (int16_t)(u >> 16);
        }
    }
}

// out[r] = sum_c mat[r,c] * v[c] mod 2^32; one warp per row.
template <typename T>
__global__ void matvec_wrap_kernel(const T* __restrict__ mat, int64_t rows, int64_t cols,
                                   const int32_t* __restrict__ v, int32_t* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = warp; r < rows; r += nwarps) {
        const T* row = mat + r * cols;
        uint32_t acc = 0;
        for (int64_t c = lane; c < cols; c += 32) acc += (uint32_t)(int32_t)row[c] * (uint32_t)v[c];
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) out[r] = (int32_t)acc;
    }
}

// Register-only fma.rm.f64 chains: the rate the FP64 pipe sustains when nothing but the FMAs is
// issued.  The ceiling of the Q16.16 GEMM's floor kernel.  Thirty-two independent chains per
// thread, laid out as that kernel's register tile is (an 8 x 4 outer product: every operand
// register feeds several FMAs in a row), which is the form the pipe runs fastest.
__global__ void fp64_fma_peak_kernel(double* __restrict__ sink, int iters, double x, double y,
                                     unsigned long long* __restrict__ clocks) {
    unsigned long long c0 = 0, t0 = 0;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        c0 = clock64();
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    }
    double acc[8][4], a[8], b[4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        a[i] = x + (double)i;
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 6755399441055744.0 + (double)(threadIdx.x + 4 * i + j);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = y + 0.25 * (double)j;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                asm volatile("fma.rm.f64 %0, %1, %2, %0;" : "+d"(acc[i][j]) : "d"(a[i]), "d"(b[j]));
    }
    double t = 0.0;
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) t += acc[i][j];
    if (t == 12345.678) sink[0] = t;  // never true: keeps the chains alive
    if (blockIdx.x == 0 && threadIdx.x == 0) {  // SM cycles and nanoseconds this block took: the clock it ran at
        unsigned long long t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        clocks[0] = clock64() - c0;
        clocks[1] = t1 - t0;
    }
}

// The same for the FP32 pipe in the form the Q16.16 floor kernel uses it: packed fma.rm.f32x2, an
// 8 x 4 tile of register pairs (64 chains per thread).  Counts FMAs, two per instruction.
__global__ void fp32_fma_peak_kernel(float* __restrict__ sink, int iters, float x, float y,
                                     unsigned long long* __restrict__ clocks) {
    unsigned long long c0 = 0, t0 = 0;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        c0 = clock64();
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    }
    unsigned long long acc[8][4], a[8], b[4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const unsigned int av = __float_as_uint(x + (float)i);
        a[i] = ((unsigned long long)av << 32) | av;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const unsigned int s = __float_as_uint(8388608.0f + (float)((threadIdx.x + 4 * i + j) & 255));
            acc[i][j] = ((unsigned long long)s << 32) | s;
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const unsigned int lo = __float_as_uint(y + 0.25f * (float)j), hi = __float_as_uint(y + 0.125f * (float)j);
        b[j] = ((unsigned long long)hi << 32) | lo;
    }
    // 2 x 2 blocks of the tile walked in a ring (every FMA shares an operand register with the one
    // before it): the fastest of the orders tried for a register-only loop (32.0 TFMA/s; rows
    // outermost 30.4, columns outermost 31.5, serpentine 31.7, a scalar fma.rm.f32 8 x 8 tile 28.0)
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < 8; i += 2)
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                asm volatile("fma.rm.f32x2 %0, %1, %2, %0;" : "+l"(acc[i][j]) : "l"(a[i]), "l"(b[j]));
                asm volatile("fma.rm.f32x2 %0, %1, %2, %0;" : "+l"(acc[i][j + 1]) : "l"(a[i]), "l"(b[j + 1]));
                asm volatile("fma.rm.f32x2 %0, %1, %2, %0;" : "+l"(acc[i + 1][j + 1]) : "l"(a[i + 1]), "l"(b[j + 1]));
                asm volatile("fma.rm.f32x2 %0, %1, %2, %0;" : "+l"(acc[i + 1][j]) : "l"(a[i + 1]), "l"(b[j]));
            }
    }
    unsigned long long t = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) t ^= acc[i][j];
    if (t == 0x123456789abcdefull) sink[0] = 1.0f;  // never true: keeps the chains alive
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        clocks[0] = clock64() - c0;
        clocks[1] = t1 - t0;
    }
}

// One of the two peak kernels, timed: FMA / s over the whole device and the SM clock it ran at.
template <typename Launch>
int64_t time_peak_kernel(DeviceCtx* ctx, const char* name, double fma_per_thread, Launch launch, double* fma_per_s,
                         double* sm_mhz) {
    const int threads = 256, blocks = ctx->sm_count;
    unsigned long long* clocks = nullptr;
    MB200_CUDA(cudaMalloc(&clocks, 2 * sizeof(unsigned long long) + sizeof(double)));
    cudaEvent_t e0, e1;
    MB200_CUDA(cudaEventCreate(&e0));
    MB200_CUDA(cudaEventCreate(&e1));
    float ms = 0.f;
    for (int rep = 0; rep < 2; ++rep) {
        MB200_CUDA(cudaEventRecord(e0, ctx->stream));
        launch(blocks, threads, clocks);
        MB200_CUDA(cudaEventRecord(e1, ctx->stream));
        count_launch();
        MB200_TRY(check_launch(name));
        MB200_CUDA(cudaEventSynchronize(e1));
        MB200_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    unsigned long long h[2] = {0, 0};
    MB200_CUDA(cudaMemcpy(h, clocks, sizeof h, cudaMemcpyDeviceToHost));
    cudaFree(clocks);
    *fma_per_s = ms > 0.f ? (double)blocks * threads * fma_per_thread / (ms * 1e-3) : 0.0;
    if (sm_mhz) *sm_mhz = h[1] ? (double)h[0] * 1e3 / (double)h[1] : 0.0;
    return 0;
}

}  // namespace

int64_t measure_fp32_fma_peak(DeviceCtx* ctx, double* fma_per_s, double* sm_mhz) {
    const int iters = 1 << 13;
    return time_peak_kernel(
        ctx, "fp32_fma_peak_kernel", (double)iters * 64.0,
        [&](int blocks, int threads, unsigned long long* clocks) {
            fp32_fma_peak_kernel<<<blocks, threads, 0, ctx->stream>>>(reinterpret_cast<float*>(clocks + 2), iters, 3.0f,
                                                                     0.25f, clocks);
        },
        fma_per_s, sm_mhz);
}

// FMA / s of fp64_fma_peak_kernel on the current device (CUDA events around one launch, after a
// warm-up launch).  Synchronous.
int64_t measure_fp64_fma_peak(DeviceCtx* ctx, double* fma_per_s, double* sm_mhz) {
    const int iters = 1 << 13, threads = 256;
    const int blocks = ctx->sm_count;
    unsigned long long* clocks = nullptr;
    MB200_CUDA(cudaMalloc(&clocks, 2 * sizeof(unsigned long long) + sizeof(double)));
    double* sink = reinterpret_cast<double*>(clocks + 2);
    cudaEvent_t e0, e1;
    MB200_CUDA(cudaEventCreate(&e0));
    MB200_CUDA(cudaEventCreate(&e1));
    float ms = 0.f;
    for (int rep = 0; rep < 2; ++rep) {
        MB200_CUDA(cudaEventRecord(e0, ctx->stream));
        fp64_fma_peak_kernel<<<blocks, threads, 0, ctx->stream>>>(sink, iters, 3.0, 0.25, clocks);
        MB200_CUDA(cudaEventRecord(e1, ctx->stream));
        count_launch();
        MB200_TRY(check_launch("fp64_fma_peak_kernel"));
        MB200_CUDA(cudaEventSynchronize(e1));
        MB200_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    unsigned long long h[2] = {0, 0};
    MB200_CUDA(cudaMemcpy(h, clocks, sizeof h, cudaMemcpyDeviceToHost));
    cudaFree(clocks);
    *fma_per_s = ms > 0.f ? (double)blocks * threads * iters * 32.0 / (ms * 1e-3) : 0.0;
    if (sm_mhz) *sm_mhz = h[1] ? (double)h[0] * 1e3 / (double)h[1] : 0.0;
    return 0;
}

int64_t launch_lcg_fill(DeviceCtx* ctx, void* dst, int64_t n, int kind, uint64_t seed,
                        uint64_t offset, int shift) {
    if (n <= 0) return 0;
    const int64_t chunks = (n + LCG_CHUNK - 1) / LCG_CHUNK;
    int64_t blocks = (chunks + 255) / 256;
    if (blocks > ctx->sm_count * 16) blocks = ctx->sm_count * 16;
    if (kind == 0)
        lcg_fill_kernel<0><<<(unsigned)blocks, 256, 0, ctx->stream>>>(dst, n, seed, offset, shift);
    else if (kind == 1)
        lcg_fill_kernel<1><<<(unsigned)blocks, 256, 0, ctx->stream>>>(dst, n, seed, offset, shift);
    else if (kind == 2)
        lcg_fill_kernel<2><<<(unsigned)blocks, 256, 0, ctx->stream>>>(dst, n, seed, offset, shift);
    else
        return fail(MIND_B200_ERR_INVALID, "lcg_fill: kind must be 0 (q16), 1 (i8) or 2 (i16)");
    count_launch();
    return check_launch("lcg_fill_kernel");
}

int64_t launch_matvec_wrap(DeviceCtx* ctx, const void* mat, int elem_bytes, int64_t rows,
                           int64_t cols, const int32_t* v, int32_t* out) {
    if (rows <= 0) return 0;
    int64_t blocks = (rows + 7) / 8;
    if (blocks > ctx->sm_count * 8) blocks = ctx->sm_count * 8;
    if (elem_bytes == 1)
        matvec_wrap_kernel<int8_t><<<(unsigned)blocks, 256, 0, ctx->stream>>>(
            static_cast<const int8_t*>(mat), rows, cols, v, out);
    else if (elem_bytes == 2)
        matvec_wrap_kernel<int16_t><<<(unsigned)blocks, 256, 0, ctx->stream>>>(
            static_cast<const int16_t*>(mat), rows, cols, v, out);
    else if (elem_bytes == 4)
        matvec_wrap_kernel<int32_t><<<(unsigned)blocks, 256, 0, ctx->stream>>>(
            static_cast<const int32_t*>(mat), rows, cols, v, out);
    else
        return fail(MIND_B200_ERR_INVALID, "matvec_wrap: elem_bytes must be 1, 2 or 4");
    count_launch();
    return check_launch("matvec_wrap_kernel");
}

}  // namespace mb200
