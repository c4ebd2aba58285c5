// Operand re-layout kernels (pure data movement) that put the caller's row-major
// operands into the K-contiguous, 16-byte-pitched form the TMA tiles need:
//   - B (K x N, N contiguous) -> Bt (N x Kp, K contiguous): byte transpose;
//   - A with an unaligned base or K % 16 != 0 -> padded copy (M x Kp);
//   - int16 operands -> signed-high / unsigned-low 8-bit limb planes
//     (a = 256 * hi + lo, hi = a >> 8, lo = a & 255), B transposed on the way.
// Kp is K rounded up to 16; pad bytes are never read (the tensor map's extent is K).
#include "common.h"

namespace mb200 {
namespace {

constexpr int TT = 64;  // transpose tile edge, elements

// grid (ceil(N/64), ceil(K/64)), 256 threads. in: [K][N]; out: [N][kp].
__global__ void transpose_i8_kernel(const int8_t* __restrict__ b, int8_t* __restrict__ bt, int k,
                                    int n, int64_t kp) {
    __shared__ int8_t tile[TT][TT + 4];
    const int n0 = blockIdx.x * TT, k0 = blockIdx.y * TT;
    for (int e = threadIdx.x; e < TT * TT; e += blockDim.x) {
        const int r = e / TT, c = e % TT;  // r: k, c: n (n contiguous in global)
        const int kk = k0 + r, nn = n0 + c;
        tile[r][c] = (kk < k && nn < n) ? b[(size_t)kk * n + nn] : (int8_t)0;
    }
    __syncthreads();
    // each thread writes 4 consecutive k of one n as one 32-bit word
    for (int e = threadIdx.x; e < TT * (TT / 4); e += blockDim.x) {
        const int r = e / (TT / 4), c4 = (e % (TT / 4)) * 4;  // r: n, c4: k
        const int nn = n0 + r, kk = k0 + c4;
        if (nn < n && kk < kp) {
            const uint32_t w = (uint32_t)(uint8_t)tile[c4][r] | ((uint32_t)(uint8_t)tile[c4 + 1][r] << 8) |
                               ((uint32_t)(uint8_t)tile[c4 + 2][r] << 16) |
                               ((uint32_t)(uint8_t)tile[c4 + 3][r] << 24);
            *reinterpret_cast<uint32_t*>(bt + (size_t)nn * kp + kk) = w;
        }
    }
}

// in: [K][N] int16; out: hi / lo planes [N][kp].  The low plane is stored minus 128 (as a signed
// byte: low ^ 0x80), so that both planes of B are signed and one MMA can take them side by side;
// the GEMM adds 128 * (row sum of A) back.
__global__ void split_transpose_i16_kernel(const int16_t* __restrict__ b, int8_t* __restrict__ bt_hi,
                                           uint8_t* __restrict__ bt_lo, int k, int n, int64_t kp) {
    __shared__ int16_t tile[TT][TT + 2];
    const int n0 = blockIdx.x * TT, k0 = blockIdx.y * TT;
    for (int e = threadIdx.x; e < TT * TT; e += blockDim.x) {
        const int r = e / TT, c = e % TT;
        const int kk = k0 + r, nn = n0 + c;
        tile[r][c] = (kk < k && nn < n) ? b[(size_t)kk * n + nn] : (int16_t)0;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < TT * (TT / 4); e += blockDim.x) {
        const int r = e / (TT / 4), c4 = (e % (TT / 4)) * 4;
        const int nn = n0 + r, kk = k0 + c4;
        if (nn < n && kk < kp) {
            uint32_t hi = 0, lo = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int v = tile[c4 + j][r];
                hi |= (uint32_t)((v >> 8) & 0xff) << (8 * j);
                lo |= (uint32_t)(v & 0xff) << (8 * j);
            }
            *reinterpret_cast<uint32_t*>(bt_hi + (size_t)nn * kp + kk) = hi;
            *reinterpret_cast<uint32_t*>(bt_lo + (size_t)nn * kp + kk) = lo ^ 0x80808080u;
        }
    }
}

// src [rows][cols] int32 -> dst [cols][rows]; grid (ceil(cols/32), ceil(rows/32)), block (32, 8).
__global__ void transpose_i32_kernel(const int32_t* __restrict__ src, int32_t* __restrict__ dst,
                                     int64_t rows, int64_t cols) {
    __shared__ int32_t tile[32][33];
    const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int64_t r = r0 + j, c = c0 + threadIdx.x;
        if (r < rows && c < cols) tile[j][threadIdx.x] = src[r * cols + c];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int64_t c = c0 + j, r = r0 + threadIdx.x;
        if (r < rows && c < cols) dst[c * rows + r] = tile[threadIdx.x][j];
    }
}

// Row copy into a kp-pitched buffer; grid-stride over rows, threads over bytes.
__global__ void pad_rows_i8_kernel(const int8_t* __restrict__ a, int8_t* __restrict__ ap, int64_t m,
                                   int64_t k, int64_t kp) {
    for (int64_t r = blockIdx.x; r < m; r += gridDim.x)
        for (int64_t c = threadIdx.x; c < kp; c += blockDim.x)
            ap[r * kp + c] = c < k ? a[r * k + c] : (int8_t)0;
}

// Row-wise split of an int16 matrix into a signed high-byte plane and a low-byte plane.
// lo_xor = 0x80 stores the low plane minus 128 (see split_transpose_i16_kernel: the B operand);
// row_sums, when given, receives the int32 sum of every row (the A operand).
// One block per row at a time, so the row sum needs no atomics here.
__global__ void split_rows_i16_kernel(const int16_t* __restrict__ a, int8_t* __restrict__ hi,
                                      uint8_t* __restrict__ lo, int64_t m, int64_t k, int64_t kp,
                                      uint32_t lo_xor, int32_t* __restrict__ row_sums,
                                      int32_t* __restrict__ zero_buf, int64_t zero_n) {
    __shared__ int warp_part[8];
    for (int64_t z = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; z < zero_n; z += (int64_t)gridDim.x * blockDim.x)
        zero_buf[z] = 0;
    for (int64_t r = blockIdx.x; r < m; r += gridDim.x) {
        int sum = 0;
        for (int64_t c = threadIdx.x; c < kp; c += blockDim.x) {
            const int v = c < k ? (int)a[r * k + c] : 0;
            hi[r * kp + c] = (int8_t)(v >> 8);
            lo[r * kp + c] = (uint8_t)((v & 0xff) ^ lo_xor);
            sum += v;
        }
        if (row_sums) {  // uniform across the block
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = sum;
            __syncthreads();
            if (threadIdx.x == 0) {
                int t = 0;
                for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += warp_part[w];
                row_sums[r] = t;
            }
            __syncthreads();
        }
    }
}

// 32 int16 per thread (four 16-byte loads in flight, eight 8-byte stores); needs k % 8 == 0,
// kp == k and a 16-byte aligned base.  Byte permutes pick the low / high bytes.  Row sums (zero
// on entry) are added once per warp when its 256 elements lie in one row, else per thread.
// zero_buf: an unrelated buffer to clear on the way (the row sums of the NEXT split launch).
__global__ void split_rows_i16_vec_kernel(const uint4* __restrict__ a, uint2* __restrict__ hi,
                                          uint2* __restrict__ lo, int64_t n8, uint32_t lo_xor4,
                                          int32_t* __restrict__ row_sums, int64_t k8,
                                          int32_t* __restrict__ zero_buf, int64_t zero_n) {
    constexpr int U = 4;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int lane = threadIdx.x & 31;
    for (int64_t z = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; z < zero_n; z += stride) zero_buf[z] = 0;
    const bool small = n8 < 0x7fffffff;  // 32-bit division for the row index
    // the loop runs on the warp's first index, so that every lane takes part in the shuffles
    for (int64_t w0 = blockIdx.x * (int64_t)blockDim.x + (threadIdx.x & ~31); w0 < n8; w0 += stride * U) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (w0 + lane + u * stride < n8) v[u] = a[w0 + lane + u * stride];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = w0 + lane + u * stride;
            const bool ok = i < n8;
            uint2 h = make_uint2(0u, 0u), l = make_uint2(0u, 0u);
            if (ok) {
                h = make_uint2(__byte_perm(v[u].x, v[u].y, 0x7531), __byte_perm(v[u].z, v[u].w, 0x7531));
                l = make_uint2(__byte_perm(v[u].x, v[u].y, 0x6420), __byte_perm(v[u].z, v[u].w, 0x6420));
                hi[i] = h;
                lo[i] = make_uint2(l.x ^ lo_xor4, l.y ^ lo_xor4);
            }
            if (row_sums) {  // uniform
                int sum = 256 * (__dp4a((int)h.x, 0x01010101, 0) + __dp4a((int)h.y, 0x01010101, 0)) +
                          (int)(__dp4a(l.x, 0x01010101u, 0u) + __dp4a(l.y, 0x01010101u, 0u));
                const int64_t first = w0 + u * stride;  // the warp's first vector: a multiple of 32
                if (k8 % 32 == 0) {  // a warp's 256 elements never straddle rows
                    sum = __reduce_add_sync(0xffffffffu, sum);
                    if (lane == 0 && first < n8)
                        atomicAdd(row_sums + (small ? (int64_t)((uint32_t)first / (uint32_t)k8) : first / k8), sum);
                } else {
                    const int64_t r = !ok ? -1 : small ? (int64_t)((uint32_t)i / (uint32_t)k8) : i / k8;
                    const int64_t r_first = __shfl_sync(0xffffffffu, r, 0);
                    if (__all_sync(0xffffffffu, !ok || r == r_first)) {
                        sum = __reduce_add_sync(0xffffffffu, sum);
                        if (lane == 0 && r_first >= 0) atomicAdd(row_sums + r_first, sum);
                    } else if (ok) {
                        atomicAdd(row_sums + r, sum);
                    }
                }
            }
        }
    }
}

// Both operands of the int16 GEMM split in ONE launch, each row owned by a group of G threads
// (a warp for short rows, the whole block for long ones), so that a row sum is a plain store:
// no atomics, nothing to clear first.  A thread takes 16 consecutive int16 (two 16-byte loads
// that bypass L1 and are marked evict-first in L2: the input is read once, while the planes
// written here are read again by the GEMM right away and should stay in L2) and stores 16 bytes
// to each plane.  Needs K % 16 == 0, dense rows and 16-byte aligned bases.
struct SplitJob {
    const uint4* src;
    uint4* hi;
    uint4* lo;
    int64_t rows, pairs_per_row;  // a pair = two 16-byte vectors = 16 elements
    uint32_t lo_xor4;
    int32_t* row_sums;
    int n_blocks;
    int group;  // threads that share a row: 32 (short rows) or 256
};

__device__ __forceinline__ uint64_t evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint4 ld_once(const uint4* p, uint64_t policy) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(policy));
    return v;
}

__global__ void __launch_bounds__(256) split_i16_fused_kernel(const SplitJob j0, const SplitJob j1) {
    __shared__ int warp_part[8];
    // the GEMM that follows is launched so that it may start (up to its own wait) while this runs
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const bool first = (int)blockIdx.x < j0.n_blocks;
    const SplitJob& job = first ? j0 : j1;
    const int b = first ? (int)blockIdx.x : (int)blockIdx.x - j0.n_blocks;
    const int G = job.group, GROUPS = 256 / G;  // uniform over the block
    const int g = threadIdx.x / G, t = threadIdx.x % G;
    const int64_t ppr = job.pairs_per_row;
    const uint64_t once = evict_first_policy();
    for (int64_t row = (int64_t)b * GROUPS + g; row < job.rows; row += (int64_t)job.n_blocks * GROUPS) {
        int sum = 0;
        const uint4* src = job.src + row * ppr * 2;
        uint4* hi = job.hi + row * ppr;
        uint4* lo = job.lo + row * ppr;
        for (int64_t p0 = t; p0 < ppr; p0 += 2 * G) {
            const int64_t p1 = p0 + G;
            const bool two = p1 < ppr;
            uint4 v[4];
            v[0] = ld_once(src + 2 * p0, once);
            v[1] = ld_once(src + 2 * p0 + 1, once);
            if (two) {
                v[2] = ld_once(src + 2 * p1, once);
                v[3] = ld_once(src + 2 * p1 + 1, once);
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (u == 1 && !two) break;
                const uint4 x = v[2 * u], y = v[2 * u + 1];
                const uint4 h = make_uint4(__byte_perm(x.x, x.y, 0x7531), __byte_perm(x.z, x.w, 0x7531),
                                           __byte_perm(y.x, y.y, 0x7531), __byte_perm(y.z, y.w, 0x7531));
                const uint4 l = make_uint4(__byte_perm(x.x, x.y, 0x6420), __byte_perm(x.z, x.w, 0x6420),
                                           __byte_perm(y.x, y.y, 0x6420), __byte_perm(y.z, y.w, 0x6420));
                const int64_t p = u ? p1 : p0;
                hi[p] = h;
                lo[p] = make_uint4(l.x ^ job.lo_xor4, l.y ^ job.lo_xor4, l.z ^ job.lo_xor4, l.w ^ job.lo_xor4);
                if (job.row_sums)
                    sum += 256 * (__dp4a((int)h.x, 0x01010101, 0) + __dp4a((int)h.y, 0x01010101, 0) +
                                  __dp4a((int)h.z, 0x01010101, 0) + __dp4a((int)h.w, 0x01010101, 0)) +
                           (int)(__dp4a(l.x, 0x01010101u, 0u) + __dp4a(l.y, 0x01010101u, 0u) +
                                 __dp4a(l.z, 0x01010101u, 0u) + __dp4a(l.w, 0x01010101u, 0u));
            }
        }
        if (job.row_sums) {  // uniform per group; for G = 256 the whole block walks the same rows
            sum = __reduce_add_sync(0xffffffffu, sum);
            if (G == 32) {
                if (t == 0) job.row_sums[row] = sum;
            } else {
                if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = sum;
                __syncthreads();
                if (threadIdx.x == 0) {
                    int total = 0;
#pragma unroll
                    for (int w = 0; w < 8; ++w) total += warp_part[w];
                    job.row_sums[row] = total;
                }
                __syncthreads();
            }
        }
    }
}

// int32 matrix [rows][cols] -> byte planes [rows][pitch] (cols % 4 == 0, 16-byte aligned source).
// WHAT = 0: the four bytes of each element (plane 3 holds the signed top byte);
// WHAT = 1: the two bytes of (element >> 16), i.e. planes 0 / 1 = bytes 2 / 3 of the element;
// WHAT = 2: those two, then planes 2 / 3 = bytes 0 / 1 (the high half first, then the low half).
template <int WHAT>
__global__ void split_i32_bytes_kernel(const int4* __restrict__ src, uint8_t* __restrict__ p0,
                                       uint8_t* __restrict__ p1, uint8_t* __restrict__ p2,
                                       uint8_t* __restrict__ p3, int64_t rows, int64_t cols4, int64_t pitch) {
    const int64_t total = rows * cols4;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cols4, c = (i - r * cols4) * 4;
        const int4 v = src[i];
        // byte b of the four elements, packed in element order
        const uint32_t lo01 = __byte_perm(v.x, v.y, 0x5140), lo23 = __byte_perm(v.z, v.w, 0x5140);  // bytes 0,1
        const uint32_t hi01 = __byte_perm(v.x, v.y, 0x7362), hi23 = __byte_perm(v.z, v.w, 0x7362);  // bytes 2,3
        // lo01 = [x.b0, y.b0, x.b1, y.b1], lo23 = [z.b0, w.b0, z.b1, w.b1]; likewise hi* for bytes 2, 3
        const uint32_t b0 = __byte_perm(lo01, lo23, 0x5410), b1 = __byte_perm(lo01, lo23, 0x7632);
        const uint32_t b2 = __byte_perm(hi01, hi23, 0x5410), b3 = __byte_perm(hi01, hi23, 0x7632);
        const int64_t o = r * pitch + c;
        if (WHAT == 0) {
            *reinterpret_cast<uint32_t*>(p0 + o) = b0;
            *reinterpret_cast<uint32_t*>(p1 + o) = b1;
            *reinterpret_cast<uint32_t*>(p2 + o) = b2;
            *reinterpret_cast<uint32_t*>(p3 + o) = b3;
        } else {
            *reinterpret_cast<uint32_t*>(p0 + o) = b2;
            *reinterpret_cast<uint32_t*>(p1 + o) = b3;
            if (WHAT == 2) {
                *reinterpret_cast<uint32_t*>(p2 + o) = b0;
                *reinterpret_cast<uint32_t*>(p3 + o) = b1;
            }
        }
    }
}

// a[m][k] -> four byte planes [m][kp] and (a & 0xffff) as binary32, transposed to [k][mp]: one tile
// of 64 rows by 64 of K per call (256 threads), the transposition through shared memory so that
// both sides move whole lines.
__device__ __forceinline__ void split_q16_a_tile(float (&ft)[64][65], int tile_k, int tile_r,
                                                 const int32_t* __restrict__ a, uint8_t* __restrict__ p0,
                                                 uint8_t* __restrict__ p1, uint8_t* __restrict__ p2,
                                                 uint8_t* __restrict__ p3, float* __restrict__ a_low_t, int m, int k,
                                                 int64_t kp, int64_t mp, bool vec) {
    const int r0 = tile_r * 64, k0 = tile_k * 64, tid = threadIdx.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = (tid >> 4) + 16 * i, kq = (tid & 15) * 4;
        int4 v = make_int4(0, 0, 0, 0);
        const bool inside = r0 + r < m && k0 + kq < k;
        if (inside) {
            const int32_t* src = a + (size_t)(r0 + r) * k + k0 + kq;
            if (vec) {  // K % 4 == 0 and a 16-byte aligned base
                v = *reinterpret_cast<const int4*>(src);
            } else {    // element by element; past the row's end the group is filled with zeros
                const int left = k - (k0 + kq);
                v.x = src[0];
                if (left > 1) v.y = src[1];
                if (left > 2) v.z = src[2];
                if (left > 3) v.w = src[3];
            }
        }
        ft[kq][r] = q16_low_half_f32(v.x);
        ft[kq + 1][r] = q16_low_half_f32(v.y);
        ft[kq + 2][r] = q16_low_half_f32(v.z);
        ft[kq + 3][r] = q16_low_half_f32(v.w);
        if (inside) {
            const uint32_t lo01 = __byte_perm(v.x, v.y, 0x5140), lo23 = __byte_perm(v.z, v.w, 0x5140);
            const uint32_t hi01 = __byte_perm(v.x, v.y, 0x7362), hi23 = __byte_perm(v.z, v.w, 0x7362);
            const int64_t o = (int64_t)(r0 + r) * kp + k0 + kq;
            *reinterpret_cast<uint32_t*>(p0 + o) = __byte_perm(lo01, lo23, 0x5410);
            *reinterpret_cast<uint32_t*>(p1 + o) = __byte_perm(lo01, lo23, 0x7632);
            *reinterpret_cast<uint32_t*>(p2 + o) = __byte_perm(hi01, hi23, 0x5410);
            *reinterpret_cast<uint32_t*>(p3 + o) = __byte_perm(hi01, hi23, 0x7632);
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int kk = (tid >> 4) + 16 * i, rq = (tid & 15) * 4;
        if (k0 + kk < k && r0 + rq < mp)  // rows past m were read as zeros
            *reinterpret_cast<float4*>(a_low_t + (size_t)(k0 + kk) * mp + r0 + rq) =
                make_float4(ft[kk][rq], ft[kk][rq + 1], ft[kk][rq + 2], ft[kk][rq + 3]);
    }
}

// Everything the fused Q16.16 kernel reads, in one launch: blocks [0, a_blocks) split A (above),
// blocks [a_blocks, a_blocks + b_blocks) split B into its four byte planes and (b & 0xffff) * 2^-16
// as binary32, the remaining blocks (if any) zero C for a product whose tiles are shared between
// CTAs.  The kernel after this one may start while it runs (its set-up touches no global
// memory; it waits for this grid before it reads or writes anything).
struct SplitQ16Job {
    const int32_t *a, *b;
    uint8_t *ap[4], *bp[4];
    float *a_low_t, *b_low;
    int32_t* c_zero;  // nullptr: C is not touched
    int vec_a, vec_b, vec_c;  // 16-byte accesses allowed on that operand (aligned base, row length a multiple of 4)
    int m, k, n;
    int64_t kp, np, mp;
    int a_tiles_k, a_blocks, b_blocks;
};

__global__ void __launch_bounds__(256) split_q16_ab_kernel(const SplitQ16Job job) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float ft[64][65];
    const int blk = blockIdx.x;
    if (blk < job.a_blocks) {
        split_q16_a_tile(ft, blk % job.a_tiles_k, blk / job.a_tiles_k, job.a, job.ap[0], job.ap[1], job.ap[2],
                         job.ap[3], job.a_low_t, job.m, job.k, job.kp, job.mp, job.vec_a != 0);
    } else if (blk < job.a_blocks + job.b_blocks) {
        const int64_t cols4 = (job.n + 3) / 4, total = (int64_t)job.k * cols4;
        for (int64_t i = (int64_t)(blk - job.a_blocks) * 256 + threadIdx.x; i < total; i += (int64_t)job.b_blocks * 256) {
            const int64_t r = i / cols4, c = (i - r * cols4) * 4;
            const int32_t* src = job.b + r * job.n + c;
            int4 v = make_int4(0, 0, 0, 0);
            if (job.vec_b) {
                v = *reinterpret_cast<const int4*>(src);
            } else {
                const int64_t left = job.n - c;
                v.x = src[0];
                if (left > 1) v.y = src[1];
                if (left > 2) v.z = src[2];
                if (left > 3) v.w = src[3];
            }
            const uint32_t lo01 = __byte_perm(v.x, v.y, 0x5140), lo23 = __byte_perm(v.z, v.w, 0x5140);
            const uint32_t hi01 = __byte_perm(v.x, v.y, 0x7362), hi23 = __byte_perm(v.z, v.w, 0x7362);
            const int64_t o = r * job.np + c;
            *reinterpret_cast<uint32_t*>(job.bp[0] + o) = __byte_perm(hi01, hi23, 0x5410);  // bytes of b >> 16
            *reinterpret_cast<uint32_t*>(job.bp[1] + o) = __byte_perm(hi01, hi23, 0x7632);
            *reinterpret_cast<uint32_t*>(job.bp[2] + o) = __byte_perm(lo01, lo23, 0x5410);  // bytes of b & 0xffff
            *reinterpret_cast<uint32_t*>(job.bp[3] + o) = __byte_perm(lo01, lo23, 0x7632);
            *reinterpret_cast<float4*>(job.b_low + o) =
                make_float4(q16_low_half_scaled_f32(v.x), q16_low_half_scaled_f32(v.y), q16_low_half_scaled_f32(v.z),
                            q16_low_half_scaled_f32(v.w));
        }
    } else {
        const int z_blocks = gridDim.x - job.a_blocks - job.b_blocks;
        const int64_t first = (int64_t)(blk - job.a_blocks - job.b_blocks) * 256 + threadIdx.x, step = (int64_t)z_blocks * 256;
        if (job.vec_c) {
            int4* dst = reinterpret_cast<int4*>(job.c_zero);
            for (int64_t i = first; i < (int64_t)job.m * job.n / 4; i += step) dst[i] = make_int4(0, 0, 0, 0);
        } else {
            for (int64_t i = first; i < (int64_t)job.m * job.n; i += step) job.c_zero[i] = 0;
        }
    }
}

}  // namespace

// See split_q16_ab_kernel.  b_low has B's plane pitch np (in elements); zero_c: also clear c[m][n].
int64_t launch_split_q16_ab(DeviceCtx* ctx, const int32_t* a, const int32_t* b, uint8_t* const ap[4],
                            uint8_t* const bp[4], float* a_low_t, float* b_low, int32_t* c, bool zero_c, int64_t m,
                            int64_t k, int64_t n, int64_t kp, int64_t np, int64_t mp) {
    if (m <= 0 || k <= 0 || n <= 0) return 0;
    SplitQ16Job job;
    job.a = a;
    job.b = b;
    for (int i = 0; i < 4; ++i) {
        job.ap[i] = ap[i];
        job.bp[i] = bp[i];
    }
    job.a_low_t = a_low_t;
    job.b_low = b_low;
    job.c_zero = zero_c ? c : nullptr;
    job.vec_a = (k % 4 == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0) ? 1 : 0;
    job.vec_b = (n % 4 == 0 && reinterpret_cast<uintptr_t>(b) % 16 == 0) ? 1 : 0;
    job.vec_c = ((m * n) % 4 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0) ? 1 : 0;
    job.m = (int)m;
    job.k = (int)k;
    job.n = (int)n;
    job.kp = kp;
    job.np = np;
    job.mp = mp;
    const int64_t a_blocks = ((k + 63) / 64) * ((m + 63) / 64);
    int64_t b_blocks = (k * ((n + 3) / 4) + 1023) / 1024, z_blocks = zero_c ? (m * n / 4 + 2047) / 2048 + 1 : 0;
    if (b_blocks > ctx->sm_count * 16) b_blocks = ctx->sm_count * 16;
    if (z_blocks > ctx->sm_count * 8) z_blocks = ctx->sm_count * 8;
    if (a_blocks + b_blocks + z_blocks > 0x7fffffff) return fail(MIND_B200_ERR_TOO_LARGE, "operand split grid too large");
    job.a_tiles_k = (int)((k + 63) / 64);
    job.a_blocks = (int)a_blocks;
    job.b_blocks = (int)b_blocks;
    split_q16_ab_kernel<<<(unsigned)(a_blocks + b_blocks + z_blocks), 256, 0, ctx->stream>>>(job);
    count_launch();
    return check_launch("split_q16_ab_kernel");
}

int64_t launch_split_i32_bytes(DeviceCtx* ctx, const int32_t* src, uint8_t* const planes[4], int what,
                               int64_t rows, int64_t cols, int64_t pitch) {
    const int64_t total = rows * (cols / 4);
    if (total <= 0) return 0;
    int64_t blocks = (total + 255) / 256;
    if (blocks > ctx->sm_count * 64) blocks = ctx->sm_count * 64;
    const int4* s4 = reinterpret_cast<const int4*>(src);
    if (what == 0)
        split_i32_bytes_kernel<0><<<(unsigned)blocks, 256, 0, ctx->stream>>>(s4, planes[0], planes[1], planes[2],
                                                                             planes[3], rows, cols / 4, pitch);
    else if (what == 2)
        split_i32_bytes_kernel<2><<<(unsigned)blocks, 256, 0, ctx->stream>>>(s4, planes[0], planes[1], planes[2],
                                                                             planes[3], rows, cols / 4, pitch);
    else
        split_i32_bytes_kernel<1><<<(unsigned)blocks, 256, 0, ctx->stream>>>(s4, planes[0], planes[1], nullptr,
                                                                             nullptr, rows, cols / 4, pitch);
    count_launch();
    return check_launch("split_i32_bytes_kernel");
}

int64_t launch_transpose_i8(DeviceCtx* ctx, const int8_t* b, int8_t* bt, int64_t k, int64_t n,
                            int64_t kp) {
    dim3 grid((unsigned)((n + TT - 1) / TT), (unsigned)((kp + TT - 1) / TT));
    if (grid.y > 65535) return fail(MIND_B200_ERR_TOO_LARGE, "K above 4194240 is not supported");
    transpose_i8_kernel<<<grid, 256, 0, ctx->stream>>>(b, bt, (int)k, (int)n, kp);
    count_launch();
    return check_launch("transpose_i8_kernel");
}

int64_t launch_split_transpose_i16(DeviceCtx* ctx, const int16_t* b, int8_t* bt_hi, uint8_t* bt_lo,
                                   int64_t k, int64_t n, int64_t kp) {
    dim3 grid((unsigned)((n + TT - 1) / TT), (unsigned)((kp + TT - 1) / TT));
    if (grid.y > 65535) return fail(MIND_B200_ERR_TOO_LARGE, "K above 4194240 is not supported");
    split_transpose_i16_kernel<<<grid, 256, 0, ctx->stream>>>(b, bt_hi, bt_lo, (int)k, (int)n, kp);
    count_launch();
    return check_launch("split_transpose_i16_kernel");
}

int64_t launch_transpose_i32(DeviceCtx* ctx, const int32_t* src, int32_t* dst, int64_t rows,
                             int64_t cols) {
    dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32));
    if (grid.y > 65535) return fail(MIND_B200_ERR_TOO_LARGE, "more than 2097120 rows to transpose");
    transpose_i32_kernel<<<grid, dim3(32, 8), 0, ctx->stream>>>(src, dst, rows, cols);
    count_launch();
    return check_launch("transpose_i32_kernel");
}

int64_t launch_pad_rows_i8(DeviceCtx* ctx, const int8_t* a, int8_t* ap, int64_t m, int64_t k,
                           int64_t kp) {
    unsigned grid = (unsigned)(m < ctx->sm_count * 16 ? m : ctx->sm_count * 16);
    pad_rows_i8_kernel<<<grid, 256, 0, ctx->stream>>>(a, ap, m, k, kp);
    count_launch();
    return check_launch("pad_rows_i8_kernel");
}

bool split_i16_pair_usable(const int16_t* a, int64_t k, const int16_t* b, int64_t n) {
    return k % 16 == 0 && n % 16 == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0 &&
           reinterpret_cast<uintptr_t>(b) % 16 == 0;
}

// A (m x k, plain low plane, row sums) and B (k x n, low plane minus 128) in one launch; the
// planes keep each operand's own orientation and pitch (k resp. n).
int64_t launch_split_i16_pair(DeviceCtx* ctx, const int16_t* a, int8_t* a_hi, uint8_t* a_lo, int32_t* a_row_sums,
                              int64_t m, int64_t k, const int16_t* b, int8_t* b_hi, uint8_t* b_lo, int64_t n) {
    auto job = [&](const int16_t* src, int8_t* hi, uint8_t* lo, int64_t rows, int64_t cols, uint32_t x, int32_t* sums) {
        SplitJob j;
        j.src = reinterpret_cast<const uint4*>(src);
        j.hi = reinterpret_cast<uint4*>(hi);
        j.lo = reinterpret_cast<uint4*>(lo);
        j.rows = rows;
        j.pairs_per_row = cols / 16;
        j.lo_xor4 = x * 0x01010101u;
        j.row_sums = sums;
        j.group = j.pairs_per_row <= 64 ? 32 : 256;  // a warp per short row, the block per long one
        const int groups = 256 / j.group;
        j.n_blocks = (int)((rows + groups - 1) / groups);  // capped below: one wave for both jobs
        if (j.n_blocks < 1) j.n_blocks = 1;
        return j;
    };
    SplitJob ja = job(a, a_hi, a_lo, m, k, 0u, a_row_sums);
    SplitJob jb = job(b, b_hi, b_lo, k, n, 0x80u, nullptr);
    // One wave: eight blocks per SM in all, shared between the operands by their sizes, each
    // block walking several rows (a second wave would run at a fraction of the bandwidth).
    const int64_t wave = (int64_t)ctx->sm_count * 8;
    if ((int64_t)ja.n_blocks + jb.n_blocks > wave) {
        const double wa = (double)m * k, wb = (double)k * n;
        int64_t na = (int64_t)((double)wave * wa / (wa + wb));
        if (na < 1) na = 1;
        if (na > wave - 1) na = wave - 1;
        if (na > ja.n_blocks) na = ja.n_blocks;
        int64_t nb = wave - na;
        if (nb > jb.n_blocks) {
            nb = jb.n_blocks;
            na = wave - nb < ja.n_blocks ? wave - nb : ja.n_blocks;
        }
        ja.n_blocks = (int)na;
        jb.n_blocks = (int)nb;
    }
    const unsigned grid = (unsigned)(ja.n_blocks + jb.n_blocks);
    split_i16_fused_kernel<<<grid, 256, 0, ctx->stream>>>(ja, jb);
    count_launch();
    return check_launch("split_i16_fused_kernel");
}

int64_t launch_split_rows_i16(DeviceCtx* ctx, const int16_t* a, int8_t* hi, uint8_t* lo, int64_t m,
                              int64_t k, int64_t kp, bool lo_minus_128, int32_t* row_sums, bool sums_are_zero,
                              int32_t* zero_buf, int64_t zero_n) {
    const uint32_t x = lo_minus_128 ? 0x80u : 0u;
    if (kp == k && k % 8 == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0) {
        if (row_sums && !sums_are_zero) MB200_CUDA(cudaMemsetAsync(row_sums, 0, (size_t)m * 4, ctx->stream));
        const int64_t n8 = m * k / 8;
        int64_t blocks = (n8 + 256 * 4 - 1) / (256 * 4);  // one pass: four vectors per thread
        if (blocks > ctx->sm_count * 256) blocks = ctx->sm_count * 256;
        if (blocks < 1) blocks = 1;
        split_rows_i16_vec_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(
            reinterpret_cast<const uint4*>(a), reinterpret_cast<uint2*>(hi),
            reinterpret_cast<uint2*>(lo), n8, x * 0x01010101u, row_sums, k / 8, zero_buf, zero_n);
    } else {
        unsigned grid = (unsigned)(m < ctx->sm_count * 16 ? m : ctx->sm_count * 16);
        if (grid < 1) grid = 1;
        split_rows_i16_kernel<<<grid, 256, 0, ctx->stream>>>(a, hi, lo, m, k, kp, x, row_sums, zero_buf, zero_n);
    }
    count_launch();
    return check_launch("split_rows_i16_kernel");
}

}  // namespace mb200
