// Device-buffer runtime with the shape of the reference's MindRuntime trait
// (allocate / run_op / synchronize / deallocate over opaque handles), so that a
// Rust `impl MindRuntime` is a thin shim over these calls.
#include <string.h>

#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.h"

namespace mb200 {
namespace {

struct Tensor {
    void* ptr = nullptr;
    int dtype = 0;  // 0 = i8, 1 = i16, 2 = i32 / Q16.16
    std::vector<int64_t> shape;
    size_t bytes = 0;
    int device = 0;
};

std::mutex g_rt_mutex;
std::unordered_map<int64_t, Tensor> g_tensors;
int64_t g_next_handle = 1;

int elem_size(int dtype) { return dtype == 0 ? 1 : (dtype == 1 ? 2 : 4); }

Tensor* find(int64_t h) {
    auto it = g_tensors.find(h);
    return it == g_tensors.end() ? nullptr : &it->second;
}

int64_t dim(const Tensor* t, size_t i) { return i < t->shape.size() ? t->shape[i] : 1; }

}  // namespace
}  // namespace mb200

using namespace mb200;

extern "C" {

int64_t mind_b200_rt_allocate(int64_t dtype, const int64_t* shape, int64_t rank, int64_t* handle_out) {
    clear_error();
    if (dtype < 0 || dtype > 2 || rank < 0 || rank > 8 || (rank > 0 && !shape) || !handle_out)
        return fail(MIND_B200_ERR_INVALID, "rt_allocate: bad descriptor");
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    Tensor t;
    t.dtype = (int)dtype;
    size_t count = 1;
    for (int64_t i = 0; i < rank; ++i) {
        if (shape[i] < 0) return fail(MIND_B200_ERR_INVALID, "rt_allocate: negative dimension");
        t.shape.push_back(shape[i]);
        count *= (size_t)shape[i];
    }
    t.bytes = count * elem_size(t.dtype);
    t.device = ctx->device;
    if (t.bytes) {
        cudaError_t e = cudaMalloc(&t.ptr, t.bytes);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(MIND_B200_ERR_CUDA, "rt_allocate: cudaMalloc(%zu) failed: %s", t.bytes, cudaGetErrorString(e));
        }
    }
    std::lock_guard<std::mutex> lock(g_rt_mutex);
    const int64_t h = g_next_handle++;
    g_tensors[h] = t;
    *handle_out = h;
    return 0;
}

int64_t mind_b200_rt_deallocate(int64_t handle) {
    clear_error();
    std::lock_guard<std::mutex> lock(g_rt_mutex);
    Tensor* t = find(handle);
    if (!t) return fail(MIND_B200_ERR_INVALID, "rt_deallocate: unknown handle %lld", (long long)handle);
    if (t->ptr) {
        cudaDeviceSynchronize();
        cudaFree(t->ptr);
    }
    g_tensors.erase(handle);
    return 0;
}

// The reference's DType has no int8 / int16 (src/types/mod.rs:32-47), so a MindRuntime shim
// allocates such operands as int32-tagged byte buffers whose last dimension is the row length in
// bytes / 4.  This re-tags a buffer as the element type an op reads: same bytes, last dimension
// rescaled (x 4 for int8, x 2 for int16 when coming from int32).
int64_t mind_b200_rt_retag(int64_t handle, int64_t dtype) {
    clear_error();
    if (dtype < 0 || dtype > 2) return fail(MIND_B200_ERR_INVALID, "rt_retag: dtype must be 0 (i8), 1 (i16) or 2 (i32)");
    std::lock_guard<std::mutex> lock(g_rt_mutex);
    Tensor* t = find(handle);
    if (!t) return fail(MIND_B200_ERR_INVALID, "rt_retag: unknown handle %lld", (long long)handle);
    if (t->dtype == (int)dtype) return 0;
    if (t->shape.empty()) return fail(MIND_B200_ERR_INVALID, "rt_retag: a scalar cannot be re-tagged");
    const int64_t row_bytes = t->shape.back() * elem_size(t->dtype);
    if (row_bytes % elem_size((int)dtype))
        return fail(MIND_B200_ERR_INVALID, "rt_retag: a row of %lld bytes is not a whole number of elements", (long long)row_bytes);
    t->shape.back() = row_bytes / elem_size((int)dtype);
    t->dtype = (int)dtype;
    return 0;
}

int64_t mind_b200_rt_upload(int64_t handle, const void* host_src, int64_t bytes) {
    clear_error();
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    std::lock_guard<std::mutex> lock(g_rt_mutex);
    Tensor* t = find(handle);
    if (!t || bytes < 0 || (size_t)bytes > t->bytes || (!host_src && bytes))
        return fail(MIND_B200_ERR_INVALID, "rt_upload: bad handle or size");
    if (bytes) MB200_CUDA(cudaMemcpyAsync(t->ptr, host_src, (size_t)bytes, cudaMemcpyHostToDevice, ctx->stream));
    MB200_CUDA(cudaStreamSynchronize(ctx->stream));
    return 0;
}

int64_t mind_b200_rt_download(int64_t handle, void* host_dst, int64_t bytes) {
    clear_error();
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return MIND_B200_ERR_NO_DEVICE;
    std::lock_guard<std::mutex> lock(g_rt_mutex);
    Tensor* t = find(handle);
    if (!t || bytes < 0 || (size_t)bytes > t->bytes || (!host_dst && bytes))
        return fail(MIND_B200_ERR_INVALID, "rt_download: bad handle or size");
    if (bytes) MB200_CUDA(cudaMemcpyAsync(host_dst, t->ptr, (size_t)bytes, cudaMemcpyDeviceToHost, ctx->stream));
    MB200_CUDA(cudaStreamSynchronize(ctx->stream));
    return 0;
}

int64_t mind_b200_rt_device_ptr(int64_t handle, int64_t* ptr_out) {
    clear_error();
    std::lock_guard<std::mutex> lock(g_rt_mutex);
    Tensor* t = find(handle);
    if (!t || !ptr_out) return fail(MIND_B200_ERR_INVALID, "rt_device_ptr: bad handle");
    *ptr_out = (int64_t)(uintptr_t)t->ptr;
    return 0;
}

int64_t mind_b200_rt_run_op(const char* op, const int64_t* inputs, int64_t n_inputs,
                            const int64_t* outputs, int64_t n_outputs) {
    clear_error();
    if (!op) return fail(MIND_B200_ERR_INVALID, "rt_run_op: null op name");
    if (strncmp(op, "__mind_blas_", 12) == 0) op += 12;
    if (strncmp(op, "__mind_b200_", 12) == 0) op += 12;
    Tensor in[2], out;
    {
        std::lock_guard<std::mutex> lock(g_rt_mutex);
        if (n_inputs != 2 || n_outputs != 1 || !inputs || !outputs)
            return fail(MIND_B200_ERR_INVALID, "rt_run_op: '%s' takes 2 inputs and 1 output", op);
        Tensor* t0 = find(inputs[0]);
        Tensor* t1 = find(inputs[1]);
        Tensor* to = find(outputs[0]);
        if (!t0 || !t1 || !to) return fail(MIND_B200_ERR_INVALID, "rt_run_op: unknown handle");
        in[0] = *t0;
        in[1] = *t1;
        out = *to;
    }
    const int64_t a = (int64_t)(uintptr_t)in[0].ptr, b = (int64_t)(uintptr_t)in[1].ptr;
    const int64_t c = (int64_t)(uintptr_t)out.ptr;
    const bool is_gemm = strncmp(op, "matmul_mm_", 10) == 0;
    if (is_gemm) {
        const int64_t m = dim(&in[0], 0), k = dim(&in[0], 1), n = dim(&in[1], 1);
        if (dim(&in[1], 0) != k || (size_t)(m * n * 4) > out.bytes)
            return fail(MIND_B200_ERR_INVALID, "rt_run_op: '%s' shape mismatch", op);
        const int want = strstr(op, "_i8") ? 0 : (strstr(op, "_i16") ? 1 : 2);
        if (in[0].dtype != want || in[1].dtype != want || out.dtype != 2)
            return fail(MIND_B200_ERR_INVALID, "rt_run_op: '%s' dtype mismatch", op);
        if (!strcmp(op, "matmul_mm_i8_v") || !strcmp(op, "matmul_mm_i8_mt_v"))
            return __mind_blas_matmul_mm_i8_v(a, b, c, m, k, n);
        if (!strcmp(op, "matmul_mm_q16_v") || !strcmp(op, "matmul_mm_q16_mt_v"))
            return __mind_blas_matmul_mm_q16_v(a, b, c, m, k, n);
        if (!strcmp(op, "matmul_mm_i16")) return __mind_b200_matmul_mm_i16(a, b, c, m, k, n);
    } else {
        const int64_t rows = dim(&in[0], 0), cols = dim(&in[0], 1);
        if (dim(&in[1], 0) != cols || (size_t)(rows * 4) > out.bytes)
            return fail(MIND_B200_ERR_INVALID, "rt_run_op: '%s' shape mismatch", op);
        if (!strcmp(op, "gemv_q16_mt") || !strcmp(op, "matmul_rmajor_q16_v")) {
            if (in[0].dtype != 2 || in[1].dtype != 2 || out.dtype != 2)
                return fail(MIND_B200_ERR_INVALID, "rt_run_op: '%s' dtype mismatch", op);
            return __mind_blas_gemv_q16_mt(a, b, c, rows, cols);
        }
        if (!strcmp(op, "matmul_rmajor_i16_v")) {
            if (in[0].dtype != 1 || in[1].dtype != 1 || out.dtype != 2)
                return fail(MIND_B200_ERR_INVALID, "rt_run_op: '%s' dtype mismatch", op);
            return __mind_blas_matmul_rmajor_i16_v(a, b, c, rows, cols);
        }
    }
    return fail(MIND_B200_ERR_INVALID, "rt_run_op: unknown op '%s'", op);
}

int64_t mind_b200_rt_synchronize(void) { return mind_b200_synchronize(); }

}  // extern "C"
