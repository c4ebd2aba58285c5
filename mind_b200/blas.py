"""ctypes mirror of the reference's deterministic BLAS intrinsics, for tests and benches.

Each function has the name and argument order of the MIND intrinsic it calls
(``__mind_blas_<name>``; see ``include/mind_b200.h``).  Operands may be numpy arrays
(host memory: the call stages them through the GPU and is synchronous), torch CUDA
tensors (device memory: the call only enqueues work) or raw integer addresses.
Nothing here computes: every function forwards to ``libmind_b200.so`` and raises
``MindB200Error`` on a negative status.
"""
from __future__ import annotations

import numpy as np

from . import check, last_error, lib, MindB200Error


def addr(x) -> int:
    """Raw address of a numpy array, a torch tensor, or an int passed through."""
    if isinstance(x, (int, np.integer)):
        return int(x)
    if isinstance(x, np.ndarray):
        if not x.flags["C_CONTIGUOUS"]:
            raise ValueError("operands must be C-contiguous")
        return x.ctypes.data
    if hasattr(x, "data_ptr"):
        if not x.is_contiguous():
            raise ValueError("operands must be contiguous")
        return x.data_ptr()
    raise TypeError(f"cannot take the address of {type(x)!r}")


def _call6(name, a, b, c, m, k, n):
    return check(getattr(lib(), name)(addr(a), addr(b), addr(c), m, k, n))


def _call5(name, w, x, y, rows, cols):
    return check(getattr(lib(), name)(addr(w), addr(x), addr(y), rows, cols))


def _dot(name, a, b, n):
    v = getattr(lib(), name)(addr(a), addr(b), n)
    msg = last_error()
    if msg:
        raise MindB200Error(-1, msg)
    return int(v)


def matmul_mm_i8_v(a, b, c, m, k, n):
    return _call6("__mind_blas_matmul_mm_i8_v", a, b, c, m, k, n)


def matmul_mm_i8_mt_v(a, b, c, m, k, n):
    return _call6("__mind_blas_matmul_mm_i8_mt_v", a, b, c, m, k, n)


def matmul_mm_q16_v(a, b, c, m, k, n):
    return _call6("__mind_blas_matmul_mm_q16_v", a, b, c, m, k, n)


def matmul_mm_q16_mt_v(a, b, c, m, k, n):
    return _call6("__mind_blas_matmul_mm_q16_mt_v", a, b, c, m, k, n)


def matmul_mm_i16(a, b, c, m, k, n):
    return _call6("__mind_b200_matmul_mm_i16", a, b, c, m, k, n)


def gemv_q16_mt(catalog, query, scores, m, k):
    return _call5("__mind_blas_gemv_q16_mt", catalog, query, scores, m, k)


def matmul_rmajor_q16_v(w, x, y, rows, cols):
    return _call5("__mind_blas_matmul_rmajor_q16_v", w, x, y, rows, cols)


def matmul_rmajor_i16_v(w, x, y, rows, cols):
    return _call5("__mind_blas_matmul_rmajor_i16_v", w, x, y, rows, cols)


def dot_q16_v(a, b, n):
    return _dot("__mind_blas_dot_q16_v", a, b, n)


def dot_l1_q16_v(a, b, n):
    return _dot("__mind_blas_dot_l1_q16_v", a, b, n)


def dot_i16_v(a, b, n):
    return _dot("__mind_blas_dot_i16_v", a, b, n)


STATIC_SCRATCH_BYTES = 8 * 1024 * 1024


def matmul_mm_i8_static(a, b, c, m, k, n, stream: int = 0):
    """int8 GEMM for callers that may not allocate GPU memory (device operands only).

    Same bytes as ``matmul_mm_i8_v``; the re-laid-out operands live in a fixed 8 MiB array
    inside the library instead of a cudaMalloc'ed buffer, so larger shapes are refused with
    ``ERR_TOO_LARGE``.  Synchronous.  See ``mind_b200_matmul_mm_i8_static`` in the header.
    """
    import ctypes as C
    f = lib().mind_b200_matmul_mm_i8_static
    f.argtypes, f.restype = [C.c_int64] * 7, C.c_int64
    return check(f(addr(a), addr(b), addr(c), m, k, n, int(stream)))


def gemmq_bt(a, bt, c, m, k, n):
    """The identity gate's ``gemmq``: B is passed transposed (N x K)."""
    return _call6("gemmq", a, bt, c, m, k, n)


# ---- library control ---------------------------------------------------------------
def set_stream(stream: int) -> None:
    check(lib().mind_b200_set_stream(int(stream)))


def synchronize() -> None:
    check(lib().mind_b200_synchronize())


def device_count() -> int:
    return int(lib().mind_b200_device_count())


def kernel_launches() -> int:
    return int(lib().mind_b200_kernel_launches())


def reserve(scratch_bytes: int, staging_bytes: int) -> None:
    check(lib().mind_b200_reserve(int(scratch_bytes), int(staging_bytes)))


def set_gemm_path(path: int) -> None:
    check(lib().mind_b200_set_gemm_path(int(path)))


def set_tile_order(group_m: int, raster: int = 0) -> None:
    check(lib().mind_b200_set_tile_order(int(group_m), int(raster)))


def set_devices(count: int) -> None:
    """GPUs a host-operand call is spread over (1 = the current device only)."""
    check(lib().mind_b200_set_devices(int(count)))


def devices() -> int:
    return int(lib().mind_b200_devices())


def shutdown() -> None:
    check(lib().mind_b200_shutdown())


KIND_Q16, KIND_I8, KIND_I16 = 0, 1, 2


def lcg_fill(dst, n: int, kind: int, seed: int, offset: int = 0, shift: int = 12) -> None:
    seed &= 0xFFFFFFFFFFFFFFFF
    if seed >= 1 << 63:
        seed -= 1 << 64
    check(lib().mind_b200_lcg_fill(addr(dst), n, kind, seed, offset, shift))


def matvec_wrap(mat, elem_bytes: int, rows: int, cols: int, v, out) -> None:
    check(lib().mind_b200_matvec_wrap(addr(mat), elem_bytes, rows, cols, addr(v), addr(out)))


def profile(enable: bool) -> None:
    """Start / stop timing the dominant kernel of every call with CUDA events."""
    check(lib().mind_b200_profile(1 if enable else 0))


def fp64_fma_peak(with_clock: bool = False):
    """Measured FP64 FMA rate of the current device, FMA per second (and, with_clock, the SM clock
    in MHz the measuring loop ran at)."""
    import ctypes as C
    f = lib().mind_b200_fp64_fma_peak
    f.argtypes, f.restype = [C.POINTER(C.c_double), C.POINTER(C.c_double)], C.c_int64
    v, mhz = C.c_double(0.0), C.c_double(0.0)
    check(f(C.byref(v), C.byref(mhz)))
    return (float(v.value), float(mhz.value)) if with_clock else float(v.value)


def fp32_fma_peak(with_clock: bool = False):
    """Measured FP32 FMA rate of the current device in the packed round-down form the Q16.16 floor
    kernel uses, FMA per second (and, with_clock, the SM clock in MHz the loop ran at)."""
    import ctypes as C
    f = lib().mind_b200_fp32_fma_peak
    f.argtypes, f.restype = [C.POINTER(C.c_double), C.POINTER(C.c_double)], C.c_int64
    v, mhz = C.c_double(0.0), C.c_double(0.0)
    check(f(C.byref(v), C.byref(mhz)))
    return (float(v.value), float(mhz.value)) if with_clock else float(v.value)


def set_q16_split(side_sms: int) -> None:
    """Q16.16 hybrid, measurement knob: SMs of the tensor-core half beside the floor kernel
    (0 = in sequence, -1 = by size)."""
    import ctypes as C
    f = lib().mind_b200_set_q16_split
    f.argtypes, f.restype = [C.c_int64], C.c_int64
    check(f(int(side_sms)))


def profile_read() -> tuple[int, float]:
    """(kernels timed since the last read, their summed duration in ms)."""
    import ctypes as C
    n, ms = C.c_int64(0), C.c_double(0.0)
    check(lib().mind_b200_profile_read(C.byref(n), C.byref(ms)))
    return int(n.value), float(ms.value)
