"""mind_b200 -- MIND's deterministic integer BLAS (int8 / int16 / Q16.16 GEMM, GEMV, dot)
on NVIDIA B200, behind the reference's own ``__mind_blas_*`` i64 C ABI.

The product is ``lib/libmind_b200.so`` (hand-written CUDA for sm_100a, built by
``mind_b200.build``); this package is only the loader and a thin ctypes mirror of
the intrinsic surface (``mind_b200.blas``) for tests and measurements.  There is no
CPU fallback: when the shared library is missing or no B200 is usable, calls fail.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libmind_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_PKG), "include", "mind_b200.h")

ERR_INVALID, ERR_CUDA, ERR_NO_DEVICE, ERR_TIMEOUT, ERR_TOO_LARGE = -1, -2, -3, -4, -5

_lib = None


class MindB200Error(RuntimeError):
    """A libmind_b200 entry point returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libmind_b200 error {code}: {message}")
        self.code = code


def lib() -> C.CDLL:
    """Loads libmind_b200.so (never builds it, never substitutes anything for it)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m mind_b200.build` "
                "(needs nvcc); there is no fallback implementation")
        L = C.CDLL(LIB_PATH)
        i64 = C.c_int64
        six = ["__mind_blas_matmul_mm_i8_v", "__mind_blas_matmul_mm_i8_mt_v",
               "__mind_blas_matmul_mm_q16_v", "__mind_blas_matmul_mm_q16_mt_v",
               "__mind_b200_matmul_mm_i16", "gemmq", "gemmq_kn", "gemmqmm", "gemmi8", "gemmi8mt",
               "mind_b200_lcg_fill", "mind_b200_matvec_wrap"]
        five = ["__mind_blas_gemv_q16_mt", "__mind_blas_matmul_rmajor_q16_v",
                "__mind_blas_matmul_rmajor_i16_v", "mmq", "mmi16", "gemvq"]
        three = ["__mind_blas_dot_q16_v", "__mind_blas_dot_l1_q16_v", "__mind_blas_dot_i16_v",
                 "dotq", "dotl1q", "doti16"]
        for names, n in ((six, 6), (five, 5), (three, 3)):
            for name in names:
                f = getattr(L, name)
                f.argtypes, f.restype = [i64] * n, i64
        L.mind_b200_last_error.restype = C.c_char_p
        for name, n in (("mind_b200_set_stream", 1), ("mind_b200_synchronize", 0),
                        ("mind_b200_device_count", 0), ("mind_b200_kernel_launches", 0),
                        ("mind_b200_reserve", 2), ("mind_b200_set_gemm_path", 1),
                        ("mind_b200_profile", 1), ("mind_b200_set_devices", 1), ("mind_b200_devices", 0),
                        ("mind_b200_shutdown", 0), ("mind_b200_set_tile_order", 2),
                        ("mind_b200_rt_deallocate", 1), ("mind_b200_rt_retag", 2), ("mind_b200_rt_synchronize", 0)):
            f = getattr(L, name)
            f.argtypes, f.restype = [i64] * n, i64
        pi64 = C.POINTER(i64)
        L.mind_b200_profile_read.argtypes = [pi64, C.POINTER(C.c_double)]
        L.mind_b200_profile_read.restype = i64
        L.mind_b200_rt_allocate.argtypes, L.mind_b200_rt_allocate.restype = [i64, pi64, i64, pi64], i64
        L.mind_b200_rt_upload.argtypes, L.mind_b200_rt_upload.restype = [i64, C.c_void_p, i64], i64
        L.mind_b200_rt_download.argtypes, L.mind_b200_rt_download.restype = [i64, C.c_void_p, i64], i64
        L.mind_b200_rt_device_ptr.argtypes, L.mind_b200_rt_device_ptr.restype = [i64, pi64], i64
        L.mind_b200_rt_run_op.argtypes = [C.c_char_p, pi64, i64, pi64, i64]
        L.mind_b200_rt_run_op.restype = i64
        _lib = L
    return _lib


def last_error() -> str | None:
    msg = lib().mind_b200_last_error()
    return msg.decode() if msg else None


def check(status: int) -> int:
    if status < 0:
        raise MindB200Error(status, last_error() or "no message")
    return status
