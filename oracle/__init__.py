"""ctypes front end of the CPU checker (``liboracle.so`` and ``_ref/libmind_ref.so``).

TEST INFRASTRUCTURE ONLY.  Nothing under ``mind_b200/`` may import this package; it
exists so that the tests, the smoke check and the CPU-baseline leg of the bench can
compare the CUDA path with an independent CPU restatement of the reference's rules
(``oracle.c``) and with the reference's own C runtime compiled as a black box
(``_ref/libmind_ref.so``, built by ``oracle/Makefile`` from the reference checkout).
"""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle.so")
REF_LIB_PATH = os.path.join(_HERE, "_ref", "libmind_ref.so")
REF_DRIVER_PATH = os.path.join(_HERE, "_ref", "xnode_driver")

_lib = None
_ref = None


def build(ref_dir: str | None = None) -> None:
    """Compile ``liboracle.so`` (and ``_ref/`` when a reference checkout is present)."""
    cmd = ["make", "-C", _HERE]
    if ref_dir:
        cmd.append(f"REF={ref_dir}")
    subprocess.run(cmd, check=True, stdout=subprocess.DEVNULL)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        L = C.CDLL(LIB_PATH)
        p, i64 = C.c_void_p, C.c_int64
        L.oracle_lcg_fill_q16.argtypes = [C.POINTER(C.c_uint64), p, i64, C.c_int]
        L.oracle_lcg_fill_i8.argtypes = [C.POINTER(C.c_uint64), p, i64]
        L.oracle_lcg_fill_i16.argtypes = [C.POINTER(C.c_uint64), p, i64]
        for name in ("oracle_gemm_i8", "oracle_gemm_q16", "oracle_gemm_q16_bt", "oracle_gemm_i16"):
            getattr(L, name).argtypes = [p, p, p, i64, i64, i64]
            getattr(L, name).restype = None
        for name in ("oracle_gemv_q16", "oracle_gemv_i16"):
            getattr(L, name).argtypes = [p, p, p, i64, i64]
            getattr(L, name).restype = None
        for name in ("oracle_dot_q16", "oracle_dot_l1_q16", "oracle_dot_i16"):
            getattr(L, name).argtypes = [p, p, i64]
            getattr(L, name).restype = i64
        L.oracle_row_bands.argtypes = [i64, i64, p, p]
        L.oracle_row_bands.restype = i64
        for name in ("baseline_gemm_i8_mt", "baseline_gemm_i8_vnni_mt", "baseline_gemm_q16_mt", "baseline_gemm_i16_mt"):
            getattr(L, name).argtypes = [p, p, p, i64, i64, i64, i64]
            getattr(L, name).restype = i64
        for name in ("baseline_gemv_q16_mt", "baseline_gemv_i16_mt"):
            getattr(L, name).argtypes = [p, p, p, i64, i64, i64]
            getattr(L, name).restype = i64
        L.baseline_online_cpus.restype = i64
        L.reference_gemv_q16_mt.argtypes = [p, p, p, p, p, i64, i64]
        L.reference_gemv_q16_mt.restype = i64
        L.reference_gemm_q16_bt_mt.argtypes = [p, p, p, p, p, i64, i64, i64]
        L.reference_gemm_q16_bt_mt.restype = i64
        _lib = L
    return _lib


def ref_lib() -> C.CDLL | None:
    """The reference's own C runtime, or None when it was never built here."""
    global _ref
    if _ref is None and os.path.exists(REF_LIB_PATH):
        R = C.CDLL(REF_LIB_PATH)
        for name in ("__mind_blas_dot_q16", "__mind_blas_dot_l1_q16"):
            getattr(R, name).argtypes = [C.c_int64] * 3
            getattr(R, name).restype = C.c_int64
        R.__mind_blas_set_use_avx2.argtypes = [C.c_int64]
        _ref = R
    return _ref


def _ptr(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


# ------------------------------------------------------------------ generator
class Lcg:
    """The reference's seeded generator; operands drawn one after another share it."""

    def __init__(self, seed: int):
        self._state = C.c_uint64(seed & 0xFFFFFFFFFFFFFFFF)

    def q16(self, n: int, shift: int = 12) -> np.ndarray:
        out = np.empty(n, dtype=np.int32)
        lib().oracle_lcg_fill_q16(C.byref(self._state), _ptr(out), n, shift)
        return out

    def i8(self, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.int8)
        lib().oracle_lcg_fill_i8(C.byref(self._state), _ptr(out), n)
        return out

    def i16(self, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.int16)
        lib().oracle_lcg_fill_i16(C.byref(self._state), _ptr(out), n)
        return out


def lcg_python(seed: int, n: int) -> list[int]:
    """Pure-Python statement of the generator's u32 stream (small n only)."""
    s, out = seed & (2**64 - 1), []
    for _ in range(n):
        s = (s * 1664525 + 1013904223) & (2**64 - 1)
        out.append((s >> 16) & 0xFFFFFFFF)
    return out


# --------------------------------------------------------------------- rules
def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def gemm_i8(a, b, m, k, n):
    a, b = _c(a, np.int8), _c(b, np.int8)
    c = np.empty(m * n, dtype=np.int32)
    lib().oracle_gemm_i8(_ptr(a), _ptr(b), _ptr(c), m, k, n)
    return c


def gemm_i16(a, b, m, k, n):
    a, b = _c(a, np.int16), _c(b, np.int16)
    c = np.empty(m * n, dtype=np.int32)
    lib().oracle_gemm_i16(_ptr(a), _ptr(b), _ptr(c), m, k, n)
    return c


def gemm_q16(a, b, m, k, n):
    a, b = _c(a, np.int32), _c(b, np.int32)
    c = np.empty(m * n, dtype=np.int32)
    lib().oracle_gemm_q16(_ptr(a), _ptr(b), _ptr(c), m, k, n)
    return c


def gemm_q16_bt(a, bt, m, k, n):
    a, bt = _c(a, np.int32), _c(bt, np.int32)
    c = np.empty(m * n, dtype=np.int32)
    lib().oracle_gemm_q16_bt(_ptr(a), _ptr(bt), _ptr(c), m, k, n)
    return c


def gemv_q16(w, x, rows, cols):
    w, x = _c(w, np.int32), _c(x, np.int32)
    y = np.empty(rows, dtype=np.int32)
    lib().oracle_gemv_q16(_ptr(w), _ptr(x), _ptr(y), rows, cols)
    return y


def gemv_i16(w, x, rows, cols):
    w, x = _c(w, np.int16), _c(x, np.int16)
    y = np.empty(rows, dtype=np.int32)
    lib().oracle_gemv_i16(_ptr(w), _ptr(x), _ptr(y), rows, cols)
    return y


def dot_q16(a, b):
    a, b = _c(a, np.int32), _c(b, np.int32)
    return int(lib().oracle_dot_q16(_ptr(a), _ptr(b), a.size))


def dot_l1_q16(a, b):
    a, b = _c(a, np.int32), _c(b, np.int32)
    return int(lib().oracle_dot_l1_q16(_ptr(a), _ptr(b), a.size))


def dot_i16(a, b):
    a, b = _c(a, np.int16), _c(b, np.int16)
    return int(lib().oracle_dot_i16(_ptr(a), _ptr(b), a.size))


def row_bands(m: int, ncpu: int) -> list[tuple[int, int]]:
    s = np.zeros(256, dtype=np.int64)
    e = np.zeros(256, dtype=np.int64)
    used = lib().oracle_row_bands(m, ncpu, _ptr(s), _ptr(e))
    return [(int(s[i]), int(e[i])) for i in range(used)]


# ----------------------------------------------------------------- the hash
def canonical_hash_i32(v: np.ndarray) -> str:
    """sha256 of the i32 little-endian bytes in row-major order
    (tests/cross_substrate_identity.rs:804-810 of the reference)."""
    return hashlib.sha256(np.ascontiguousarray(v, dtype="<i4").tobytes()).hexdigest()


def canonical_hash_i64_scalar(v: int) -> str:
    """sha256 of one i64, little-endian (the dot workloads' encoding)."""
    return hashlib.sha256(int(v).to_bytes(8, "little", signed=True)).hexdigest()


# ------------------------------------------------------ pure-numpy restatement
def gemm_q16_numpy(a, b, m, k, n):
    """Independent numpy statement of the Q16.16 GEMM rule (small shapes)."""
    a64 = np.asarray(a, dtype=np.int64).reshape(m, k)
    b64 = np.asarray(b, dtype=np.int64).reshape(k, n)
    acc = np.zeros((m, n), dtype=np.int64)
    for kk in range(k):
        acc += (a64[:, kk : kk + 1] * b64[kk : kk + 1, :]) >> 16
    return acc.astype(np.int32).reshape(-1)


def gemm_int_numpy(a, b, m, k, n):
    """Independent numpy statement of the shift-free (i8 / i16) GEMM rule."""
    a64 = np.asarray(a, dtype=np.int64).reshape(m, k)
    b64 = np.asarray(b, dtype=np.int64).reshape(k, n)
    return (a64 @ b64).astype(np.int32).reshape(-1)


# ------------------------------------------------------------- timing ports
def baseline_gemm_i8(a, b, m, k, n, threads=0):
    c = np.empty(m * n, dtype=np.int32)
    used = lib().baseline_gemm_i8_mt(_ptr(a), _ptr(b), _ptr(c), m, k, n, threads)
    return c, int(used)


def have_vnni() -> bool:
    """True when the host CPU can run the reference's opt-in vpdpbusd rung."""
    f = lib().baseline_have_vnni
    f.restype = C.c_int64
    return bool(f())


def baseline_gemm_i8_vnni(a, b, m, k, n, threads=0):
    c = np.empty(m * n, dtype=np.int32)
    used = lib().baseline_gemm_i8_vnni_mt(_ptr(a), _ptr(b), _ptr(c), m, k, n, threads)
    if used < 0:
        raise RuntimeError("this CPU has no AVX-512 VNNI")
    return c, int(used)


def baseline_gemm_q16(a, b, m, k, n, threads=0):
    c = np.empty(m * n, dtype=np.int32)
    used = lib().baseline_gemm_q16_mt(_ptr(a), _ptr(b), _ptr(c), m, k, n, threads)
    return c, int(used)


def baseline_gemm_i16(a, b, m, k, n, threads=0):
    c = np.empty(m * n, dtype=np.int32)
    used = lib().baseline_gemm_i16_mt(_ptr(a), _ptr(b), _ptr(c), m, k, n, threads)
    return c, int(used)


def baseline_gemv_q16(w, x, rows, cols, threads=0):
    y = np.empty(rows, dtype=np.int32)
    used = lib().baseline_gemv_q16_mt(_ptr(w), _ptr(x), _ptr(y), rows, cols, threads)
    return y, int(used)


def baseline_gemv_i16(w, x, rows, cols, threads=0):
    y = np.empty(rows, dtype=np.int32)
    used = lib().baseline_gemv_i16_mt(_ptr(w), _ptr(x), _ptr(y), rows, cols, threads)
    return y, int(used)


def _ref_fns():
    R = ref_lib()
    if R is None:
        raise RuntimeError("oracle/_ref/libmind_ref.so was not built")
    return (C.cast(R.__mind_blas_dot_q16, C.c_void_p), C.cast(R.__mind_blas_mt_dispatch, C.c_void_p))


def reference_gemv_q16(w, x, rows, cols):
    """GEMV by the reference's own C dot and thread pool (see cpu_baseline.c)."""
    dot, disp = _ref_fns()
    y = np.empty(rows, dtype=np.int32)
    used = lib().reference_gemv_q16_mt(dot, disp, _ptr(w), _ptr(x), _ptr(y), rows, cols)
    return y, int(used)


def reference_gemm_q16_bt(a, bt, m, k, n):
    """Q16.16 GEMM as row dots over B-transposed, by the reference's own C dot and pool."""
    dot, disp = _ref_fns()
    c = np.empty(m * n, dtype=np.int32)
    used = lib().reference_gemm_q16_bt_mt(dot, disp, _ptr(a), _ptr(bt), _ptr(c), m, k, n)
    return c, int(used)


def online_cpus() -> int:
    return int(lib().baseline_online_cpus())
