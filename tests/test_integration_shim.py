"""integration/mind_b200_native.c: the C file a MIND project lists under
`[targets.*].native_sources` so that its `func.call @__mind_blas_*` resolve to libmind_b200.so.

Compiled here with gcc exactly as a C source with no special flags (mindc compiles it with its
own clang invocation and links `-ldl -lpthread -lm`, src/project/link.rs:113-115 of the
reference), loaded, and called through: argument checks and the no-GPU refusal on CPU, parity
with the oracle on a GPU."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

import mind_b200
import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "integration", "mind_b200_native.c")

CHILD = r"""
import ctypes as C, os, sys
import numpy as np
sys.path.insert(0, %(root)r)
import oracle as O
L = C.CDLL(%(shim)r)
i64 = C.c_int64
f = L.__mind_blas_matmul_mm_i8_v
f.argtypes, f.restype = [i64] * 6, i64
L.mind_b200_native_last_error.restype = C.c_char_p
mode = sys.argv[1]
a = np.zeros(16, dtype=np.int8); c = np.zeros(16, dtype=np.int32)
if mode == "missing":
    assert f(a.ctypes.data, a.ctypes.data, c.ctypes.data, 4, 4, 4) == -3
    assert b"cannot load" in L.mind_b200_native_last_error()
    d = L.__mind_blas_dot_q16_v; d.argtypes, d.restype = [i64] * 3, i64
    assert d(a.ctypes.data, a.ctypes.data, 4) == 0
elif mode == "cpu":
    assert f(a.ctypes.data, a.ctypes.data, c.ctypes.data, 0, 4, 4) == 0      # empty: nothing to do
    assert f(a.ctypes.data, a.ctypes.data, c.ctypes.data, -1, 4, 4) == -1    # the library's own check
    assert b"negative" in L.mind_b200_native_last_error()
    rc = f(a.ctypes.data, a.ctypes.data, c.ctypes.data, 4, 4, 4)
    assert rc in (0, -3), rc                                                # -3: no B200 here, no fallback
else:
    g = O.Lcg(0xDEADBEEF)
    m, k, n = 96, 80, 72
    a8, b8 = g.i8(m * k), g.i8(k * n)
    c = np.empty(m * n, dtype=np.int32)
    assert f(a8.ctypes.data, b8.ctypes.data, c.ctypes.data, m, k, n) == 0
    assert np.array_equal(c, O.gemm_i8(a8, b8, m, k, n))
    aq, bq = g.q16(m * k), g.q16(k * n)
    q = L.__mind_blas_matmul_mm_q16_mt_v; q.argtypes, q.restype = [i64] * 6, i64
    assert q(aq.ctypes.data, bq.ctypes.data, c.ctypes.data, m, k, n) == 0
    assert np.array_equal(c, O.gemm_q16(aq, bq, m, k, n))
    v = L.__mind_blas_gemv_q16_mt; v.argtypes, v.restype = [i64] * 5, i64
    y = np.empty(m, dtype=np.int32)
    assert v(aq.ctypes.data, bq.ctypes.data, y.ctypes.data, m, k) == 0
    assert np.array_equal(y, O.gemv_q16(aq, bq[:k], m, k))
    d = L.__mind_blas_dot_q16_v; d.argtypes, d.restype = [i64] * 3, i64
    assert d(aq.ctypes.data, bq.ctypes.data, k) == O.dot_q16(aq[:k], bq[:k])
print("ok")
"""


@pytest.fixture(scope="module")
def shim(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("shim") / "libmind_b200_native.so")
    subprocess.run(["gcc", "-O2", "-Wall", "-Wextra", "-Werror", "-fPIC", "-shared", "-o", out, SRC,
                    "-ldl", "-lpthread", "-lm"], check=True)
    return out


def run_child(shim, mode, lib_path):
    env = dict(os.environ, MIND_B200_LIB=lib_path)
    return subprocess.run([sys.executable, "-c", CHILD % {"root": ROOT, "shim": shim}, mode],
                          capture_output=True, text=True, env=env, timeout=600)


def test_shim_defines_the_intrinsic_surface(shim):
    L = C.CDLL(shim)
    for name in ("__mind_blas_matmul_mm_i8_v", "__mind_blas_matmul_mm_i8_mt_v", "__mind_blas_matmul_mm_q16_v",
                 "__mind_blas_matmul_mm_q16_mt_v", "__mind_blas_gemv_q16_mt", "__mind_blas_matmul_rmajor_q16_v",
                 "__mind_blas_matmul_rmajor_i16_v", "__mind_blas_dot_q16_v", "__mind_blas_dot_l1_q16_v",
                 "__mind_blas_dot_i16_v", "__mind_b200_matmul_mm_i16"):
        assert hasattr(L, name), name


def test_mind_toml_fragment_uses_only_keys_the_reference_parses():
    text = open(os.path.join(ROOT, "integration", "Mind.toml.fragment")).read()
    keys = re.findall(r"^(\w+)\s*=", text, flags=re.M)
    # TargetConfig, src/project/mod.rs:505-554 of the reference
    assert set(keys) <= {"backend", "simd", "compute", "arch", "output", "sources", "native_sources", "target"}
    assert "backend" in keys and "native_sources" in keys


def test_shim_reports_a_missing_library(shim):
    r = run_child(shim, "missing", "/nonexistent/libmind_b200.so")
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr


def test_shim_forwards_argument_checks_and_refusal(shim):
    r = run_child(shim, "cpu", mind_b200.LIB_PATH)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_shim_parity_on_gpu(shim, gpu):
    r = run_child(shim, "gpu", mind_b200.LIB_PATH)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr
