"""The C-ABI library loads and exports every symbol include/mind_b200.h declares; without
a GPU the compute entry points refuse cleanly (no CPU fallback, no abort)."""
import ctypes as C
import re

import numpy as np
import pytest

import mind_b200
from mind_b200 import blas


def declared_symbols():
    text = open(mind_b200.HEADER_PATH).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"^\s*(?:const\s+char\s*\*|int64_t)\s+(\w+)\s*\(", text, flags=re.M)


def test_header_declares_the_reference_surface():
    names = declared_symbols()
    for required in ("__mind_blas_matmul_mm_i8_v", "__mind_blas_matmul_mm_i8_mt_v",
                     "__mind_blas_matmul_mm_q16_v", "__mind_blas_matmul_mm_q16_mt_v",
                     "__mind_blas_gemv_q16_mt", "__mind_blas_matmul_rmajor_q16_v",
                     "__mind_blas_matmul_rmajor_i16_v", "__mind_blas_dot_q16_v",
                     "__mind_blas_dot_i16_v", "__mind_blas_dot_l1_q16_v",
                     "__mind_b200_matmul_mm_i16",
                     # what the reference's xnode_driver.c dlsym()s:
                     "dotq", "dotl1q", "mmq", "mmi16", "gemmq", "gemmi8"):
        assert required in names


def test_library_exports_every_declared_symbol():
    L = C.CDLL(mind_b200.LIB_PATH)
    missing = [n for n in declared_symbols() if not hasattr(L, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_product_package_does_not_touch_the_oracle():
    import os
    pkg = os.path.dirname(mind_b200.__file__)
    for root, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(root, f)).read()
                assert "import oracle" not in text and "liboracle" not in text, f


def test_no_gpu_means_a_clean_refusal():
    if blas.device_count() > 0:
        pytest.skip("a B200 is present; the refusal path is for machines without one")
    a = np.zeros(16, dtype=np.int8)
    c = np.zeros(16, dtype=np.int32)
    with pytest.raises(mind_b200.MindB200Error) as e:
        blas.matmul_mm_i8_v(a, a, c, 4, 4, 4)
    assert e.value.code == mind_b200.ERR_NO_DEVICE
    assert "no CPU fallback" in str(e.value) or "fallback" in str(e.value)


def test_argument_checks_need_no_gpu():
    a = np.zeros(16, dtype=np.int8)
    c = np.zeros(16, dtype=np.int32)
    with pytest.raises(mind_b200.MindB200Error) as e:
        blas.matmul_mm_i8_v(a, a, c, -1, 4, 4)
    assert e.value.code == mind_b200.ERR_INVALID
    # empty output: nothing to do, success, as in the reference (M <= 0 writes nothing)
    assert blas.matmul_mm_i8_v(a, a, c, 0, 4, 4) == 0
    assert blas.gemv_q16_mt(0, 0, 0, 0, 5) == 0
    # the reference's dot returns 0 for null / empty input
    assert blas.dot_q16_v(0, 0, 10) == 0
    assert blas.dot_q16_v(a, a, 0) == 0
