"""The CPU oracle against the reference's committed golden hashes, the reference's own C
runtime (when it was built), an independent numpy statement, and the timing ports."""
import json
import os

import numpy as np
import pytest

import oracle as O

HERE = os.path.dirname(os.path.abspath(__file__))
REF = json.load(open(os.path.join(HERE, "golden", "reference_hashes.json")))
SELF = json.load(open(os.path.join(HERE, "golden", "oracle_hashes.json")))
SEED = 0xDEADBEEF


def _hashes(workload):
    entry = REF[workload]
    assert entry["input"]["seed"] == SEED
    vals = set(entry["hashes"].values())
    assert len(vals) == 1, "the reference pins one hash for every substrate"
    return vals.pop()


def test_lcg_matches_pure_python_statement():
    u = O.lcg_python(SEED, 64)
    g = O.Lcg(SEED)
    q = g.q16(64)
    assert [int(np.int32(np.uint32(x))) >> 12 for x in u] == q.tolist()
    g = O.Lcg(SEED)
    assert [int(np.int8(np.uint8((x >> 16) & 0xFF))) for x in u] == g.i8(64).tolist()
    g = O.Lcg(SEED)
    assert [int(np.int16(np.uint16((x >> 16) & 0xFFFF))) for x in u] == g.i16(64).tolist()


@pytest.mark.parametrize("w", ["gemm-i8-64x64x64", "gemm-i8-mt-64x64x64", "gemm-i8-vnni-64x64x64"])
def test_golden_gemm_i8(w):
    g = O.Lcg(SEED)
    a, b = g.i8(64 * 64), g.i8(64 * 64)
    assert O.canonical_hash_i32(O.gemm_i8(a, b, 64, 64, 64)) == _hashes(w)


@pytest.mark.parametrize("w", ["gemm-q16-64x64x64", "gemm-q16-fused-64x64x64"])
def test_golden_gemm_q16(w):
    g = O.Lcg(SEED)
    a, b = g.q16(64 * 64), g.q16(64 * 64)
    assert O.canonical_hash_i32(O.gemm_q16(a, b, 64, 64, 64)) == _hashes(w)
    bt = np.ascontiguousarray(b.reshape(64, 64).T).reshape(-1)
    assert O.canonical_hash_i32(O.gemm_q16_bt(a, bt, 64, 64, 64)) == _hashes(w)


def test_golden_gemv_q16():
    g = O.Lcg(SEED)
    w, x = g.q16(256 * 256), g.q16(256)
    assert O.canonical_hash_i32(O.gemv_q16(w, x, 256, 256)) == _hashes("gemv-q16-256x256")


def test_golden_gemv_i16():
    g = O.Lcg(SEED)
    w, x = g.i16(256 * 256), g.i16(256)
    assert O.canonical_hash_i32(O.gemv_i16(w, x, 256, 256)) == _hashes("gemv-i16-256x256")


def test_golden_dots():
    g = O.Lcg(SEED)
    a, b = g.q16(65536), g.q16(65536)
    assert O.canonical_hash_i64_scalar(O.dot_q16(a, b)) == _hashes("dot-l2-q16")
    assert O.canonical_hash_i64_scalar(O.dot_l1_q16(a, b)) == _hashes("dot-l1-q16")
    g = O.Lcg(SEED)
    a, b = g.i16(4096), g.i16(4096)
    assert O.canonical_hash_i64_scalar(O.dot_i16(a, b)) == _hashes("dot-i16-4096")


@pytest.mark.skipif(O.ref_lib() is None, reason="the reference's C runtime was not built here")
@pytest.mark.parametrize("n", [0, 1, 2, 7, 8, 9, 15, 16, 17, 31, 32, 33, 1024, 4096, 65537])
def test_against_reference_c_runtime(n):
    """Lengths of the reference's own smoke test (tests/blas_vec_q16_smoke.rs:96)."""
    R = O.ref_lib()
    g = O.Lcg(0x1234 + n)
    a, b = g.q16(n, 0), g.q16(n, 0)  # full-range i32: sums overflow 2^31, pinning wrap
    a12, b12 = a >> 12, b >> 12     # the reference generator's own value range
    for avx2 in (0, 1):
        R.__mind_blas_set_use_avx2(avx2)
        assert R.__mind_blas_dot_q16(a.ctypes.data, b.ctypes.data, n) == O.dot_q16(a, b)
        assert R.__mind_blas_dot_l1_q16(a12.ctypes.data, b12.ctypes.data, n) == O.dot_l1_q16(a12, b12)
    # On full-range operands the reference's AVX2 L1 path subtracts in 32 bits and departs
    # from its own scalar oracle (|a-b| >= 2^31); the scalar rule, which its compiler-emitted
    # kernel documents as normative (src/mlir/lowering.rs:6035-6055), is the one restated.
    R.__mind_blas_set_use_avx2(0)
    assert R.__mind_blas_dot_l1_q16(a.ctypes.data, b.ctypes.data, n) == O.dot_l1_q16(a, b)
    R.__mind_blas_set_use_avx2(1)


def test_numpy_statement_agrees():
    g = O.Lcg(99)
    m, k, n = 9, 33, 17
    a, b = g.q16(m * k, 0), g.q16(k * n, 0)
    assert np.array_equal(O.gemm_q16(a, b, m, k, n), O.gemm_q16_numpy(a, b, m, k, n))
    a, b = g.i16(m * k), g.i16(k * n)
    assert np.array_equal(O.gemm_i16(a, b, m, k, n), O.gemm_int_numpy(a, b, m, k, n))
    a, b = g.i8(m * k), g.i8(k * n)
    assert np.array_equal(O.gemm_i8(a, b, m, k, n), O.gemm_int_numpy(a, b, m, k, n))


def test_wrap_not_saturate():
    """Full-range operands push the sums past 2^31: the committed hash pins wrap."""
    e = SELF["gemm-q16-64x64x64-shift0-wrap"]
    g = O.Lcg(e["seed"])
    a, b = g.q16(64 * 64, 0), g.q16(64 * 64, 0)
    c = O.gemm_q16(a, b, 64, 64, 64)
    assert O.canonical_hash_i32(c) == e["sha256"]
    exact = np.zeros((64, 64), dtype=object)
    a2, b2 = a.reshape(64, 64).astype(object), b.reshape(64, 64).astype(object)
    for kk in range(64):
        exact += np.array([[(int(x) * int(y)) >> 16 for y in b2[kk]] for x in a2[:, kk]], dtype=object)
    assert max(abs(int(v)) for v in exact.reshape(-1)) > 2**31
    wrapped = [((int(v) + 2**31) % 2**32) - 2**31 for v in exact.reshape(-1)]
    assert wrapped == c.tolist()


def test_self_generated_fixtures():
    e = SELF["gemm-i8-256x256x256"]
    g = O.Lcg(e["seed"])
    a, b = g.i8(256 * 256), g.i8(256 * 256)
    assert O.canonical_hash_i32(O.gemm_i8(a, b, 256, 256, 256)) == e["sha256"]
    e = SELF["gemv-q16-512x130"]
    g = O.Lcg(e["seed"])
    w, x = g.q16(512 * 130), g.q16(130)
    assert O.canonical_hash_i32(O.gemv_q16(w, x, 512, 130)) == e["sha256"]
    # the workload names of the reference's reproducibility harness (no hash committed upstream yet)
    for n in (32, 256):
        e = SELF[f"matmul-q16-{n}"]
        g = O.Lcg(e["seed"])
        a, b = g.q16(n * n, e["shift"]), g.q16(n * n, e["shift"])
        assert O.canonical_hash_i32(O.gemm_q16(a, b, n, n, n)) == e["sha256"]


@pytest.mark.parametrize("m,k,n,threads", [(1, 1, 1, 1), (37, 130, 75, 3), (130, 513, 129, 8), (5, 0, 7, 2)])
def test_timing_ports_match_oracle(m, k, n, threads):
    g = O.Lcg(m * 1000 + k)
    a, b = g.i8(m * k), g.i8(k * n)
    assert np.array_equal(O.baseline_gemm_i8(a, b, m, k, n, threads)[0], O.gemm_i8(a, b, m, k, n))
    a, b = g.q16(m * k, 0), g.q16(k * n, 0)
    assert np.array_equal(O.baseline_gemm_q16(a, b, m, k, n, threads)[0], O.gemm_q16(a, b, m, k, n))
    assert np.array_equal(O.baseline_gemv_q16(a, b[:k], m, k, threads)[0], O.gemv_q16(a, b[:k], m, k))
    a, b = g.i16(m * k), g.i16(k * n)
    assert np.array_equal(O.baseline_gemm_i16(a, b, m, k, n, threads)[0], O.gemm_i16(a, b, m, k, n))
    assert np.array_equal(O.baseline_gemv_i16(a, b[:k], m, k, threads)[0], O.gemv_i16(a, b[:k], m, k))


def test_row_band_rule():
    """T = max(1, min(ncpu, M, 256)), band = ceil(M/T) (src/mlir/lowering.rs:10146-10205)."""
    assert O.row_bands(10, 4) == [(0, 3), (3, 6), (6, 9), (9, 10)]
    assert O.row_bands(3, 8) == [(0, 1), (1, 2), (2, 3)]
    assert O.row_bands(1000, 1000)[-1][1] == 1000 and len(O.row_bands(1000, 1000)) <= 256
    assert O.row_bands(0, 4) == []


@pytest.mark.skipif(O.ref_lib() is None, reason="the reference's C runtime was not built here")
def test_reference_driven_baseline_matches_oracle():
    """The timed Q16.16 CPU baseline (the reference's own dot + thread pool) gives the oracle's bytes."""
    g = O.Lcg(77)
    rows, cols = 301, 1030
    w, x = g.q16(rows * cols), g.q16(cols)
    y, used = O.reference_gemv_q16(w, x, rows, cols)
    assert used >= 1 and np.array_equal(y, O.gemv_q16(w, x, rows, cols))
    m, k, n = 37, 130, 75
    a, b = g.q16(m * k, 0), g.q16(k * n, 0)
    bt = np.ascontiguousarray(b.reshape(k, n).T).reshape(-1)
    c, _ = O.reference_gemm_q16_bt(a, bt, m, k, n)
    assert np.array_equal(c, O.gemm_q16(a, b, m, k, n))
