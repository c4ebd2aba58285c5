"""Parity of the CUDA path with the CPU oracle, through the C ABI, on a real B200.

Integer work: every comparison is bit-exact (np.array_equal / sha256 equality)."""
import json
import os
import subprocess

import numpy as np
import pytest

import oracle as O

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
REF = json.load(open(os.path.join(HERE, "golden", "reference_hashes.json")))
SELF = json.load(open(os.path.join(HERE, "golden", "oracle_hashes.json")))
SEED = 0xDEADBEEF


def ref_hash(w):
    return next(iter(REF[w]["hashes"].values()))


# Tile edges of the GPU kernels (128 / 256 rows, 128-byte K slabs, 16-byte pitches).
GEMM_SHAPES = [
    (1, 1, 1), (1, 16, 1), (7, 15, 7), (63, 17, 65), (64, 64, 64), (65, 31, 63),
    (127, 32, 129), (128, 128, 256), (129, 33, 255), (255, 127, 257), (256, 129, 128),
    (257, 130, 1), (1, 511, 257), (130, 513, 70), (128, 1, 256), (300, 256, 520),
    (5, 0, 9), (384, 1024, 512), (100, 2048, 36),
    # few tiles, long K: every tile's K range is split across SMs and summed with atomics
    (64, 4096, 64), (130, 3000, 40), (257, 1100, 300), (16, 16384, 16),
]
PATHS = [3, 2, 1, 0, 4, 5]  # single CTA, CTA pairs, CUDA cores, auto, pairs / single with B transposed first
PATHS_I8 = PATHS + [10, 12]  # int8 only: the narrow-tile kernel / the 256 x 512-tile pair kernel at every shape


@pytest.fixture(autouse=True)
def _default_path(gpu):
    gpu.set_gemm_path(0)
    yield
    gpu.set_gemm_path(0)


# --------------------------------------------------------------- golden vectors
def test_golden_gemm_i8_all_paths(gpu):
    g = O.Lcg(SEED)
    a, b = g.i8(64 * 64), g.i8(64 * 64)
    for path in PATHS_I8:
        gpu.set_gemm_path(path)
        for fn in (gpu.matmul_mm_i8_v, gpu.matmul_mm_i8_mt_v):
            c = np.full(64 * 64, -1, dtype=np.int32)
            assert fn(a, b, c, 64, 64, 64) == 0
            assert O.canonical_hash_i32(c) == ref_hash("gemm-i8-64x64x64"), path


def test_golden_gemm_q16(gpu):
    g = O.Lcg(SEED)
    a, b = g.q16(64 * 64), g.q16(64 * 64)
    for fn in (gpu.matmul_mm_q16_v, gpu.matmul_mm_q16_mt_v):
        c = np.full(64 * 64, -1, dtype=np.int32)
        fn(a, b, c, 64, 64, 64)
        assert O.canonical_hash_i32(c) == ref_hash("gemm-q16-fused-64x64x64")
    bt = np.ascontiguousarray(b.reshape(64, 64).T).reshape(-1)
    c = np.full(64 * 64, -1, dtype=np.int32)
    gpu.gemmq_bt(a, bt, c, 64, 64, 64)
    assert O.canonical_hash_i32(c) == ref_hash("gemm-q16-64x64x64")


def test_golden_gemv_and_dots(gpu):
    g = O.Lcg(SEED)
    w, x = g.q16(256 * 256), g.q16(256)
    for fn in (gpu.gemv_q16_mt, gpu.matmul_rmajor_q16_v):
        y = np.full(256, -1, dtype=np.int32)
        fn(w, x, y, 256, 256)
        assert O.canonical_hash_i32(y) == ref_hash("gemv-q16-256x256")
    g = O.Lcg(SEED)
    w, x = g.i16(256 * 256), g.i16(256)
    y = np.full(256, -1, dtype=np.int32)
    gpu.matmul_rmajor_i16_v(w, x, y, 256, 256)
    assert O.canonical_hash_i32(y) == ref_hash("gemv-i16-256x256")
    g = O.Lcg(SEED)
    a, b = g.q16(65536), g.q16(65536)
    assert O.canonical_hash_i64_scalar(gpu.dot_q16_v(a, b, 65536)) == ref_hash("dot-l2-q16")
    assert O.canonical_hash_i64_scalar(gpu.dot_l1_q16_v(a, b, 65536)) == ref_hash("dot-l1-q16")
    g = O.Lcg(SEED)
    a, b = g.i16(4096), g.i16(4096)
    assert O.canonical_hash_i64_scalar(gpu.dot_i16_v(a, b, 4096)) == ref_hash("dot-i16-4096")


def test_reference_xnode_driver_runs_unmodified(gpu):
    """The reference's own C driver (compiled from its sources) against this library."""
    if not os.path.exists(O.REF_DRIVER_PATH):
        pytest.skip("oracle/_ref/xnode_driver was not built (no reference checkout at build time)")
    import mind_b200
    r = subprocess.run([O.REF_DRIVER_PATH, mind_b200.LIB_PATH, "b200"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all canaries MATCH" in r.stdout
    out = dict(line.split()[:2] for line in r.stdout.splitlines() if line.startswith("  "))
    for w in ("dot-l2-q16", "dot-l1-q16", "gemv-q16-256x256", "gemv-i16-256x256",
              "gemm-q16-64x64x64", "gemm-i8-64x64x64"):
        assert out[w] == ref_hash(w), w


# ------------------------------------------------------------------ edge shapes
@pytest.mark.parametrize("path", PATHS_I8)
def test_gemm_i8_shapes(gpu, path):
    gpu.set_gemm_path(path)
    for (m, k, n) in GEMM_SHAPES:
        g = O.Lcg(0xDEADBEEF00000000 ^ (m * 1000003 + k * 1009 + n))
        a, b = g.i8(m * k), g.i8(k * n)
        c = np.full(m * n + 8, 0x5A5A5A5A, dtype=np.int32)  # canary after the output
        gpu.matmul_mm_i8_v(a, b, c, m, k, n)
        assert np.array_equal(c[: m * n], O.gemm_i8(a, b, m, k, n)), (path, m, k, n)
        assert np.all(c[m * n :] == 0x5A5A5A5A), (path, m, k, n)


@pytest.mark.parametrize("path", [0, 2, 3, 4])
def test_gemm_i8_host_operand_pipeline(gpu, path):
    """M >= 1024 with host A and / or C: row bands are uploaded, multiplied and downloaded
    in overlap.  Ragged last band, K % 16 != 0 (padded on upload), N % 16 != 0."""
    import torch
    gpu.set_gemm_path(path)
    # the last four shapes also split N into 4 / 8 column chunks on the way back to the host
    for (m, k, n) in [(1024, 64, 48), (2500, 100, 36), (1300, 256, 512), (4097, 33, 257), (8192, 512, 128),
                      (1024, 64, 4096), (1100, 48, 4160), (1024, 32, 8192), (1030, 16, 8320)]:
        g = O.Lcg(0xDEADBEEF00000000 ^ (m * 7 + k * 3 + n))
        a, b = g.i8(m * k), g.i8(k * n)
        want = O.gemm_i8(a, b, m, k, n)
        c = np.full(m * n + 8, 0x5A5A5A5A, dtype=np.int32)
        gpu.matmul_mm_i8_v(a, b, c, m, k, n)  # all host
        assert np.array_equal(c[: m * n], want), (path, m, k, n)
        assert np.all(c[m * n:] == 0x5A5A5A5A)
        ad, bd = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        c2 = np.zeros(m * n, dtype=np.int32)
        gpu.matmul_mm_i8_v(ad, bd, c2, m, k, n)  # device A and B, host C
        assert np.array_equal(c2, want), (path, m, k, n)
        cd = torch.zeros(m * n, dtype=torch.int32, device="cuda")
        gpu.matmul_mm_i8_v(a, bd, cd, m, k, n)  # host A, device C
        gpu.synchronize()
        assert np.array_equal(cd.cpu().numpy(), want), (path, m, k, n)


@pytest.mark.parametrize("path", PATHS)
def test_gemm_i16_shapes(gpu, path):
    gpu.set_gemm_path(path)
    for (m, k, n) in GEMM_SHAPES:
        g = O.Lcg(0xDEADBEEF00000000 ^ (m * 1000003 + k * 1009 + n + 1))
        a, b = g.i16(m * k), g.i16(k * n)  # full range: sums wrap for k >= 2
        c = np.full(m * n + 8, 0x5A5A5A5A, dtype=np.int32)
        gpu.matmul_mm_i16(a, b, c, m, k, n)
        assert np.array_equal(c[: m * n], O.gemm_i16(a, b, m, k, n)), (path, m, k, n)
        assert np.all(c[m * n :] == 0x5A5A5A5A)


# 0: by size; 1: all-integer kernel; 6: FP64-pipe kernel alone; 7: tensor-core linear part + the floor
# term on the FP32 pipe (8: one after the other, 9: side by side on two streams, both adding onto C);
# 14: the hybrid with the floor term on the FP64 pipe
Q16_PATHS = [0, 1, 6, 7, 8, 9, 14]


@pytest.mark.parametrize("path", Q16_PATHS)
def test_gemm_q16_shapes(gpu, path):
    gpu.set_gemm_path(path)
    # the last shape has a long K on a single output tile: many blocks add into the same outputs
    for (m, k, n) in GEMM_SHAPES + [(256, 64, 128), (1024, 1024, 64), (260, 132, 516), (70, 8200, 68)]:
        for shift in (12, 0):  # the reference's range, and full range (wrap past 2^31)
            g = O.Lcg(0xDEADBEEF00000000 ^ (m * 1000003 + k * 1009 + n + 2))
            a, b = g.q16(m * k, shift), g.q16(k * n, shift)
            c = np.full(m * n + 8, 0x5A5A5A5A, dtype=np.int32)
            gpu.matmul_mm_q16_v(a, b, c, m, k, n)
            assert np.array_equal(c[: m * n], O.gemm_q16(a, b, m, k, n)), (m, k, n, shift)
            assert np.all(c[m * n :] == 0x5A5A5A5A)


def test_random_shapes_all_kernels(gpu):
    """Forty seeded random shapes per kernel family (ragged in every dimension), default paths."""
    rng = np.random.default_rng(20260101)
    for t in range(40):
        m, k, n = (int(v) for v in rng.integers(1, 400, size=3))
        if t % 5 == 0:
            k = int(rng.integers(1, 40)) * 16       # aligned K: A is read in place
        if t % 7 == 0:
            n = int(rng.integers(1, 30)) * 16       # aligned N: B is read in place
        g = O.Lcg(int(rng.integers(1, 2**62)))
        a, b = g.i8(m * k), g.i8(k * n)
        c = np.empty(m * n, dtype=np.int32)
        gpu.matmul_mm_i8_v(a, b, c, m, k, n)
        assert np.array_equal(c, O.gemm_i8(a, b, m, k, n)), ("i8", m, k, n)
        a, b = g.i16(m * k), g.i16(k * n)
        gpu.matmul_mm_i16(a, b, c, m, k, n)
        assert np.array_equal(c, O.gemm_i16(a, b, m, k, n)), ("i16", m, k, n)
        a, b = g.q16(m * k, 0), g.q16(k * n, 0)
        gpu.matmul_mm_q16_v(a, b, c, m, k, n)
        assert np.array_equal(c, O.gemm_q16(a, b, m, k, n)), ("q16", m, k, n)
        y = np.empty(m, dtype=np.int32)
        gpu.gemv_q16_mt(a, b[:k], y, m, k)
        assert np.array_equal(y, O.gemv_q16(a, b[:k], m, k)), ("gemv", m, k)


def test_random_shapes_fused_q16(gpu):
    """Seeded random shapes through the fused Q16.16 kernel (forced at every size): half of them
    with K and N multiples of 4 (16-byte loads, tensor stores), half fully ragged (element-wise
    operand split, the warp's own stores), some with every operand one element off a 16-byte
    boundary; tiles ragged on every side, one to several hundred stream-K units per CTA,
    full-range operands, against the CPU oracle."""
    rng = np.random.default_rng(20260202)
    gpu.set_gemm_path(7)
    try:
        for t in range(20):
            m = int(rng.integers(1, 700))
            k = int(rng.integers(1, 200)) * 4
            n = int(rng.integers(1, 180)) * 4
            if t % 2 == 1:
                k, n = int(rng.integers(1, 800)), int(rng.integers(1, 700))
            if t == 0:
                m, k, n = 129, 36, 132          # a unit and a bit, two tiles and a bit
            if t == 1:
                m, k, n = 1, 1, 1
            g = O.Lcg(int(rng.integers(1, 2**62)))
            off = 1 if t % 4 >= 2 else 0        # operands one element past a 16-byte boundary
            abuf, bbuf = g.q16(m * k + off, 0), g.q16(k * n + off, 0)
            a, b = abuf[off:], bbuf[off:]
            cbuf = np.full(m * n + 8 + off, 0x5A5A5A5A, dtype=np.int32)
            c = cbuf[off:]
            gpu.matmul_mm_q16_v(a, b, c, m, k, n)
            assert np.array_equal(c[: m * n], O.gemm_q16(np.ascontiguousarray(a), np.ascontiguousarray(b), m, k, n)), (m, k, n, off)
            assert np.all(c[m * n :] == 0x5A5A5A5A) and (off == 0 or cbuf[0] == 0x5A5A5A5A)
    finally:
        gpu.set_gemm_path(0)


def test_q16_extreme_values(gpu):
    """INT_MIN / INT_MAX / -1 / 0x7FFF8000...: the hi/lo split must be exact everywhere."""
    specials = np.array([-2**31, 2**31 - 1, -1, 0, 1, 0x7FFF8000, 0x7FFF7FFF, -0x8000, 0x8000,
                         0x7FFF, -0x7FFF, 0xFFFF, -0x10000, 0x10000, -0x7FFF8000, 65535 * 32768],
                        dtype=np.int64).astype(np.int32)
    k = specials.size
    a = np.ascontiguousarray(np.tile(specials, (k, 1)))            # every special in every row
    b = np.ascontiguousarray(np.stack([np.roll(specials, s) for s in range(k)], axis=1))
    c = np.empty(k * k, dtype=np.int32)
    gpu.matmul_mm_q16_v(a.reshape(-1), b.reshape(-1), c, k, k, k)
    assert np.array_equal(c, O.gemm_q16(a.reshape(-1), b.reshape(-1), k, k, k))
    for r in range(k):
        x = np.ascontiguousarray(np.roll(specials, r))
        y = np.empty(1, dtype=np.int32)
        gpu.gemv_q16_mt(specials, x, y, 1, k)
        assert int(y[0]) == O.dot_q16(specials, x)
        assert gpu.dot_q16_v(specials, x, k) == O.dot_q16(specials, x)
        assert gpu.dot_l1_q16_v(specials, x, k) == O.dot_l1_q16(specials, x)


def test_q16_floor_chain_range_and_long_k(gpu):
    """The hybrid's floor kernel adds floor(a * (b & 0xffff) / 65536) to a binary64 chain that is
    exact for 2^20 terms of either sign at full magnitude; longer K is cut into slices.  Drive
    both ends of the range across one slice boundary: a = INT_MIN / INT_MAX with b & 0xffff =
    0xffff for K = 2^20 + 48, several blocks sharing one output tile."""
    m, n, k = 8, 4, (1 << 20) + 48
    gpu.set_gemm_path(14)
    try:
        for aval in (-2**31, 2**31 - 1):
            a = np.full(m * k, aval, dtype=np.int64).astype(np.int32)
            a[:: 7] = 12345                                  # not all equal
            b = np.full(k * n, 0xFFFF, dtype=np.int32)
            b[:: 5] = -1                                     # b >> 16 = -1, low half 0xffff
            c = np.empty(m * n, dtype=np.int32)
            gpu.matmul_mm_q16_v(a, b, c, m, k, n)
            assert np.array_equal(c, O.gemm_q16(a, b, m, k, n)), aval
    finally:
        gpu.set_gemm_path(0)


@pytest.mark.parametrize("path", [7, 8, 9])
def test_q16_f32_chain_holds_128_full_terms(gpu, path):
    """The default hybrid adds floor((a & 0xffff) * (b & 0xffff) / 65536) to binary32 chains that
    start at 2^23 and are emptied every 128 products; a chain is exact only while it stays below
    2^24.  Every product at the largest possible term (both low halves 0xffff, term 65534), every
    sign combination of the high halves, K across several emptyings and not a multiple of 128."""
    m, n, k = 136, 132, 128 * 5 + 20
    gpu.set_gemm_path(path)
    try:
        for aval, bval in ((-1, -1), (0xFFFF, 0xFFFF), (0x7FFFFFFF, -1), (-1, 0x7FFFFFFF), (-0x7FFF0001, 0x7FFFFFFF)):
            a = np.full(m * k, aval, dtype=np.int64).astype(np.int32)
            b = np.full(k * n, bval, dtype=np.int64).astype(np.int32)
            a[:: 257] = 0x1234FFFE                           # not all equal
            b[:: 263] = -0x10000 + 0xFFFE
            c = np.empty(m * n, dtype=np.int32)
            gpu.matmul_mm_q16_v(a, b, c, m, k, n)
            assert np.array_equal(c, O.gemm_q16(a, b, m, k, n)), (aval, bval)
        # a very long K on a single small tile: every CTA of the fused kernel adds its share of the
        # same outputs (tensor reductions), and the chains are emptied 8000 times per output
        m, n, k = 8, 4, (1 << 20) + 48
        a = np.full(m * k, -1, dtype=np.int32)
        a[:: 7] = 0x7FFFFFFF
        b = np.full(k * n, 0xFFFF, dtype=np.int32)
        b[:: 5] = -1
        c = np.empty(m * n, dtype=np.int32)
        gpu.matmul_mm_q16_v(a, b, c, m, k, n)
        assert np.array_equal(c, O.gemm_q16(a, b, m, k, n))
    finally:
        gpu.set_gemm_path(0)


def test_wrap_fixture_and_overflowing_i8(gpu):
    e = SELF["gemm-q16-64x64x64-shift0-wrap"]
    g = O.Lcg(e["seed"])
    a, b = g.q16(64 * 64, 0), g.q16(64 * 64, 0)
    c = np.empty(64 * 64, dtype=np.int32)
    gpu.matmul_mm_q16_v(a, b, c, 64, 64, 64)
    assert O.canonical_hash_i32(c) == e["sha256"]
    # int8: all -128 x -128 with K = 2^17 + 256 sums to 2^31 + 2^22: i32 wraps
    m, k, n = 128, (1 << 17) + 256, 16
    a = np.full(m * k, -128, dtype=np.int8)
    b = np.full(k * n, -128, dtype=np.int8)
    for path in (3, 2, 4, 5, 10, 12):
        gpu.set_gemm_path(path)
        c = np.empty(m * n, dtype=np.int32)
        gpu.matmul_mm_i8_v(a, b, c, m, k, n)
        want = np.int64(16384) * k
        assert np.all(c.astype(np.int64) == ((want + 2**31) % 2**32) - 2**31)
    # unsigned limb products overflow an accumulator too: int16 operands 255 (hi limb 0, lo limb
    # 255) with K = 40000 put 65025 * 40000 > 2^31 into the lo.lo accumulator; same for the
    # byte planes of the Q16.16 hybrid (a = 255, b = 255 << 16)
    m, k, n = 128, 40000, 16
    a16 = np.full(m * k, 255, dtype=np.int16)
    b16 = np.full(k * n, 255, dtype=np.int16)
    want = np.int64(65025) * k
    for path in (3, 2):
        gpu.set_gemm_path(path)
        c = np.empty(m * n, dtype=np.int32)
        gpu.matmul_mm_i16(a16, b16, c, m, k, n)
        assert np.all(c.astype(np.int64) == ((want + 2**31) % 2**32) - 2**31)
    gpu.set_gemm_path(7)
    aq = np.full(m * k, 255, dtype=np.int32)
    bq = np.full(k * n, 255 << 16, dtype=np.int32)
    c = np.empty(m * n, dtype=np.int32)
    gpu.matmul_mm_q16_v(aq, bq, c, m, k, n)
    assert np.array_equal(c, O.gemm_q16(aq, bq, m, k, n))
    assert np.all(c.astype(np.int64) == ((want + 2**31) % 2**32) - 2**31)


@pytest.mark.parametrize("rows,cols", [(1, 1), (2, 3), (4, 4), (8, 16), (16, 9), (3, 65), (512, 130),
                                       (256, 130), (11922, 384), (5, 0), (3, 4096), (1, 65537), (700, 2048)])
def test_gemv_shapes(gpu, rows, cols):
    g = O.Lcg(0xDEADBEEF00000000 ^ ((rows << 20) ^ cols))
    w, x = g.q16(rows * cols), g.q16(cols)
    y = np.full(rows + 4, 0x5A5A5A5A, dtype=np.int32)
    gpu.gemv_q16_mt(w, x, y, rows, cols)
    assert np.array_equal(y[:rows], O.gemv_q16(w, x, rows, cols))
    assert np.all(y[rows:] == 0x5A5A5A5A)
    w, x = g.i16(rows * cols), g.i16(cols)
    y = np.full(rows + 4, 0x5A5A5A5A, dtype=np.int32)
    gpu.matmul_rmajor_i16_v(w, x, y, rows, cols)
    assert np.array_equal(y[:rows], O.gemv_i16(w, x, rows, cols))
    assert np.all(y[rows:] == 0x5A5A5A5A)


def test_gemv_fixture_512x130(gpu):
    e = SELF["gemv-q16-512x130"]
    g = O.Lcg(e["seed"])
    w, x = g.q16(512 * 130), g.q16(130)
    y = np.empty(512, dtype=np.int32)
    gpu.gemv_q16_mt(w, x, y, 512, 130)
    assert O.canonical_hash_i32(y) == e["sha256"]


@pytest.mark.parametrize("n", [1, 2, 7, 8, 9, 15, 16, 17, 31, 32, 33, 1024, 4096, 65537])
def test_dot_lengths(gpu, n):
    """Lengths of the reference's smoke test (tests/blas_vec_q16_smoke.rs:96)."""
    g = O.Lcg(0x1234 + n)
    a, b = g.q16(n, 0), g.q16(n, 0)
    assert gpu.dot_q16_v(a, b, n) == O.dot_q16(a, b)
    assert gpu.dot_l1_q16_v(a, b, n) == O.dot_l1_q16(a, b)
    a, b = g.i16(n), g.i16(n)
    assert gpu.dot_i16_v(a, b, n) == O.dot_i16(a, b)


def test_matmul_row_equals_dot(gpu):
    """tests/blas_vec_q16_smoke.rs:577-624: each matmul row equals the dot of that row."""
    g = O.Lcg(7)
    rows, cols = 9, 133
    w, x = g.q16(rows * cols), g.q16(cols)
    y = np.empty(rows, dtype=np.int32)
    gpu.matmul_rmajor_q16_v(w, x, y, rows, cols)
    for r in range(rows):
        assert int(y[r]) == gpu.dot_q16_v(np.ascontiguousarray(w[r * cols:(r + 1) * cols]), x, cols)


def test_unaligned_operands(gpu):
    """Any element-aligned address is legal input (the reference loads with alignment 1/2/4)."""
    m, k, n = 70, 48, 36
    g = O.Lcg(11)
    for path in PATHS_I8:
        gpu.set_gemm_path(path)
        abuf, bbuf = g.i8(m * k + 3), g.i8(k * n + 5)
        a, b = abuf[3:], bbuf[5:]
        cbuf = np.zeros(m * n + 1, dtype=np.int32)
        gpu.matmul_mm_i8_v(a.ctypes.data, b.ctypes.data, cbuf[1:].ctypes.data, m, k, n)
        assert np.array_equal(cbuf[1:], O.gemm_i8(a.copy(), b.copy(), m, k, n))
        abuf, bbuf = g.i16(m * k + 1), g.i16(k * n + 3)
        a, b = abuf[1:], bbuf[3:]
        gpu.matmul_mm_i16(a.ctypes.data, b.ctypes.data, cbuf[1:].ctypes.data, m, k, n)
        assert np.array_equal(cbuf[1:], O.gemm_i16(a.copy(), b.copy(), m, k, n))
    abuf, bbuf = g.q16(m * k + 1), g.q16(k * n + 3)
    a, b = abuf[1:], bbuf[3:]
    cbuf = np.zeros(m * n + 1, dtype=np.int32)
    gpu.matmul_mm_q16_v(a.ctypes.data, b.ctypes.data, cbuf[1:].ctypes.data, m, k, n)
    assert np.array_equal(cbuf[1:], O.gemm_q16(a.copy(), b.copy(), m, k, n))
    wbuf, xbuf = g.q16(m * k + 1), g.q16(k + 1)
    y = np.zeros(m + 1, dtype=np.int32)
    gpu.gemv_q16_mt(wbuf[1:].ctypes.data, xbuf[1:].ctypes.data, y[1:].ctypes.data, m, k)
    assert np.array_equal(y[1:], O.gemv_q16(wbuf[1:].copy(), xbuf[1:].copy(), m, k))


def test_bounded_wait_gives_up_cleanly(gpu):
    """Every mbarrier wait in the GEMM kernels is bounded.  A one-warp kernel waits on a barrier
    that nothing completes (limit 50 ms): the call must come back with ERR_TIMEOUT, and the
    context must still compute correctly afterwards.  Nothing faults or hangs."""
    import ctypes as C
    import mind_b200
    f = mind_b200.lib().mind_b200_selftest_wait_timeout
    f.argtypes, f.restype = [C.c_int64], C.c_int64
    assert f(50) == mind_b200.ERR_TIMEOUT
    assert "bounded wait" in mind_b200.last_error()
    g = O.Lcg(3)
    a, b = g.i8(256 * 128), g.i8(128 * 256)
    c = np.empty(256 * 256, dtype=np.int32)
    gpu.matmul_mm_i8_v(a, b, c, 256, 128, 256)
    assert np.array_equal(c, O.gemm_i8(a, b, 256, 128, 256))
    assert f(0) == mind_b200.ERR_INVALID


def test_narrow_tile_kernel_is_the_default_for_few_tiles(gpu):
    """Benchmark configuration 1 (int8 256^3, seed rule of benches/det_matmul_i8.rs:431-445) and
    its neighbours run on the 128 x 64-tile kernel by default; B read in place (N % 16 == 0, the
    64-byte-swizzled MN-major tile) and B transposed first (N % 16 != 0) must both give the
    oracle's bytes, and the same bytes as the wide-tile kernel."""
    for (m, k, n) in [(256, 256, 256), (512, 512, 512), (256, 1920, 64), (130, 256, 1008), (256, 256, 250)]:
        g = O.Lcg(0xDEADBEEF00000000 ^ n)
        a, b = g.i8(m * k), g.i8(k * n)
        want = O.gemm_i8(a, b, m, k, n)
        for path in (0, 10, 11):
            gpu.set_gemm_path(path)
            c = np.full(m * n + 8, 0x5A5A5A5A, dtype=np.int32)
            gpu.matmul_mm_i8_v(a, b, c, m, k, n)
            assert np.array_equal(c[: m * n], want), (path, m, k, n)
            assert np.all(c[m * n:] == 0x5A5A5A5A)
    e = SELF.get("gemm-i8-256x256x256")
    if e:
        g = O.Lcg(e["seed"])
        a, b = g.i8(256 * 256), g.i8(256 * 256)
        c = np.empty(256 * 256, dtype=np.int32)
        gpu.set_gemm_path(0)
        gpu.matmul_mm_i8_v(a, b, c, 256, 256, 256)
        assert O.canonical_hash_i32(c) == e["sha256"]


def test_set_stream_orders_the_new_stream_after_the_old(gpu):
    """Device-pointer calls are asynchronous and share one scratch buffer per device.  A call
    that re-lays B out in scratch (N % 16 != 0) is queued on stream A; the library is switched to
    stream B at once, with no host synchronisation, and a second call with another shape rewrites
    the same scratch.  The switch must order B after A: both results equal the oracle."""
    import torch
    torch.cuda.set_device(0)
    sa, sb = torch.cuda.Stream(), torch.cuda.Stream()
    g = O.Lcg(4242)
    m1, k1, n1 = 1500, 2048, 1000   # transposing path, a few hundred microseconds of work
    m2, k2, n2 = 300, 520, 200
    a1, b1 = g.i8(m1 * k1), g.i8(k1 * n1)
    a2, b2 = g.i8(m2 * k2), g.i8(k2 * n2)
    want1, want2 = O.gemm_i8(a1, b1, m1, k1, n1), O.gemm_i8(a2, b2, m2, k2, n2)
    d = lambda x: torch.from_numpy(x).cuda()
    da1, db1, da2, db2 = d(a1), d(b1), d(a2), d(b2)
    torch.cuda.synchronize()
    try:
        for rep in range(4):
            c1 = torch.zeros(m1 * n1, dtype=torch.int32, device="cuda")
            c2 = torch.zeros(m2 * n2, dtype=torch.int32, device="cuda")
            torch.cuda.synchronize()
            gpu.set_stream(sa.cuda_stream)
            gpu.matmul_mm_i8_v(da1, db1, c1, m1, k1, n1)
            gpu.set_stream(sb.cuda_stream)          # no synchronisation in between
            gpu.matmul_mm_i8_v(da2, db2, c2, m2, k2, n2)
            torch.cuda.synchronize()
            assert np.array_equal(c1.cpu().numpy(), want1), rep
            assert np.array_equal(c2.cpu().numpy(), want2), rep
    finally:
        torch.cuda.synchronize()
        gpu.set_stream(torch.cuda.current_stream().cuda_stream)


def test_scratch_growth_keeps_captured_graphs_valid(gpu):
    """A captured graph holds the scratch addresses it was recorded with.  (1) A call that would
    have to grow the scratch while its stream is being captured is refused with a clear error,
    and the capture goes on.  (2) After a capture has been seen, a later, larger call (which
    grows the scratch) must not free the block the graph still uses: the replay is still right."""
    import mind_b200
    import torch
    torch.cuda.set_device(0)
    gpu.shutdown()                               # start from empty scratch, whatever ran before
    gpu.set_stream(torch.cuda.current_stream().cuda_stream)
    side = torch.cuda.Stream()
    g = O.Lcg(99)
    m, k, n = 200, 300, 250                      # N % 16 != 0: B is transposed into scratch
    a, b = g.i8(m * k), g.i8(k * n)
    want = O.gemm_i8(a, b, m, k, n)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    mb, kb, nb = 4000, 5000, 4100                # needs far more scratch than anything before it
    big_a = torch.zeros(mb * kb, dtype=torch.int8, device="cuda")
    big_b = torch.ones(kb * nb, dtype=torch.int8, device="cuda")
    big_c = torch.empty(mb * nb, dtype=torch.int32, device="cuda")
    out = torch.zeros(m * n, dtype=torch.int32, device="cuda")
    graph = torch.cuda.CUDAGraph()
    try:
        with torch.cuda.stream(side):
            gpu.set_stream(side.cuda_stream)
            gpu.matmul_mm_i8_v(da, db, out, m, k, n)     # warm-up: sizes the scratch for this shape
            torch.cuda.synchronize()
            out.zero_()
            with torch.cuda.graph(graph, stream=side):
                gpu.matmul_mm_i8_v(da, db, out, m, k, n)
                with pytest.raises(mind_b200.MindB200Error) as e:
                    gpu.matmul_mm_i8_v(big_a, big_b, big_c, mb, kb, nb)   # would have to grow: refused
                assert e.value.code == mind_b200.ERR_INVALID and "captured" in str(e.value)
        gpu.set_stream(torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), want)
        gpu.matmul_mm_i8_v(big_a, big_b, big_c, mb, kb, nb)               # grows the scratch now
        gpu.synchronize()
        assert int(big_c.abs().max()) == 0
        big_a.fill_(1)                                                     # and overwrite it with other bytes
        gpu.matmul_mm_i8_v(big_a, big_b, big_c, mb, kb, nb)
        gpu.synchronize()
        assert int(big_c.min()) == kb and int(big_c.max()) == kb
        out.zero_()
        graph.replay()                                                     # the old block is still alive
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), want)
    finally:
        torch.cuda.synchronize()
        gpu.set_stream(torch.cuda.current_stream().cuda_stream)


def test_errors_do_not_abort(gpu):
    import mind_b200
    a = np.zeros(16, dtype=np.int8)
    c = np.zeros(16, dtype=np.int32)
    with pytest.raises(mind_b200.MindB200Error) as e:
        gpu.matmul_mm_i8_v(0, a, c, 4, 4, 4)
    assert e.value.code == mind_b200.ERR_INVALID
    with pytest.raises(mind_b200.MindB200Error):
        gpu.matmul_mm_q16_v(a.ctypes.data + 1, a, c, 2, 2, 2)  # misaligned int32
    gpu.matmul_mm_i8_v(a, a, c, 4, 4, 4)  # and the library still works afterwards
    assert np.all(c == 0)


def test_calls_from_several_host_threads(gpu):
    """The reference's intrinsics may be called from any thread (its MT forms take a process-wide
    lock, runtime-support/mind_intrinsics.c:1929 and :1976); here calls are serialised inside the library
    and every thread must get its own exact result, host operands and all kernel families mixed."""
    import threading
    errors = []

    def worker(t):
        try:
            g = O.Lcg(1000 + t)
            for it in range(6):
                m, k, n = 40 + 13 * t + it, 64 + 16 * ((t + it) % 5), 48 + 16 * t
                a8, b8 = g.i8(m * k), g.i8(k * n)
                c = np.empty(m * n, dtype=np.int32)
                gpu.matmul_mm_i8_v(a8, b8, c, m, k, n)
                assert np.array_equal(c, O.gemm_i8(a8, b8, m, k, n)), ("i8", t, it)
                aq, bq = g.q16(m * k), g.q16(k * n)
                gpu.matmul_mm_q16_v(aq, bq, c, m, k, n)
                assert np.array_equal(c, O.gemm_q16(aq, bq, m, k, n)), ("q16", t, it)
                y = np.empty(m, dtype=np.int32)
                gpu.gemv_q16_mt(aq, bq[:k], y, m, k)
                assert np.array_equal(y, O.gemv_q16(aq, bq[:k], m, k)), ("gemv", t, it)
                assert gpu.dot_q16_v(aq[:k], bq[:k], k) == O.dot_q16(aq[:k], bq[:k]), ("dot", t, it)
        except BaseException as ex:  # noqa: BLE001 - reported in the main thread
            errors.append(ex)

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(4)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors


def test_i16_rows_extreme_values(gpu):
    """int16 row reductions split x into bytes for dp2a: every corner of the 16-bit range, in
    every position of a 16-byte vector, vectorised (aligned) and scalar (odd length) paths."""
    specials = np.array([-32768, 32767, -1, 0, 1, 255, 256, -256, -255, 127, 128, -128, -129, 0x7F00, -0x7F00, 0x00FF],
                        dtype=np.int16)
    for cols in (16, 64, 1024, 1037):
        reps = -(-cols // specials.size)
        w = np.stack([np.tile(np.roll(specials, s), reps)[:cols] for s in range(16)]).astype(np.int16)
        for shift in range(16):
            x = np.tile(np.roll(specials, -shift), reps)[:cols].astype(np.int16)
            y = np.empty(16, dtype=np.int32)
            gpu.matmul_rmajor_i16_v(np.ascontiguousarray(w).reshape(-1), x, y, 16, cols)
            assert np.array_equal(y, O.gemv_i16(np.ascontiguousarray(w).reshape(-1), x, 16, cols)), (cols, shift)
            assert gpu.dot_i16_v(np.ascontiguousarray(w[3]), x, cols) == O.dot_i16(np.ascontiguousarray(w[3]), x)
