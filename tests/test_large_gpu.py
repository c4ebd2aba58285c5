"""Device-resident operands, the on-device input generator, the benchmark
configurations at full size (checked through size-independent properties where the
O(N^3) oracle is too slow), determinism across repeats, and the runtime mirror."""
import ctypes as C
import json
import os

import numpy as np
import pytest

import oracle as O

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
SELF = json.load(open(os.path.join(HERE, "golden", "oracle_hashes.json")))
torch = pytest.importorskip("torch")


@pytest.fixture(autouse=True)
def _stream(gpu):
    torch.cuda.set_device(0)
    gpu.set_stream(torch.cuda.current_stream().cuda_stream)
    gpu.set_gemm_path(0)
    yield
    gpu.set_gemm_path(0)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def lcg_dev(gpu, n, kind, seed, offset=0, shift=12):
    dt = {0: torch.int32, 1: torch.int8, 2: torch.int16}[kind]
    t = torch.empty(n, dtype=dt, device="cuda")
    gpu.lcg_fill(t, n, kind, seed, offset, shift)
    return t


def test_device_generator_matches_host(gpu):
    seed = 0xDEADBEEF00000000 ^ 12345
    n = 100003
    g = O.Lcg(seed)
    a8, b16, c32 = g.i8(n), g.i16(n), g.q16(n, 13)
    assert np.array_equal(lcg_dev(gpu, n, 1, seed).cpu().numpy(), a8)
    assert np.array_equal(lcg_dev(gpu, n, 2, seed, offset=n).cpu().numpy(), b16)
    assert np.array_equal(lcg_dev(gpu, n, 0, seed, offset=2 * n, shift=13).cpu().numpy(), c32)
    host = np.empty(77, dtype=np.int8)  # host destination goes through staging
    gpu.lcg_fill(host, 77, 1, seed)
    assert np.array_equal(host, a8[:77])


def test_device_pointers_all_kernels(gpu):
    g = O.Lcg(5)
    m, k, n = 200, 320, 136
    a, b = g.i8(m * k), g.i8(k * n)
    for path in (3, 2, 1, 0, 4, 5):
        gpu.set_gemm_path(path)
        c = torch.full((m * n,), -1, dtype=torch.int32, device="cuda")
        gpu.matmul_mm_i8_v(dev(a), dev(b), c, m, k, n)
        gpu.synchronize()
        assert np.array_equal(c.cpu().numpy(), O.gemm_i8(a, b, m, k, n)), path
    a, b = g.i16(m * k), g.i16(k * n)
    for path in (3, 2, 1, 0, 4, 5):
        gpu.set_gemm_path(path)
        c = torch.full((m * n,), -1, dtype=torch.int32, device="cuda")
        gpu.matmul_mm_i16(dev(a), dev(b), c, m, k, n)
        gpu.synchronize()
        assert np.array_equal(c.cpu().numpy(), O.gemm_i16(a, b, m, k, n)), path
    a, b = g.q16(m * k), g.q16(k * n)
    c = torch.full((m * n,), -1, dtype=torch.int32, device="cuda")
    gpu.matmul_mm_q16_v(dev(a), dev(b), c, m, k, n)
    y = torch.full((m,), -1, dtype=torch.int32, device="cuda")
    gpu.gemv_q16_mt(dev(a), dev(b[:k]), y, m, k)
    gpu.synchronize()
    assert np.array_equal(c.cpu().numpy(), O.gemm_q16(a, b, m, k, n))
    assert np.array_equal(y.cpu().numpy(), O.gemv_q16(a, b[:k], m, k))
    # mixed: host A, device B, host C
    ch = np.empty(m * n, dtype=np.int32)
    gpu.matmul_mm_q16_v(a, dev(b), ch, m, k, n)
    assert np.array_equal(ch, O.gemm_q16(a, b, m, k, n))


def test_config1_int8_256(gpu):
    e = SELF["gemm-i8-256x256x256"]
    a = lcg_dev(gpu, 256 * 256, 1, e["seed"])
    b = lcg_dev(gpu, 256 * 256, 1, e["seed"], offset=256 * 256)
    hashes = set()
    for path in (3, 2, 1, 0, 4, 5):
        gpu.set_gemm_path(path)
        for _ in range(16):  # the reference's same-process repeat gate uses 16 fresh buffers
            c = torch.empty(256 * 256, dtype=torch.int32, device="cuda")
            gpu.matmul_mm_i8_v(a, b, c, 256, 256, 256)
            hashes.add(O.canonical_hash_i32(c.cpu().numpy()))
    assert hashes == {e["sha256"]}


def test_config2_q16_1024(gpu):
    e = SELF["gemm-q16-1024x1024x1024-shift13"]
    n = 1024
    a = lcg_dev(gpu, n * n, 0, e["seed"], shift=13)
    b = lcg_dev(gpu, n * n, 0, e["seed"], offset=n * n, shift=13)
    c = torch.empty(n * n, dtype=torch.int32, device="cuda")
    gpu.matmul_mm_q16_v(a, b, c, n, n, n)
    assert O.canonical_hash_i32(c.cpu().numpy()) == e["sha256"]


def test_reproducibility_harness_workloads(gpu):
    """matmul-q16-32 / -256 / -1024 (docs/rfcs/0020-mind-bench-reproducibility-harness.md:93-95):
    every Q16.16 GEMM form reproduces the oracle's hash, host and device operands alike."""
    for n in (32, 256, 1024):
        e = SELF[f"matmul-q16-{n}"]
        a = lcg_dev(gpu, n * n, 0, e["seed"], shift=e["shift"])
        b = lcg_dev(gpu, n * n, 0, e["seed"], offset=n * n, shift=e["shift"])
        for path in (0, 1, 6, 7, 8, 9):
            gpu.set_gemm_path(path)
            c = torch.empty(n * n, dtype=torch.int32, device="cuda")
            gpu.matmul_mm_q16_mt_v(a, b, c, n, n, n)
            assert O.canonical_hash_i32(c.cpu().numpy()) == e["sha256"], (n, path)
        gpu.set_gemm_path(0)
        ch = np.empty(n * n, dtype=np.int32)
        gpu.matmul_mm_q16_v(a.cpu().numpy(), b.cpu().numpy(), ch, n, n, n)
        assert O.canonical_hash_i32(ch) == e["sha256"], n


def freivalds(gpu, a, b, c, m, k, n, elem_bytes, rounds=4):
    """Exact check in Z/2^32: C.v == A.(B.v) for random int32 vectors v."""
    gen = torch.Generator(device="cuda").manual_seed(1234)
    for _ in range(rounds):
        v = torch.randint(-2**31, 2**31 - 1, (n,), dtype=torch.int32, device="cuda", generator=gen)
        bv = torch.empty(k, dtype=torch.int32, device="cuda")
        abv = torch.empty(m, dtype=torch.int32, device="cuda")
        cv = torch.empty(m, dtype=torch.int32, device="cuda")
        gpu.matvec_wrap(b, elem_bytes, k, n, v, bv)
        gpu.matvec_wrap(a, elem_bytes, m, k, bv, abv)
        gpu.matvec_wrap(c, 4, m, n, v, cv)
        gpu.synchronize()
        if not torch.equal(abv, cv):
            return False
    return True


def test_matvec_wrap_helper(gpu):
    g = O.Lcg(3)
    m, k = 37, 91
    a = g.i16(m * k)
    v = g.q16(k, 0)
    out = np.empty(m, dtype=np.int32)
    gpu.matvec_wrap(a, 2, m, k, v, out)
    want = (a.reshape(m, k).astype(np.int64) @ v.astype(np.int64)).astype(np.int32)
    assert np.array_equal(out, want)


@pytest.mark.parametrize("path", [3, 2, 5])
def test_config3_i16_4096(gpu, path):
    gpu.set_gemm_path(path)
    n = 4096
    seed = 0xDEADBEEF00000000 ^ 4096
    a = lcg_dev(gpu, n * n, 2, seed)
    b = lcg_dev(gpu, n * n, 2, seed, offset=n * n)
    c = torch.empty(n * n, dtype=torch.int32, device="cuda")
    gpu.matmul_mm_i16(a, b, c, n, n, n)
    gpu.synchronize()
    assert freivalds(gpu, a, b, c, n, n, n, 2)
    # sampled row bands against the CPU oracle: first, last, and one in the middle
    ah, bh, ch = a.cpu().numpy(), b.cpu().numpy(), c.cpu().numpy().reshape(n, n)
    for r0 in (0, 2047, n - 2):
        want = O.gemm_i16(ah[r0 * n:(r0 + 2) * n], bh, 2, n, n).reshape(2, n)
        assert np.array_equal(ch[r0:r0 + 2], want)
    # and the whole matrix against the independent CUDA-core kernel
    gpu.set_gemm_path(1)
    c2 = torch.empty(n * n, dtype=torch.int32, device="cuda")
    gpu.matmul_mm_i16(a, b, c2, n, n, n)
    gpu.synchronize()
    assert torch.equal(c, c2)


def test_config4_gemv_16384(gpu):
    n = 16384
    seed = 0xDEADBEEF00000000 ^ ((n << 20) ^ n)
    w = lcg_dev(gpu, n * n, 0, seed, shift=15)
    x = lcg_dev(gpu, n, 0, seed, offset=n * n, shift=15)
    y = torch.empty(n, dtype=torch.int32, device="cuda")
    gpu.gemv_q16_mt(w, x, y, n, n)
    gpu.synchronize()
    want, _ = O.baseline_gemv_q16(w.cpu().numpy(), x.cpu().numpy(), n, n)
    assert np.array_equal(y.cpu().numpy(), want)
    # 256 stability re-runs, as the reference's MT bench does (benches/det_gemv_q16_mt.rs:71)
    for _ in range(256):
        y2 = torch.empty(n, dtype=torch.int32, device="cuda")
        gpu.gemv_q16_mt(w, x, y2, n, n)
        assert torch.equal(y, y2)


@pytest.mark.parametrize("path", [3, 2, 4])
def test_config5_int8_16384(gpu, path):
    gpu.set_gemm_path(path)
    n = 16384
    seed = 0xDEADBEEF00000000 ^ 16384
    a = lcg_dev(gpu, n * n, 1, seed)
    b = lcg_dev(gpu, n * n, 1, seed, offset=n * n)
    c = torch.empty(n * n, dtype=torch.int32, device="cuda")
    gpu.matmul_mm_i8_v(a, b, c, n, n, n)
    gpu.synchronize()
    assert freivalds(gpu, a, b, c, n, n, n, 1)
    ah, bh = a[: 2 * n].cpu().numpy(), b.cpu().numpy()
    assert np.array_equal(c[: 2 * n].cpu().numpy(), O.gemm_i8(ah, bh, 2, n, n))
    ah = a[(n - 2) * n:].cpu().numpy()
    assert np.array_equal(c[(n - 2) * n:].cpu().numpy(), O.gemm_i8(ah, bh, 2, n, n))
    # a row-sharded run (2 bands, as 2 GPUs would split it) gives the same bytes
    c2 = torch.empty(n * n, dtype=torch.int32, device="cuda")
    half = n // 2
    gpu.matmul_mm_i8_v(a[: half * n], b, c2[: half * n], half, n, n)
    gpu.matmul_mm_i8_v(a[half * n:], b, c2[half * n:], half, n, n)
    gpu.synchronize()
    assert torch.equal(c, c2)


def test_runtime_mirror(gpu):
    """allocate / run_op / synchronize / deallocate (src/runtime_interface.rs:26-52), every op name."""
    import mind_b200
    L = mind_b200.lib()
    m, k, n = 48, 80, 32
    g = O.Lcg(21)

    def alloc(dtype, *shape):
        h = C.c_int64(0)
        arr = (C.c_int64 * len(shape))(*shape)
        assert L.mind_b200_rt_allocate(dtype, arr, len(shape), C.byref(h)) == 0
        return h.value

    def run(op, dtype, a, b, a_shape, b_shape, out_shape):
        ha, hb, hc = alloc(dtype, *a_shape), alloc(dtype, *b_shape), alloc(2, *out_shape)
        assert L.mind_b200_rt_upload(ha, a.ctypes.data, a.nbytes) == 0
        assert L.mind_b200_rt_upload(hb, b.ctypes.data, b.nbytes) == 0
        ins, outs = (C.c_int64 * 2)(ha, hb), (C.c_int64 * 1)(hc)
        assert L.mind_b200_rt_run_op(op, ins, 2, outs, 1) == 0, L.mind_b200_last_error()
        assert L.mind_b200_rt_synchronize() == 0
        c = np.empty(int(np.prod(out_shape)), dtype=np.int32)
        assert L.mind_b200_rt_download(hc, c.ctypes.data, c.nbytes) == 0
        return c, (ha, hb, hc), (ins, outs)

    a8, b8 = g.i8(m * k), g.i8(k * n)
    c, handles, (ins, outs) = run(b"matmul_mm_i8_v", 0, a8, b8, (m, k), (k, n), (m, n))
    assert np.array_equal(c, O.gemm_i8(a8, b8, m, k, n))
    assert L.mind_b200_rt_run_op(b"no_such_op", ins, 2, outs, 1) == mind_b200.ERR_INVALID
    assert b"unknown op" in L.mind_b200_last_error()
    # an op given operands of the wrong element type is refused, not run on reinterpreted bytes
    assert L.mind_b200_rt_run_op(b"matmul_mm_q16_v", ins, 2, outs, 1) == mind_b200.ERR_INVALID
    assert b"dtype mismatch" in L.mind_b200_last_error()
    for h in handles:
        assert L.mind_b200_rt_deallocate(h) == 0
    assert L.mind_b200_rt_deallocate(handles[0]) == mind_b200.ERR_INVALID

    # what a MindRuntime shim does (the reference's DType has no int8): int32-tagged byte buffers,
    # last dimension = row bytes / 4, re-tagged as int8 for the op
    ha, hb, hc = alloc(2, m, k // 4), alloc(2, k, n // 4), alloc(2, m, n)
    assert L.mind_b200_rt_upload(ha, a8.ctypes.data, a8.nbytes) == 0
    assert L.mind_b200_rt_upload(hb, b8.ctypes.data, b8.nbytes) == 0
    assert L.mind_b200_rt_retag(ha, 0) == 0 and L.mind_b200_rt_retag(hb, 0) == 0
    assert L.mind_b200_rt_retag(ha, 0) == 0                      # already int8: nothing to do
    ins, outs = (C.c_int64 * 2)(ha, hb), (C.c_int64 * 1)(hc)
    assert L.mind_b200_rt_run_op(b"matmul_mm_i8_mt_v", ins, 2, outs, 1) == 0, L.mind_b200_last_error()
    c = np.empty(m * n, dtype=np.int32)
    assert L.mind_b200_rt_download(hc, c.ctypes.data, c.nbytes) == 0
    assert np.array_equal(c, O.gemm_i8(a8, b8, m, k, n))
    assert L.mind_b200_rt_retag(hc, 7) == mind_b200.ERR_INVALID
    for h in (ha, hb, hc):
        assert L.mind_b200_rt_deallocate(h) == 0

    aq, bq = g.q16(m * k), g.q16(k * n)
    for op in (b"matmul_mm_q16_v", b"__mind_blas_matmul_mm_q16_mt_v"):
        c, handles, _ = run(op, 2, aq, bq, (m, k), (k, n), (m, n))
        assert np.array_equal(c, O.gemm_q16(aq, bq, m, k, n)), op
        for h in handles:
            assert L.mind_b200_rt_deallocate(h) == 0
    a16, b16 = g.i16(m * k), g.i16(k * n)
    c, handles, _ = run(b"__mind_b200_matmul_mm_i16", 1, a16, b16, (m, k), (k, n), (m, n))
    assert np.array_equal(c, O.gemm_i16(a16, b16, m, k, n))
    for h in handles:
        assert L.mind_b200_rt_deallocate(h) == 0
    for op in (b"gemv_q16_mt", b"matmul_rmajor_q16_v"):
        c, handles, _ = run(op, 2, aq, bq[:k], (m, k), (k,), (m,))
        assert np.array_equal(c, O.gemv_q16(aq, bq[:k], m, k)), op
        for h in handles:
            assert L.mind_b200_rt_deallocate(h) == 0
    c, handles, _ = run(b"matmul_rmajor_i16_v", 1, a16, b16[:k], (m, k), (k,), (m,))
    assert np.array_equal(c, O.gemv_i16(a16, b16[:k], m, k))
    for h in handles:
        assert L.mind_b200_rt_deallocate(h) == 0


def test_shutdown_and_reload(gpu):
    """The library gives back what it holds on the GPU: mind_b200_shutdown() frees it and the next
    call rebuilds it; dlclose() runs the same teardown (the reference joins its thread pool in
    a destructor, runtime-support/mind_intrinsics.c:2065-2081) and a fresh dlopen() works again.
    Run in a child process, which owns its own copy of the library."""
    import subprocess
    import sys
    import mind_b200
    root = os.path.dirname(HERE)
    script = r"""
import ctypes as C, sys
import numpy as np
sys.path.insert(0, %r)
import oracle as O
LIB = %r
g = O.Lcg(31)
m, k, n = 300, 200, 136
a, b = g.i8(m * k), g.i8(k * n)
want = O.gemm_i8(a, b, m, k, n)
def product(L):
    f = L.__mind_blas_matmul_mm_i8_v
    f.argtypes, f.restype = [C.c_int64] * 6, C.c_int64
    c = np.zeros(m * n, dtype=np.int32)
    assert f(a.ctypes.data, b.ctypes.data, c.ctypes.data, m, k, n) == 0
    assert np.array_equal(c, want)
def free_bytes():
    import torch
    return torch.cuda.mem_get_info(0)[0]
L = C.CDLL(LIB)
L.mind_b200_shutdown.restype = C.c_int64
L.mind_b200_reserve.argtypes, L.mind_b200_reserve.restype = [C.c_int64] * 2, C.c_int64
product(L)
assert L.mind_b200_reserve(256 << 20, 256 << 20) == 0
held = free_bytes()
assert L.mind_b200_shutdown() == 0
assert free_bytes() > held, "shutdown released no device memory"
product(L)                      # contexts are rebuilt on demand
assert L.mind_b200_shutdown() == 0
assert L.mind_b200_shutdown() == 0   # twice is fine
product(L)
import _ctypes
handle = L._handle
del L
_ctypes.dlclose(handle)         # runs the library's destructor
L2 = C.CDLL(LIB)
product(L2)
print("reload ok")
""" % (root, mind_b200.LIB_PATH)
    r = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "reload ok" in r.stdout, r.stdout + r.stderr


def test_stability_reruns(gpu):
    """The reference's multithreaded benches re-run each kernel 256 times into fresh buffers and
    require identical bytes every time (benches/det_matmul_q16_mt.rs:88, :292-301)."""
    n = 512
    seed = 0xDEADBEEF00000000 ^ n
    a = lcg_dev(gpu, n * n, 0, seed)
    b = lcg_dev(gpu, n * n, 0, seed, offset=n * n)
    want = torch.from_numpy(O.gemm_q16(a.cpu().numpy(), b.cpu().numpy(), n, n, n)).cuda()
    for path in (0, 6, 8, 9, 1):  # fused hybrid (the default at this size), single FP64-pipe kernel, two-kernel hybrid in sequence / side by side, all-integer
        gpu.set_gemm_path(path)
        for _ in range(256 if path != 1 else 32):
            c = torch.empty(n * n, dtype=torch.int32, device="cuda")
            gpu.matmul_mm_q16_mt_v(a, b, c, n, n, n)
            assert torch.equal(c, want), path
    gpu.set_gemm_path(0)
    a8 = lcg_dev(gpu, 1024 * 1024, 1, seed)
    b8 = lcg_dev(gpu, 1024 * 1024, 1, seed, offset=1024 * 1024)
    first = None
    for path in (3, 2):
        gpu.set_gemm_path(path)
        for _ in range(128):
            c = torch.empty(1024 * 1024, dtype=torch.int32, device="cuda")
            gpu.matmul_mm_i8_mt_v(a8, b8, c, 1024, 1024, 1024)
            if first is None:
                first = c
            assert torch.equal(c, first), path
    # tall-and-skinny: the K range of the single tile is split across SMs and summed with atomics
    gpu.set_gemm_path(0)
    m, k, n = 64, 8192, 64
    at = lcg_dev(gpu, m * k, 1, seed)
    bt = lcg_dev(gpu, k * n, 1, seed, offset=m * k)
    want = torch.from_numpy(O.gemm_i8(at.cpu().numpy(), bt.cpu().numpy(), m, k, n)).cuda()
    a16 = lcg_dev(gpu, m * k, 2, seed)
    b16 = lcg_dev(gpu, k * n, 2, seed, offset=m * k)
    want16 = torch.from_numpy(O.gemm_i16(a16.cpu().numpy(), b16.cpu().numpy(), m, k, n)).cuda()
    for _ in range(128):
        c = torch.empty(m * n, dtype=torch.int32, device="cuda")
        gpu.matmul_mm_i8_v(at, bt, c, m, k, n)
        assert torch.equal(c, want)
        gpu.matmul_mm_i16(a16, b16, c, m, k, n)
        assert torch.equal(c, want16)


def test_q16_fused_kernel_under_producer_lag(gpu):
    """The fused Q16.16 kernel's FP32 stages are a TMA ring that the compute warps release with an
    mbarrier arrive.  Operands larger than L2 per call make the producer lag now and then, which
    is when a release that could overtake the last reads of a stage showed (one tile in thirty at
    2048^3 before the release was tied to the use of those reads).  Full-range operands, several
    shapes (ragged ones too), every run against the all-integer kernel's bytes."""
    for (m, k, n, reps) in ((2048, 2048, 2048, 12), (2048, 1024, 2048, 12), (1000, 2052, 1500, 8), (3000, 516, 3004, 8),
                            (4096, 2048, 64, 6), (64, 2048, 4096, 6), (11922, 384, 64, 6)):  # narrow: the build that skips padding halves
        seed = 0xDEADBEEF00000000 ^ (m * 131 + k * 17 + n)
        a = lcg_dev(gpu, m * k, 0, seed, shift=0)
        b = lcg_dev(gpu, k * n, 0, seed, offset=m * k, shift=0)
        want = torch.empty(m * n, dtype=torch.int32, device="cuda")
        gpu.set_gemm_path(1)
        gpu.matmul_mm_q16_v(a, b, want, m, k, n)
        for path in (8, 7):
            gpu.set_gemm_path(path)
            for _ in range(reps if path == 7 else 1):
                c = torch.zeros(m * n, dtype=torch.int32, device="cuda")
                gpu.matmul_mm_q16_v(a, b, c, m, k, n)
                gpu.synchronize()
                assert torch.equal(c, want), (path, m, k, n)
    gpu.set_gemm_path(0)


def test_q16_fused_ragged_and_unaligned_device_operands(gpu):
    """Device operands one element past a 16-byte boundary, K and N not multiples of 4: the fused
    kernel's operand split reads them element by element, and a C that a tensor map cannot
    address is written by the warps themselves (stores for whole-K runs, red.global.add otherwise)."""
    for (m, k, n, off) in ((777, 1030, 515, 1), (640, 512, 384, 1), (300, 2049, 130, 0), (129, 4099, 131, 3)):
        seed = 0xDEADBEEF00000000 ^ (m * 131 + k * 17 + n)
        abuf = lcg_dev(gpu, m * k + off, 0, seed, shift=0)
        bbuf = lcg_dev(gpu, k * n + off, 0, seed, offset=m * k + off, shift=0)
        a, b = abuf[off:], bbuf[off:]
        cbuf = torch.full((m * n + off + 8,), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
        c = cbuf[off:]
        want = torch.empty(m * n, dtype=torch.int32, device="cuda")
        gpu.set_gemm_path(1)
        gpu.matmul_mm_q16_v(a, b, want, m, k, n)
        gpu.set_gemm_path(7)
        for _ in range(3):
            gpu.matmul_mm_q16_v(a, b, c, m, k, n)
            gpu.synchronize()
            assert torch.equal(c[: m * n], want), (m, k, n, off)
            assert bool((c[m * n :] == 0x5A5A5A5A).all()) and bool((cbuf[:off] == 0x5A5A5A5A).all())
    gpu.set_gemm_path(0)


def test_cuda_graph_capture_and_replay(gpu):
    """Device-pointer calls are plain stream work: after one warm-up call (scratch sized, kernel
    attributes set) they can be captured into a CUDA graph and replayed, the two-stream Q16.16
    hybrid included (its side stream forks from and joins the captured stream)."""
    n = 1024
    seed = 0xDEADBEEF00000000 ^ n
    a8 = lcg_dev(gpu, n * n, 1, seed)
    b8 = lcg_dev(gpu, n * n, 1, seed, offset=n * n)
    a16 = lcg_dev(gpu, n * n, 2, seed)
    b16 = lcg_dev(gpu, n * n, 2, seed, offset=n * n)
    aq = lcg_dev(gpu, n * n, 0, seed, shift=13)
    bq = lcg_dev(gpu, n * n, 0, seed, offset=n * n, shift=13)
    side = torch.cuda.Stream()
    cases = [("i8", 0, lambda c: gpu.matmul_mm_i8_v(a8, b8, c, n, n, n)),
             ("i16", 0, lambda c: gpu.matmul_mm_i16(a16, b16, c, n, n, n)),
             ("q16 one kernel", 6, lambda c: gpu.matmul_mm_q16_v(aq, bq, c, n, n, n)),
             ("q16 fused kernel (launched programmatically behind its operand split)", 7,
              lambda c: gpu.matmul_mm_q16_v(aq, bq, c, n, n, n)),
             ("q16 hybrid in sequence", 8, lambda c: gpu.matmul_mm_q16_v(aq, bq, c, n, n, n)),
             ("q16 hybrid side by side", 9, lambda c: gpu.matmul_mm_q16_v(aq, bq, c, n, n, n)),
             ("gemv", 0, lambda c: gpu.gemv_q16_mt(aq, bq, c, n, n))]
    try:
        for name, path, call in cases:
            gpu.set_gemm_path(path)
            want = torch.empty(n * n, dtype=torch.int32, device="cuda")
            gpu.set_stream(torch.cuda.current_stream().cuda_stream)
            call(want)
            torch.cuda.synchronize()
            out = torch.zeros(n * n, dtype=torch.int32, device="cuda")
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                gpu.set_stream(side.cuda_stream)
                call(out)                      # warm-up on the capturing stream
                torch.cuda.synchronize()
                out.zero_()
                with torch.cuda.graph(graph, stream=side):
                    call(out)
            gpu.set_stream(torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            assert int(out.abs().max()) == 0, name   # capture records, it does not run
            for _ in range(3):
                out.zero_()
                graph.replay()
                torch.cuda.synchronize()
                rows = n if name == "gemv" else n * n
                assert torch.equal(out[:rows], want[:rows]), name
    finally:
        gpu.set_gemm_path(0)
        gpu.set_stream(torch.cuda.current_stream().cuda_stream)


def test_pinned_host_operands_through_the_pipeline(gpu):
    """Page-locked host operands (what the end-to-end bench passes): uploads and downloads are
    then truly asynchronous, so the band / chunk ordering is what keeps the bytes right."""
    m, k, n = 4096, 1024, 8192
    seed = 0xDEADBEEF00000000 ^ 4097
    a = lcg_dev(gpu, m * k, 1, seed)
    b = lcg_dev(gpu, k * n, 1, seed, offset=m * k)
    want = torch.empty(m * n, dtype=torch.int32, device="cuda")
    gpu.matmul_mm_i8_v(a, b, want, m, k, n)
    ha, hb = a.cpu().pin_memory(), b.cpu().pin_memory()
    for rep in range(3):
        hc = torch.full((m * n,), -1, dtype=torch.int32).pin_memory()
        gpu.matmul_mm_i8_v(ha, hb, hc, m, k, n)          # all three on the host
        assert torch.equal(hc, want.cpu()), rep
    hc = torch.full((m * n,), -1, dtype=torch.int32).pin_memory()
    gpu.matmul_mm_i8_v(a, hb, hc, m, k, n)               # A on the device
    assert torch.equal(hc, want.cpu())
    hc = torch.full((m * n,), -1, dtype=torch.int32).pin_memory()
    gpu.matmul_mm_i8_v(ha, b, hc, m, k, n)               # B on the device
    assert torch.equal(hc, want.cpu())


def test_few_very_long_rows(gpu):
    """A long dot product is one row: it is cut into pieces, one block each, and the pieces are
    added up in a fixed order.  Device and host operands, all three element kinds, and a length
    that cannot be cut evenly (single-block path)."""
    for n in (1 << 22, (1 << 22) + 4 * 37):
        a = lcg_dev(gpu, n, 0, 77, shift=12)
        b = lcg_dev(gpu, n, 0, 77, offset=n, shift=12)
        ah, bh = a.cpu().numpy(), b.cpu().numpy()
        assert gpu.dot_q16_v(a, b, n) == O.dot_q16(ah, bh), n
        assert gpu.dot_l1_q16_v(a, b, n) == O.dot_l1_q16(ah, bh), n
        assert gpu.dot_q16_v(ah, bh, n) == O.dot_q16(ah, bh), n
    n = 1 << 23
    a16 = lcg_dev(gpu, n, 2, 78)
    b16 = lcg_dev(gpu, n, 2, 78, offset=n)
    assert gpu.dot_i16_v(a16, b16, n) == O.dot_i16(a16.cpu().numpy(), b16.cpu().numpy())
    rows, cols = 3, 1 << 21
    w = lcg_dev(gpu, rows * cols, 0, 79, shift=12)
    x = lcg_dev(gpu, cols, 0, 79, offset=rows * cols, shift=12)
    y = torch.empty(rows, dtype=torch.int32, device="cuda")
    gpu.gemv_q16_mt(w, x, y, rows, cols)
    assert np.array_equal(y.cpu().numpy(), O.gemv_q16(w.cpu().numpy(), x.cpu().numpy(), rows, cols))
