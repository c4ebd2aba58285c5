"""One call spread over several GPUs (MINDB200_DEVICES / mind_b200_set_devices).

The reference's `_mt` entry points cut one call into contiguous owner-computes row bands, one
per thread, and its gate requires the bytes not to depend on the band count
(tests/cross_substrate_identity.rs:1412-1431).  Here a band owner is a GPU; these tests need at
least two of them and compare a 2-device (and all-device) call byte for byte with the 1-device
call and with the CPU oracle."""
import numpy as np
import pytest

import oracle as O

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture()
def multi(gpu):
    if gpu.device_count() < 2:
        pytest.skip("needs at least two B200s")
    torch.cuda.set_device(0)
    gpu.set_stream(torch.cuda.current_stream().cuda_stream)
    gpu.set_gemm_path(0)
    yield gpu
    gpu.set_devices(1)
    gpu.set_gemm_path(0)


def _device_counts(gpu):
    n = gpu.device_count()
    return sorted({2, min(n, 3), n})


def test_int8_gemm_over_devices_equals_one_device(multi):
    gpu = multi
    # aligned (B read in place), ragged K (A padded on upload), ragged N (B transposed on each
    # device after the exchange), M that does not divide evenly
    for (m, k, n) in [(4096, 1024, 2048), (3001, 520, 1040), (2048, 777, 1000), (1100, 4096, 512)]:
        g = O.Lcg(0xDEADBEEF00000000 ^ (m * 31 + k * 7 + n))
        a, b = g.i8(m * k), g.i8(k * n)
        gpu.set_devices(1)
        one = np.full(m * n, -1, dtype=np.int32)
        gpu.matmul_mm_i8_v(a, b, one, m, k, n)
        # rows at both ends and across the 2-device band boundary against the CPU oracle
        band = -(-m // 2)
        for r0 in (0, band - 2, m - 3):
            rows = min(4, m - r0)
            assert np.array_equal(one[r0 * n:(r0 + rows) * n], O.gemm_i8(a[r0 * k:(r0 + rows) * k], b, rows, k, n))
        for devs in _device_counts(gpu):
            gpu.set_devices(devs)
            assert gpu.devices() == devs
            for rep in range(2):  # the second call reuses the buffers and threads of the first
                c = np.full(m * n + 8, 0x5A5A5A5A, dtype=np.int32)
                gpu.matmul_mm_i8_mt_v(a, b, c, m, k, n)
                assert np.array_equal(c[: m * n], one), (devs, m, k, n, rep)
                assert np.all(c[m * n:] == 0x5A5A5A5A)


def test_pinned_operands_and_all_paths_over_two_devices(multi):
    gpu = multi
    m, k, n = 4096, 2048, 4096
    seed = 0xDEADBEEF00000000 ^ 4099
    a = torch.empty(m * k, dtype=torch.int8, device="cuda")
    b = torch.empty(k * n, dtype=torch.int8, device="cuda")
    gpu.lcg_fill(a, m * k, 1, seed, 0, 0)
    gpu.lcg_fill(b, k * n, 1, seed, m * k, 0)
    want = torch.empty(m * n, dtype=torch.int32, device="cuda")
    gpu.matmul_mm_i8_v(a, b, want, m, k, n)
    gpu.synchronize()
    want = want.cpu()
    ha, hb = a.cpu().pin_memory(), b.cpu().pin_memory()
    gpu.set_devices(2)
    for path in (0, 2, 3, 4):
        gpu.set_gemm_path(path)
        hc = torch.full((m * n,), -1, dtype=torch.int32).pin_memory()
        gpu.matmul_mm_i8_v(ha, hb, hc, m, k, n)
        assert torch.equal(hc, want), path


def test_other_kernels_are_banded_over_devices(multi):
    gpu = multi
    gpu.set_devices(2)
    # Q16.16 GEMV: the matrix is the big operand, the vector goes to every device
    rows, cols = 5000, 1024
    g = O.Lcg(77)
    w, x = g.q16(rows * cols), g.q16(cols)
    y = np.full(rows + 4, 0x5A5A5A5A, dtype=np.int32)
    gpu.gemv_q16_mt(w, x, y, rows, cols)
    assert np.array_equal(y[:rows], O.gemv_q16(w, x, rows, cols))
    assert np.all(y[rows:] == 0x5A5A5A5A)
    w16, x16 = g.i16(rows * cols), g.i16(cols)
    gpu.matmul_rmajor_i16_v(w16, x16, y, rows, cols)
    assert np.array_equal(y[:rows], O.gemv_i16(w16, x16, rows, cols))
    # int16 and Q16.16 GEMM with a tall A (B small next to A and C)
    m, k, n = 6000, 256, 200
    a16, b16 = g.i16(m * k), g.i16(k * n)
    c = np.empty(m * n, dtype=np.int32)
    gpu.matmul_mm_i16(a16, b16, c, m, k, n)
    gpu.set_devices(1)
    c1 = np.empty(m * n, dtype=np.int32)
    gpu.matmul_mm_i16(a16, b16, c1, m, k, n)
    assert np.array_equal(c, c1)
    for r0 in (0, 2999, m - 2):
        assert np.array_equal(c[r0 * n:(r0 + 2) * n], O.gemm_i16(a16[r0 * k:(r0 + 2) * k], b16, 2, k, n))
    aq, bq = g.q16(m * k), g.q16(k * n)
    gpu.set_devices(2)
    gpu.matmul_mm_q16_mt_v(aq, bq, c, m, k, n)
    gpu.set_devices(1)
    gpu.matmul_mm_q16_mt_v(aq, bq, c1, m, k, n)
    assert np.array_equal(c, c1)
    for r0 in (0, 2999, m - 2):
        assert np.array_equal(c[r0 * n:(r0 + 2) * n], O.gemm_q16(aq[r0 * k:(r0 + 2) * k], bq, 2, k, n))


def test_device_operands_stay_on_their_device_and_foreign_ones_are_refused(multi):
    """Calls with device pointers always run on the current device alone; an operand that lives
    on another device is refused with a clear error, never copied behind the caller's back."""
    import mind_b200
    gpu = multi
    gpu.set_devices(2)
    m, k, n = 2048, 256, 512
    g = O.Lcg(5)
    a, b = g.i8(m * k), g.i8(k * n)
    want = O.gemm_i8(a, b, m, k, n)
    da, db = torch.from_numpy(a).cuda(0), torch.from_numpy(b).cuda(0)
    dc = torch.zeros(m * n, dtype=torch.int32, device="cuda:0")
    gpu.matmul_mm_i8_v(da, db, dc, m, k, n)
    gpu.synchronize()
    assert np.array_equal(dc.cpu().numpy(), want)
    foreign = torch.from_numpy(b).cuda(1)
    torch.cuda.set_device(0)
    with pytest.raises(mind_b200.MindB200Error) as e:
        gpu.matmul_mm_i8_v(da, foreign, dc, m, k, n)
    assert e.value.code == mind_b200.ERR_INVALID and "lives on device 1" in str(e.value)
    with pytest.raises(mind_b200.MindB200Error):
        gpu.set_devices(gpu.device_count() + 1)


def test_devices_come_from_the_environment(multi):
    """MINDB200_DEVICES names the GPUs a host-operand call may use: a count or a list of ordinals
    (read once, when the library first needs it)."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = ("import sys; sys.path.insert(0, %r); import numpy as np; import oracle as O; from mind_b200 import blas; "
              "print('devices', blas.devices()); m, k, n = 2048, 512, 1024; g = O.Lcg(9); a, b = g.i8(m * k), g.i8(k * n); "
              "c = np.empty(m * n, dtype=np.int32); blas.matmul_mm_i8_v(a, b, c, m, k, n); "
              "assert np.array_equal(c[:4 * n], O.gemm_i8(a[:4 * k], b, 4, k, n)); "
              "assert np.array_equal(c[-4 * n:], O.gemm_i8(a[-4 * k:], b, 4, k, n)); print('ok')") % root
    for value, want in (("2", 2), ("1,0", 2), ("", 1), ("99", multi.device_count())):
        env = dict(os.environ, MINDB200_DEVICES=value)
        r = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env, timeout=600)
        assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr
        assert f"devices {want}" in r.stdout, (value, r.stdout)
