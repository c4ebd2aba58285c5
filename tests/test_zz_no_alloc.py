"""The int8 GEMM entry point that allocates nothing (``mind_b200_matmul_mm_i8_static``).

Some callers cannot allocate GPU memory at the moment they need the product (a serving
loop where cudaMalloc is off limits, or a process whose GPU memory belongs to another
allocator), so this variant keeps its re-laid-out operands in a fixed array inside the
library.  It must give the same bytes as the regular entry point
``__mind_blas_matmul_mm_i8_v`` and as the CPU oracle -- bit for bit, as every integer check
in this suite -- on calls in a row (the array keeps the previous call's contents, so
successive calls use different shapes that would expose anything stale), and refuse what
does not fit.  The file name sorts last on purpose: a run that stops at the first failure has
already run every other test by the time it gets here.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _operands(gpu, m, k, n, seed):
    # torch generates the operands, so that when this file runs alone in a fresh process the
    # static entry point is the first thing this library is asked to do on the device
    gen = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randint(-128, 128, (m * k + 1,), dtype=torch.int8, device="cuda", generator=gen)
    b = torch.randint(-128, 128, (k * n,), dtype=torch.int8, device="cuda", generator=gen)
    return a, b


def test_static_scratch_gemm_matches_regular_entry_point(gpu):
    import mind_b200
    import oracle as O
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    cases = [
        # (m, k, n, byte offset of A): what the shape exercises
        (2048, 2048, 2040, 0),   # B transposed into the array (N % 16 != 0): 2040 x 2048 = 4 MiB of it
        (333, 1000, 517, 0),     # ragged: transposed B and padded A (K % 16 != 0) both in the array
        (2048, 2048, 2048, 0),   # everything readable in place: the array holds only the error word
        (32768, 64, 2048, 0),    # more 128 x 256 tiles than SMs: the CTA-pair kernel
        (64, 8192, 64, 0),       # one tile, long K: split across SMs, added onto a cleared C
        (200, 512, 100, 1),      # A misaligned by one byte although K % 16 == 0: padded copy
    ]
    for (m, k, n, off) in cases:
        a, b = _operands(gpu, m, k, n, 0xDEADBEEF ^ (m + 3 * n))
        a = a[off: off + m * k]
        got = torch.full((m * n,), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
        assert gpu.matmul_mm_i8_static(a.data_ptr(), b, got, m, k, n, stream) == 0
        # synchronous by contract: the result is complete when the call returns
        got_host = got.cpu()
        want = torch.full((m * n,), -1, dtype=torch.int32, device="cuda")
        gpu.set_stream(stream)
        gpu.matmul_mm_i8_v(a.data_ptr(), b, want, m, k, n)
        gpu.synchronize()
        assert torch.equal(got_host, want.cpu()), (m, k, n)
        # and against the CPU oracle: all of a small product, the first and last rows of a large one
        ah, bh = a.cpu().numpy().copy(), b.cpu().numpy()
        rows = m if m * k * n <= 2e8 else 2
        for r0 in {0, m - rows}:
            assert np.array_equal(got_host.numpy()[r0 * n:(r0 + rows) * n],
                                  O.gemm_i8(ah[r0 * k:(r0 + rows) * k], bh, rows, k, n)), (m, k, n, r0)

    # beyond the stated maximum: refused with a clear error, nothing launched
    m = k = 4096
    n = 4090  # N % 16 != 0: B must be transposed, and B^T alone is 16 MiB > 8 MiB
    a, b = _operands(gpu, m, k, n, 1)
    c = torch.zeros(m * n, dtype=torch.int32, device="cuda")
    with pytest.raises(mind_b200.MindB200Error) as e:
        gpu.matmul_mm_i8_static(a, b, c, m, k, n, stream)
    assert e.value.code == mind_b200.ERR_TOO_LARGE and "static scratch" in str(e.value)
    assert n * k > gpu.STATIC_SCRATCH_BYTES
    # sizes that would wrap a 64-bit product are refused before anything is sized
    with pytest.raises(mind_b200.MindB200Error) as e:
        gpu.matmul_mm_i8_static(a, b, c, 1 << 40, 1 << 40, 3, stream)
    assert e.value.code == mind_b200.ERR_TOO_LARGE

    # host operands would need staging memory: refused
    ah = np.zeros(16, dtype=np.int8)
    ch = np.zeros(16, dtype=np.int32)
    with pytest.raises(mind_b200.MindB200Error) as e:
        gpu.matmul_mm_i8_static(ah, ah, ch, 4, 4, 4, stream)
    assert e.value.code == mind_b200.ERR_INVALID and "host pointer" in str(e.value)
