"""The int8 GEMM entry point that allocates nothing (``mind_b200_matmul_mm_i8_static``).

Some callers cannot allocate GPU memory at the moment they need the product (a serving
loop or stream callback where cudaMalloc is off limits, or a process whose GPU memory
belongs to another allocator), so this variant keeps its re-laid-out operands in a fixed
array inside the library.  It must give the same bytes as the regular entry point
``__mind_blas_matmul_mm_i8_v`` -- bit for bit, as every integer check in this suite --
on two calls in a row (the array keeps the first call's contents, so the second call
uses a different, smaller shape that would expose anything stale), and refuse what does
not fit.  The file name sorts last on purpose: a run that stops at the first failure has
already run every other test by the time it gets here.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _operands(gpu, m, k, n, seed):
    # torch generates the operands, so that in a fresh process the static entry point is the
    # first thing this library is asked to do on the device (no context exists yet)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randint(-128, 128, (m * k,), dtype=torch.int8, device="cuda", generator=gen)
    b = torch.randint(-128, 128, (k * n,), dtype=torch.int8, device="cuda", generator=gen)
    return a, b


def test_static_scratch_gemm_matches_regular_entry_point(gpu):
    import mind_b200
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    # first call: the largest square that fits (B^T of 2048 x 2048 is 4 MiB), A used in place;
    # second call: ragged shape, K % 16 != 0, so the padded copy of A goes to the array as well.
    for (m, k, n, seed) in ((2048, 2048, 2048, 0xDEADBEEF), (333, 1000, 517, 0xDEADBEEF ^ 7)):
        a, b = _operands(gpu, m, k, n, seed)
        got = torch.full((m * n,), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
        assert gpu.matmul_mm_i8_static(a, b, got, m, k, n, stream) == 0
        # synchronous by contract: the result is complete when the call returns
        got_host = got.cpu()
        want = torch.full((m * n,), -1, dtype=torch.int32, device="cuda")
        gpu.set_stream(stream)
        gpu.matmul_mm_i8_v(a, b, want, m, k, n)
        gpu.synchronize()
        assert torch.equal(got_host, want.cpu()), (m, k, n)

    # beyond the stated maximum: refused with a clear error, nothing launched
    m = k = n = 4096  # B^T alone is 16 MiB > 8 MiB
    a, b = _operands(gpu, m, k, n, 1)
    c = torch.zeros(m * n, dtype=torch.int32, device="cuda")
    with pytest.raises(mind_b200.MindB200Error) as e:
        gpu.matmul_mm_i8_static(a, b, c, m, k, n, stream)
    assert e.value.code == mind_b200.ERR_TOO_LARGE and "static scratch" in str(e.value)
    assert n * k > gpu.STATIC_SCRATCH_BYTES

    # host operands would need staging memory: refused
    ah = np.zeros(16, dtype=np.int8)
    ch = np.zeros(16, dtype=np.int32)
    with pytest.raises(mind_b200.MindB200Error) as e:
        gpu.matmul_mm_i8_static(ah, ah, ch, 4, 4, 4, stream)
    assert e.value.code == mind_b200.ERR_INVALID and "host pointer" in str(e.value)
