"""Host logic of the multi-GPU path on CPU: the band rule, and a world-size-2 gloo run in
which each rank computes only its band (with the CPU oracle standing in for the GPU
kernel) and the gathered result equals the unsharded one."""
import os
import socket
import sys

import numpy as np
import pytest

import oracle as O
from mind_b200.shard import row_band


def test_band_rule_matches_reference_partition():
    for m in (0, 1, 2, 7, 100, 16384):
        for world in (1, 2, 4, 8):
            bands = [row_band(m, world, r) for r in range(world)]
            nonempty = [b for b in bands if b[0] < b[1]]
            assert nonempty == O.row_bands(m, world)[: len(nonempty)]
            covered = [r for s, e in bands for r in range(s, e)] if m <= 100 else None
            if covered is not None:
                assert covered == list(range(m))
            assert bands[-1][1] == m or m == 0
    with pytest.raises(ValueError):
        row_band(4, 2, 2)


def _worker(rank, world, port, m, k, n, out_dir):
    import torch
    import torch.distributed as dist
    from mind_b200.shard import all_gather_rows, row_band as rb
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = O.Lcg(0xDEADBEEF)
    a, b = g.i8(m * k), g.i8(k * n)  # every rank regenerates the inputs from the seed
    s, e = rb(m, world, rank)
    local = O.gemm_i8(a[s * k:e * k], b, e - s, k, n)
    full = all_gather_rows(torch.from_numpy(local), m, n)
    np.save(os.path.join(out_dir, f"c{rank}.npy"), full.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("m", [64, 7])
def test_two_rank_gloo_run_equals_unsharded(tmp_path, m):
    import torch.multiprocessing as mp
    k, n, world = 40, 24, 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(world, port, m, k, n, str(tmp_path)), nprocs=world, join=True)
    g = O.Lcg(0xDEADBEEF)
    a, b = g.i8(m * k), g.i8(k * n)
    want = O.gemm_i8(a, b, m, k, n).reshape(m, n)
    for r in range(world):
        assert np.array_equal(np.load(tmp_path / f"c{r}.npy"), want)
