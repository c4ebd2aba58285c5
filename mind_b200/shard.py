"""Row-band sharding of a GEMM / GEMV over the ranks of one node.

The reference parallelises these kernels as contiguous owner-computes bands of the M
output rows with no cross-band reduction (src/mlir/lowering.rs:10146-10205 of the
reference: ``band = ceil(M / T)``, band ``t`` owns rows ``[t*band, min((t+1)*band, M))``),
and its output does not depend on the band count.  Here a band owner is a GPU (one
process per GPU): A's band and C's band live only on their owner, B (or the GEMV vector)
is replicated, and there is NO data-path collective.  The optional all-gather of the C
bands keeps rank order, which is the reference's lexicographic shard order
(src/distributed/allgather.rs:7-20).
"""
from __future__ import annotations


def row_band(m: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [start, end) that `rank` of `world` owns; may be empty for trailing ranks."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank / world size")
    band = (m + world - 1) // world if m > 0 else 0
    start = min(rank * band, m)
    return start, min(start + band, m)


def all_gather_rows(local, m: int, n: int, group=None):
    """Gathers every rank's C band (a 1-D or 2-D torch tensor holding rows*n elements)
    into the full M x N matrix on every rank, bands in rank order.  Uneven last bands
    are padded to the common band height for the collective and trimmed afterwards."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    band = (m + world - 1) // world if m > 0 else 0
    start, end = row_band(m, world, rank)
    local = local.reshape(-1)
    if local.numel() != (end - start) * n:
        raise ValueError("local band has the wrong size for this rank")
    padded = local
    if end - start != band:
        padded = torch.zeros(band * n, dtype=local.dtype, device=local.device)
        padded[: local.numel()] = local
    full = torch.empty(world * band * n, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(full, padded.contiguous(), group=group)
    return full[: m * n].reshape(m, n)
