"""Row-block sharding of C = A*B across the GPUs of one node: rank r owns a contiguous block of
rows of A and C, B is replicated, nothing is exchanged on the data path.  The helpers here are the
host-side plumbing around that (torch.distributed, NCCL on GPUs, gloo on CPU in the tests); the
optional all-gather of C is the only collective.  The reference has no multi-device notion."""
from __future__ import annotations

from typing import Tuple

from . import runtime as R


def local_rows(M: int, world: int, rank: int) -> Tuple[int, int]:
    """(row0, rows) of rank's block; the first M % world ranks hold one extra row."""
    return R.shard_rows(M, world, rank)


def allgather_rows(dist, local_c, M: int, world: int, rank: int):
    """Gathers the row blocks of C from all ranks into the full [M, N] matrix on every rank."""
    import torch

    N = local_c.shape[1]
    full = torch.empty((M, N), dtype=local_c.dtype, device=local_c.device)
    if M % world == 0:
        dist.all_gather_into_tensor(full, local_c.contiguous())
        return full
    # ragged blocks: gather padded blocks, then keep each rank's real rows
    pad_rows = M // world + 1
    padded = torch.zeros((pad_rows, N), dtype=local_c.dtype, device=local_c.device)
    padded[: local_c.shape[0]] = local_c
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded)
    for r in range(world):
        row0, rows = local_rows(M, world, r)
        full[row0:row0 + rows] = parts[r][:rows]
    return full


def max_over_ranks(dist, value: float, device) -> float:
    """The slowest rank's time: what a multi-GPU number is reported as."""
    import torch

    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist is not None and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
