"""The multi-GPU path on CPU: two gloo ranks shard the rows of C = A*B, compute their blocks (with
the CPU oracle standing in for the kernel), all-gather C and agree on the max-over-ranks time.
Host-made failures only: a rank that reports an error before the collective."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from frisk_b200 import sharding as S
from frisk_b200 import workloads as W


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, N, K, fail_rank, out):
    from oracle import ref

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = W.make_workload("cfg5", M, N, K)  # same seed on every rank: B is replicated
        row0, rows = S.local_rows(M, world, rank)
        ws = W.GemmWorkload("shard", rows, N, K, W.BF16, W.BF16, B=w.B,
                            A=np.ascontiguousarray(w.A[row0:row0 + rows]))
        ok = torch.tensor([0 if rank == fail_rank else 1], dtype=torch.int32)
        # gloo has no 16-bit integer collectives: carry the bf16 bits in int32
        local = torch.from_numpy(ref.ref_gemm(ws).astype(np.int32)) if rows else torch.zeros((0, N), dtype=torch.int32)
        # every rank learns of a failed peer on the host, before the collective, and skips it
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            out[rank] = "skipped"
            return
        full = S.allgather_rows(dist, local, M, world, rank)
        want = torch.from_numpy(ref.ref_gemm(w).astype(np.int32))
        slowest = S.max_over_ranks(dist, float(rank + 1), torch.device("cpu"))
        out[rank] = (bool(torch.equal(full, want)), slowest)
    finally:
        dist.destroy_process_group()


def _run(world, M, N, K, fail_rank=-1):
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, M, N, K, fail_rank, out), nprocs=world, join=True)
    return dict(out)


@pytest.mark.parametrize("M", [64, 37])
def test_two_ranks_shard_rows_and_gather_c(M):
    out = _run(2, M, 48, 64)
    assert out == {0: (True, 2.0), 1: (True, 2.0)}


def test_a_failed_rank_makes_every_rank_skip_the_collective():
    out = _run(2, 32, 16, 32, fail_rank=1)
    assert out == {0: "skipped", 1: "skipped"}
