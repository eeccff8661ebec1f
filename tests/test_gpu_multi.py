"""Two GPUs, two processes: the all-gather of C folded into the GEMM's epilogue.  Each rank
computes its row block and stores every tile into its own copy of C and, through peer-mapped
pointers, into the other rank's; afterwards both ranks hold the whole C, bit-equal to the product
computed on one GPU and within tolerance of the CPU oracle.  Skipped on a box with one GPU (the
single-GPU form of the same code path, peers on the same device, is in test_gpu_epilogue.py)."""
import os
import socket
import sys

import numpy as np
import pytest

from frisk_b200 import workloads as W

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, M, N, K, out_dir):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    from frisk_b200 import runtime as R
    from frisk_b200 import sharding as S

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    w = W.make_workload("cfg5", M, N, K)
    row0, rows = S.local_rows(M, world, rank)
    A = torch.from_numpy(w.A[row0:row0 + rows].view(np.int16)).to(dev)
    B = torch.from_numpy(w.B.view(np.int16)).to(dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    pg = S.PeerGather(dist, M, N, 2, world, rank)
    try:
        full = pg.as_tensor(torch.int16)
        full.fill_(0x7FC0)
        torch.cuda.synchronize()
        dist.barrier()
        for epilogue in (2, 1, 4):   # 128-byte pieces, per-thread stores, TMA tensor stores
            plan = R.GemmPlan(rows, N, K, W.BF16, epilogue=epilogue)
            plan.run_ex(A, B, pg.local_c, status=status, peers=pg.peer_dsts)
            torch.cuda.synchronize()
            dist.barrier()   # every rank's stores have landed
            R.check_status(status)
            np.save(os.path.join(out_dir, f"c_rank{rank}_epi{epilogue}.npy"), full.cpu().numpy())
            plan.close()
            full.fill_(0x7FC0)
            torch.cuda.synchronize()
            dist.barrier()
        # the NCCL form of the same gather, for comparison
        plan = R.GemmPlan(rows, N, K, W.BF16)
        c_local = torch.empty((rows, N), dtype=torch.bfloat16, device=dev)
        plan.run(A, B, c_local, status=status)
        plan.close()
        gathered = S.allgather_rows(dist, c_local, M, world, rank)
        np.save(os.path.join(out_dir, f"c_rank{rank}_nccl.npy"), gathered.view(torch.int16).cpu().numpy())
    finally:
        torch.cuda.synchronize()
        pg.close(dist)
        dist.destroy_process_group()


def test_two_ranks_gather_c_through_the_epilogue(tmp_path):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from frisk_b200 import runtime as R
    from oracle import ref

    M, N, K = 1000, 1024, 512   # ragged row blocks are not needed here: 500 rows per rank
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, M, N, K, str(tmp_path)), nprocs=2, join=True)
    w = W.make_workload("cfg5", M, N, K)
    whole = R.gemm_host(w).view(np.int16)   # the same product on one GPU
    for tag in ("epi2", "epi1", "epi4", "nccl"):
        for rank in (0, 1):
            got = np.load(tmp_path / f"c_rank{rank}_{tag}.npy")
            assert np.array_equal(got, whole), f"rank {rank}, {tag}: the gathered C differs from the one-GPU product"
    ok, err, metric = W.check(W.bf16_decode(whole.view(np.uint16)), ref.ref_gemm_f64(w), W.BF16, absdot=ref.abs_dot(w))
    assert ok, (metric, err)
