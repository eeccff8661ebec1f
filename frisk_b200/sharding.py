"""Row-block sharding of C = A*B across the GPUs of one node: rank r owns a contiguous block of
rows of A and C, B is replicated, nothing is exchanged on the data path.  The helpers here are the
host-side plumbing around that (torch.distributed, NCCL on GPUs, gloo on CPU in the tests); the
optional all-gather of C is the only collective, and it has two forms: NCCL after the GEMM
(`allgather_rows`), or folded into the GEMM (`PeerGather`: every rank's epilogue stores its tiles
into every other rank's copy of C with ordinary stores over NVLink, nothing is loaded from a
peer).  The reference has no multi-device notion."""
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


class PeerGather:
    """A whole-C buffer on every rank of a node that the other ranks' GEMM epilogues store into.

    Each rank allocates [M, N] of C's element type (frisk_b200_peer_alloc), the 64-byte handles go
    round with ``all_gather_object``, and every rank maps the other ranks' buffers
    (frisk_b200_peer_open).  ``local_c`` is where this rank's GEMM writes its own rows,
    ``peer_dsts`` where the same rows start in each other rank's buffer: pass both to
    ``GemmPlan.run_ex(..., peers=...)``.  A rank may read its buffer once every rank's launch has
    completed: synchronise the stream, then ``dist.barrier()``.
    """

    def __init__(self, dist, M: int, N: int, elem_size: int, world: int, rank: int):
        import ctypes as C

        self.M, self.N, self.es, self.world, self.rank = M, N, elem_size, world, rank
        self.nbytes = M * N * elem_size
        L = R.lib()
        ptr = C.c_void_p()
        handle = C.create_string_buffer(64)
        R._check(L.frisk_b200_peer_alloc(self.nbytes, C.byref(ptr), handle), "peer_alloc")
        self.ptr = int(ptr.value)
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle.raw))
        self.peer_ptrs = {}
        for r in range(world):
            if r == rank:
                continue
            q = C.c_void_p()
            R._check(L.frisk_b200_peer_open(handles[r], C.byref(q)), f"peer_open(rank {r})")
            self.peer_ptrs[r] = int(q.value)
        self.row0, self.rows = local_rows(M, world, rank)
        offset = self.row0 * N * elem_size
        self.local_c = self.ptr + offset
        # each rank walks its peers starting with its right-hand neighbour, so that at any moment
        # the ranks' epilogues aim at different GPUs instead of all at the same one
        order = [(rank + k) % world for k in range(1, world)]
        self.peer_dsts = [self.peer_ptrs[r] + offset for r in order]

    def as_tensor(self, dtype):
        """The rank's whole-C buffer as a torch tensor [M, N] (no copy)."""
        import torch

        class _Raw:  # the CUDA array interface torch.as_tensor understands
            pass

        raw = _Raw()
        typestr = {1: "|u1", 2: "<i2", 4: "<f4"}[self.es]
        raw.__cuda_array_interface__ = {"shape": (self.M, self.N), "typestr": typestr,
                                        "data": (self.ptr, False), "version": 2}
        t = torch.as_tensor(raw, device=torch.device("cuda", torch.cuda.current_device()))
        return t.view(dtype) if t.dtype != dtype else t

    def close(self, dist=None) -> None:
        """Unmaps the peers' buffers, then (after a barrier, when `dist` is given, so that no rank
        frees memory another still has mapped) frees this rank's."""
        L = R.lib()
        for q in self.peer_ptrs.values():
            L.frisk_b200_peer_close(q)
        self.peer_ptrs = {}
        if dist is not None:
            dist.barrier()
        if self.ptr:
            L.frisk_b200_peer_free(self.ptr)
            self.ptr = 0
