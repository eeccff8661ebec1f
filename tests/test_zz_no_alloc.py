"""The skinny GEMM entry point that allocates nothing (frisk_b200_gemm_skinny_static).

It exists for hosts of the library that may not call cudaMalloc -- code that lives inside another
framework's memory pool, services whose memory budget is fixed at start-up, replays of recorded
work -- and keeps its fp32 scratch in an array inside the library image.  The test calls it
through the C ABI twice in a row (with different inputs, so stale scratch contents would show)
and compares each result with the regular entry point (caller-provided workspace) and with the
CPU oracle, within the tolerance the other GPU tests use.  The buffers the TEST needs are made by
torch; the entry point itself allocates nothing.  This file sorts last on purpose."""
import ctypes as C

import numpy as np
import pytest

from frisk_b200 import runtime as R
from frisk_b200 import workloads as W


def _desc(w):
    d = R.GemmDesc()
    d.M, d.N, d.K = w.M, w.N, w.K
    d.a_type = d.b_type = w.ab_type
    d.c_type = w.c_type
    d.transA, d.transB = int(w.transA), int(w.transB)
    d.clear_accum = int(w.clear_accum)
    d.scale_mode = 0
    return d


def test_sizes_beyond_the_built_in_scratch_are_rejected():
    L = R.lib()
    cap = L.frisk_b200_gemm_skinny_static_capacity()
    assert cap == 1 << 20
    w = W.GemmWorkload("big", 64, 32768, 64, W.BF16, W.BF16)  # 2 Mi outputs > capacity
    dummy = C.c_void_p(256)
    rc = L.frisk_b200_gemm_skinny_static(C.byref(_desc(w)), dummy, dummy, dummy, None, None, None, None)
    assert rc == -9
    assert b"exceeds" in L.frisk_b200_last_error()
    assert L.frisk_b200_gemm_skinny_static(None, dummy, dummy, dummy, None, None, None, None) == -1
    w = W.GemmWorkload("wide-m", 128, 512, 64, W.BF16, W.BF16)  # not a few-row problem
    assert L.frisk_b200_gemm_skinny_static(C.byref(_desc(w)), dummy, dummy, dummy, None, None, None, None) == -2


@pytest.mark.gpu
def test_static_scratch_entry_point_matches_the_workspace_entry_point_twice_in_a_row():
    import torch

    from oracle import ref

    dev = torch.device("cuda:0")
    L = R.lib()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second must not see the first one's partial sums
    for name, dims, seed in (("cfg3", (16, 2048, 1024), 11), ("cfg3", (48, 1024, 520), 12),
                             ("cfg3", (16, 2048, 1024), 13)):
        w = W.make_workload(name, *dims, seed=seed)
        A = torch.from_numpy(w.A.view(np.int16)).to(dev)
        B = torch.from_numpy(w.B.view(np.int16)).to(dev)
        c_static = torch.full((w.M, w.N), 0x7FC0, dtype=torch.int16, device=dev)
        c_plain = torch.full((w.M, w.N), 0x7FC0, dtype=torch.int16, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)

        rc = L.frisk_b200_gemm_skinny_static(C.byref(_desc(w)), A.data_ptr(), B.data_ptr(),
                                             c_static.data_ptr(), None, None, status.data_ptr(), stream)
        assert rc == 0, L.frisk_b200_last_error()
        R.check_status(status, stream)

        plan = R.GemmPlan.for_workload(w)
        assert plan.info["kernel_name"] == "skinny"
        ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device=dev)
        plan.run(A, B, c_plain, None, None, ws, status, stream)
        R.check_status(status, stream)
        plan.close()

        got = W.bf16_decode(c_static.cpu().numpy().view(np.uint16))
        base = W.bf16_decode(c_plain.cpu().numpy().view(np.uint16))
        floor = ref.abs_dot(w)
        ok, err, metric = W.check(got, base, W.BF16, absdot=floor)  # max relative error <= 1e-2
        assert ok, f"static vs workspace entry point: {metric} = {err}"
        ok, err, metric = W.check(got, ref.ref_gemm_f64(w), W.BF16, absdot=floor)
        assert ok, f"static entry point vs oracle: {metric} = {err}"
