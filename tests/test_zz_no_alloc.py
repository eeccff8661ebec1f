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
    d.scale_mode = int(w.scale_a is not None)
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
    # the scale mode is checked like frisk_b200_gemm_plan_create checks it
    w = W.GemmWorkload("scales", 16, 512, 64, W.E4M3, W.BF16, transB=True)
    d = _desc(w)
    d.scale_mode = 7
    assert L.frisk_b200_gemm_skinny_static(C.byref(d), dummy, dummy, dummy, dummy, dummy, None, None) == -1
    d.scale_mode = 1   # scales asked for but not given
    assert L.frisk_b200_gemm_skinny_static(C.byref(d), dummy, dummy, dummy, None, None, None, None) == -1


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


def _variant(M, N, K, ab, ct, tb, clear, seed):
    rng = np.random.default_rng(seed)
    big = ab == W.E4M3
    a = (rng.standard_normal((M, K)) * (4.0 if big else 1.0)).astype(np.float32)
    b = (rng.standard_normal((K, N)) * (4.0 if big else 0.05)).astype(np.float32)
    Bq = W.encode(b, ab)
    return W.GemmWorkload("static-variant", M, N, K, ab, ct, transB=tb, clear_accum=clear,
                          A=W.encode(a, ab), B=np.ascontiguousarray(Bq.T) if tb else Bq,
                          scale_a=(rng.uniform(0.5, 2.0, M) / 448.0).astype(np.float32) if big else None,
                          scale_b=(rng.uniform(0.5, 2.0, N) / 448.0).astype(np.float32) if big else None,
                          C0=None if clear else W.encode(rng.standard_normal((M, N)).astype(np.float32), ct))


@pytest.mark.gpu
def test_static_scratch_entry_point_other_types_scales_accumulation_and_streams():
    """The corners of the finalize kernel behind the entry point: e4m3 inputs with row and column
    scales, C += A x B into a preset C, fp32 and fp16 outputs, N not divisible by 4 (the scalar
    tail), all on a stream of the caller's.  Each result is compared with the workspace entry
    point's and with the CPU oracle; the free device memory must not move across the calls."""
    import torch

    from oracle import ref

    dev = torch.device("cuda:0")
    L = R.lib()
    side = torch.cuda.Stream(device=dev)
    cases = [
        (48, 1001, 1024, W.E4M3, W.BF16, True, True, 31),    # scales, odd N
        (7, 2304, 1096, W.F16, W.F32, False, False, 32),     # fp32 C, C += A x B
        (33, 515, 520, W.F16, W.F16, True, False, 33),       # fp16 C, odd N, C += A x B
        (16, 2048, 1024, W.BF16, W.BF16, False, True, 34),
    ]
    for M, N, K, ab, ct, tb, clear, seed in cases:
        w = _variant(M, N, K, ab, ct, tb, clear, seed)
        A = torch.from_numpy(w.A.view(np.uint8).reshape(-1)).to(dev)
        B = torch.from_numpy(w.B.view(np.uint8).reshape(-1)).to(dev)
        c_init = np.zeros((M, N), W.storage_numpy_dtype(ct)) if clear else w.C0
        c_static = torch.from_numpy(c_init.view({4: np.float32, 2: np.int16}[c_init.itemsize])).to(dev)
        c_plain = c_static.clone()
        sa = None if w.scale_a is None else torch.from_numpy(w.scale_a).to(dev)
        sb = None if w.scale_b is None else torch.from_numpy(w.scale_b).to(dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        plan = R.GemmPlan.for_workload(w)
        assert plan.info["kernel_name"] == "skinny"
        ws = torch.empty(max(plan.workspace_bytes, 16), dtype=torch.uint8, device=dev)
        side.wait_stream(torch.cuda.current_stream())

        def call(c_out):
            rc = L.frisk_b200_gemm_skinny_static(C.byref(_desc(w)), A.data_ptr(), B.data_ptr(), c_out.data_ptr(),
                                                 R._ptr(sa), R._ptr(sb), status.data_ptr(), side.cuda_stream)
            assert rc == 0, L.frisk_b200_last_error()
            R.check_status(status, side.cuda_stream)

        # The first use of a kernel in a process makes the driver load its code, which takes device
        # memory once; so one call into a spare buffer first, then the free memory is read on
        # both sides of the call under test.
        call(c_static.clone())
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        call(c_static)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_before, "the entry point changed the free device memory"
        plan.run(A, B, c_plain, sa, sb, ws, status, side.cuda_stream)
        R.check_status(status, side.cuda_stream)
        plan.close()
        got = W.decode(c_static.cpu().numpy().view(W.storage_numpy_dtype(ct)), ct)
        base = W.decode(c_plain.cpu().numpy().view(W.storage_numpy_dtype(ct)), ct)
        floor = ref.abs_dot(w)
        ok, err, metric = W.check(got, base, ab, absdot=floor)
        assert ok, f"{M}x{N}x{K}: static vs workspace entry point: {metric} = {err}"
        ok, err, metric = W.check(got, ref.ref_gemm_f64(w), ab, absdot=floor)
        assert ok, f"{M}x{N}x{K}: static entry point vs oracle: {metric} = {err}"
        del ws
