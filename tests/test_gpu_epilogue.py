"""GPU parity of the whole-tile epilogue's forms, through the C ABI: rows staged through shared
memory against per-thread row stores (bit-equal), copies of C for peers (bit-equal to C), and
frisk.reduce over the columns of C folded into the epilogue (against the numpy restatement of the
op on the stored C, and against the separate reduce kernel)."""
import numpy as np
import pytest

from frisk_b200 import runtime as R
from frisk_b200 import workloads as W
from oracle import ref

pytestmark = pytest.mark.gpu

TORCH_BITS = {4: "float32", 2: "int16", 1: "uint8"}


def make(M, N, K, ab, ct, ta=False, tb=False, clear=True, seed=0):
    rng = np.random.default_rng(seed + M + 7 * N + 13 * K)
    big = ab in (W.E4M3, W.E5M2)
    a = (rng.standard_normal((M, K)) * (4.0 if big else 1.0)).astype(np.float32)
    b = (rng.standard_normal((K, N)) * (4.0 if big else K ** -0.5)).astype(np.float32)
    Aq, Bq = W.encode(a, ab), W.encode(b, ab)
    return W.GemmWorkload("epi", M, N, K, ab, ct, transA=ta, transB=tb, clear_accum=clear,
                          A=np.ascontiguousarray(Aq.T) if ta else Aq,
                          B=np.ascontiguousarray(Bq.T) if tb else Bq,
                          scale_a=(rng.uniform(0.5, 2.0, M) / 448.0).astype(np.float32) if big else None,
                          scale_b=(rng.uniform(0.5, 2.0, N) / 448.0).astype(np.float32) if big else None,
                          C0=None if clear else W.encode(rng.standard_normal((M, N)).astype(np.float32), ct))


def to_dev(torch, arr, dev):
    import torch as T

    flat = np.ascontiguousarray(arr)
    return T.from_numpy(flat.view(getattr(np, TORCH_BITS[flat.itemsize]))).to(dev)


def device_run(w, *, ldc=0, c_offset_bytes=0, peers=0, row_reduce=None, rr_clear=True, rr_init=None, **plan_kw):
    """Runs `w` on device buffers; returns (C bits [M, N], peer copies, row-reduce dst, plan info)."""
    import torch

    dev = torch.device("cuda:0")
    ldc = ldc or w.N
    cs = W.ELEM_SIZE[w.c_type]
    plan = R.GemmPlan.for_workload(w, ldc=ldc, row_reduce=row_reduce, row_reduce_clear=rr_clear, **plan_kw)
    A, B = to_dev(torch, w.A, dev), to_dev(torch, w.B, dev)
    sa = None if w.scale_a is None else torch.from_numpy(w.scale_a).to(dev)
    sb = None if w.scale_b is None else torch.from_numpy(w.scale_b).to(dev)

    def c_buffer():
        buf = torch.full((w.M * ldc * cs + 64,), 0xA5, dtype=torch.uint8, device=dev)
        if not w.clear_accum:
            init = np.full((w.M, ldc), 0, W.storage_numpy_dtype(w.c_type))
            init[:, :w.N] = w.C0
            buf[c_offset_bytes:c_offset_bytes + w.M * ldc * cs] = torch.from_numpy(init.view(np.uint8).reshape(-1)).to(dev)
        return buf

    bufs = [c_buffer() for _ in range(1 + peers)]
    ws = torch.empty(max(plan.workspace_bytes, 16), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rr = None
    if row_reduce:
        rr0 = rr_init if rr_init is not None else np.zeros(w.M, W.storage_numpy_dtype(w.c_type))
        rr = to_dev(torch, rr0, dev)
    plan.run_ex(A, B, bufs[0].data_ptr() + c_offset_bytes, scale_a=sa, scale_b=sb, workspace=ws,
                status=status, row_reduce_dst=rr, peers=[b.data_ptr() + c_offset_bytes for b in bufs[1:]])
    R.check_status(status)
    info = plan.info
    plan.close()

    def rows_of(buf):
        raw = buf[c_offset_bytes:c_offset_bytes + w.M * ldc * cs].cpu().numpy().view(W.storage_numpy_dtype(w.c_type))
        full = raw.reshape(w.M, ldc)
        return np.ascontiguousarray(full[:, :w.N]), full[:, w.N:]

    outs = [rows_of(b) for b in bufs]
    for _, padding in outs:   # nothing beyond the N columns of a row is written
        assert (padding.view(np.uint8) == 0xA5).all() or not w.clear_accum
    rr_host = None if rr is None else rr.cpu().numpy().view(W.storage_numpy_dtype(w.c_type))
    return outs[0][0], [o[0] for o in outs[1:]], rr_host, info


CASES = [
    # M, N, K, ab, ct, transA, transB, clear, kernel
    (512, 768, 320, W.BF16, W.BF16, False, False, True, "tcgen05_pair"),
    (300, 520, 136, W.F16, W.F32, False, True, True, "tcgen05_pair"),     # fp32 C: 32-column pieces
    (260, 1000, 200, W.F16, W.F16, False, False, False, "tcgen05_pair"),  # ragged rows and columns, C +=
    (384, 512, 512, W.E4M3, W.BF16, False, True, True, "tcgen05_pair"),   # scales
    (300, 328, 272, W.E5M2, W.BF16, False, True, True, "tcgen05_pair"),   # e5m2, scales, ragged
    (128, 256, 192, W.BF16, W.BF16, True, False, True, "tcgen05"),        # one-CTA kernel
    (100, 200, 64, W.F16, W.F16, False, False, True, "tcgen05"),
    (1000, 1000, 1000, W.BF16, W.F16, False, False, True, "tcgen05_pair"),
]


@pytest.mark.parametrize("M,N,K,ab,ct,ta,tb,clear,kernel", CASES)
def test_staged_and_direct_epilogues_give_the_same_bits(M, N, K, ab, ct, ta, tb, clear, kernel):
    w = make(M, N, K, ab, ct, ta, tb, clear)
    staged, _, _, info = device_run(w, epilogue=2, force_kernel=kernel)
    direct, _, _, info1 = device_run(w, epilogue=1, force_kernel=kernel)
    assert info["kernel_name"] == kernel == info1["kernel_name"]
    assert np.array_equal(staged, direct)
    linear, _, _, _ = device_run(w, epilogue=3, force_kernel=kernel)   # unswizzled staging rows
    assert np.array_equal(linear, direct)
    ok, err, metric = W.check(W.decode(staged, ct), ref.ref_gemm_f64(w), ab, absdot=ref.abs_dot(w))
    assert ok, f"{metric} = {err}"
    # a padded row pitch keeps the staged form as long as rows stay 16-byte aligned ...
    padded, _, _, _ = device_run(w, epilogue=2, force_kernel=kernel, ldc=N + 32)
    assert np.array_equal(padded, direct)
    # ... and a C that is not 16-byte aligned falls back to element stores with the same bits
    shifted, _, _, _ = device_run(w, epilogue=2, force_kernel=kernel, ldc=N + 3,
                                  c_offset_bytes=W.ELEM_SIZE[ct])
    assert np.array_equal(shifted, direct)
    # TMA tensor stores out of the staging buffers (the CTA-pair kernel; the one-CTA kernel takes
    # the option as "staged"): the hardware clips the ragged last rows and columns
    tma, _, _, _ = device_run(w, epilogue=4, force_kernel=kernel)
    assert np.array_equal(tma, direct)
    tma_padded, _, _, _ = device_run(w, epilogue=4, force_kernel=kernel, ldc=N + 32)
    assert np.array_equal(tma_padded, direct)
    # rows off the 16-byte grid (pitch, then base): no tensor map exists, the run stores without TMA
    tma_shifted, _, _, _ = device_run(w, epilogue=4, force_kernel=kernel, ldc=N + 3,
                                      c_offset_bytes=W.ELEM_SIZE[ct])
    assert np.array_equal(tma_shifted, direct)
    tma_base, _, _, _ = device_run(w, epilogue=4, force_kernel=kernel, ldc=N + 32,
                                   c_offset_bytes=W.ELEM_SIZE[ct])
    assert np.array_equal(tma_base, direct)


@pytest.mark.parametrize("M,N,K,ab,ct,ta,tb,clear,kernel", CASES[:5])
@pytest.mark.parametrize("epilogue", [1, 2, 4])
def test_peer_copies_equal_c(M, N, K, ab, ct, ta, tb, clear, kernel, epilogue):
    """The all-gather folded into the epilogue: every destination gets the bits of C.  The peer
    buffers live on the same GPU here; across GPUs only the pointers differ."""
    w = make(M, N, K, ab, ct, ta, tb, clear, seed=3)
    base, _, _, _ = device_run(w, epilogue=epilogue, force_kernel=kernel)
    for n_peers in (1, 7):
        c, peers, _, _ = device_run(w, epilogue=epilogue, force_kernel=kernel, peers=n_peers)
        assert np.array_equal(c, base)
        for q in peers:
            assert np.array_equal(q, base)


def reduce_tolerance(kind, want, mag, dtype):
    ulp = {W.F32: 2.0 ** -23, W.F16: 2.0 ** -10, W.BF16: 2.0 ** -7}[dtype]
    if kind in ("min", "max"):
        return np.zeros_like(want)
    return 1e-5 * mag + ulp * np.abs(want)


@pytest.mark.parametrize("kind", ["max", "add", "min"])
@pytest.mark.parametrize("M,N,K,ab,ct,ta,tb,clear,kernel", [CASES[0], CASES[1], CASES[2], CASES[3], CASES[4],
                                                           (2048, 4096, 256, W.BF16, W.BF16, False, False, True, "tcgen05_pair")])
def test_row_reduce_in_the_epilogue_matches_a_reduce_of_the_stored_c(M, N, K, ab, ct, ta, tb, clear, kernel, kind):
    w = make(M, N, K, ab, ct, ta, tb, clear, seed=5)
    plain, _, _, _ = device_run(w, force_kernel=kernel)
    for epilogue in (1, 2, 4):
        c, _, got, info = device_run(w, force_kernel=kernel, epilogue=epilogue, row_reduce=kind)
        assert info["kernel_name"] == kernel
        assert np.array_equal(c, plain), "the fold must not change C"
        want, mag = ref.ref_reduce(c, 1, ct, kind)
        err = np.abs(W.decode(got, ct).astype(np.float64) - want)
        assert (err <= reduce_tolerance(kind, want, mag, ct)).all(), (kind, float(err.max()))
        # the separate reduce kernel on the stored C: same values for min / max
        if kind in ("min", "max"):
            dst = np.zeros(M, got.dtype)
            R.reduce_host(c, dst, 1, ct, kind)
            assert np.array_equal(dst, got)
    # clear = 0 folds the old destination in; run to run the sum is the same bits
    init = W.encode(np.random.default_rng(1).standard_normal(M).astype(np.float32), ct)
    _, _, got0, _ = device_run(w, force_kernel=kernel, row_reduce=kind, rr_clear=False, rr_init=init)
    _, _, got1, _ = device_run(w, force_kernel=kernel, row_reduce=kind, rr_clear=False, rr_init=init)
    assert np.array_equal(got0, got1)
    want, mag = ref.ref_reduce(plain, 1, ct, kind, clear=False, dst0=init)
    err = np.abs(W.decode(got0, ct).astype(np.float64) - want)
    assert (err <= reduce_tolerance(kind, want, mag, ct)).all(), (kind, float(err.max()))


def test_row_reduce_needs_a_whole_tile_tensor_core_plan():
    with pytest.raises(R.FriskError) as e:
        R.GemmPlan(64, 64, 64, W.F32, row_reduce="max")
    assert e.value.code == -2
    p = R.GemmPlan(16, 4096, 1024, W.BF16, row_reduce="max")   # a few-row shape: whole tiles instead
    assert p.info["kernel_name"] == "tcgen05" and p.workspace_bytes > 0
    p.close()


@pytest.mark.parametrize("M,N,K,ab,ct,ta,tb", [(1536, 2304, 256, W.BF16, W.BF16, False, False),
                                               (1000, 1000, 520, W.F16, W.F16, False, True),
                                               (768, 1280, 512, W.E4M3, W.BF16, False, True)])
def test_tile_walks_and_l2_hints_do_not_change_the_bits(M, N, K, ab, ct, ta, tb):
    """Bands of tile rows, panels of tile columns, and the L2 eviction hints of the loads are
    about where the bytes come from, never about what is computed."""
    w = make(M, N, K, ab, ct, ta, tb, seed=8)
    base, _, _, info = device_run(w, force_kernel="tcgen05_pair")
    ok, err, metric = W.check(W.decode(base, ct), ref.ref_gemm_f64(w), ab, absdot=ref.abs_dot(w))
    assert ok, f"{metric} = {err}"
    for kw in (dict(panel_tiles=1), dict(panel_tiles=2), dict(panel_tiles=3, l2_hints=3), dict(panel_tiles=64),
               dict(band_tiles=2, l2_hints=1), dict(l2_hints=2)):
        got, _, _, _ = device_run(w, force_kernel="tcgen05_pair", **kw)
        assert np.array_equal(got, base), kw
