"""GPU parity: the CUDA kernels, called through the C ABI, against the CPU oracle on the same
seeded inputs.  Tolerances (written where they are applied, frisk_b200/workloads.py::check):
fp32 -> relative Frobenius error <= 1e-4; fp16/bf16 -> max relative error <= 1e-2;
e4m3 (after scaling) -> max relative error <= 2e-2.  Full-size configurations are checked on
sampled rows plus size-independent properties (exact scaling by two, row-permutation equivariance,
zero-padding of K, run-to-run bit equality for the kernels that do not use atomics)."""
import numpy as np
import pytest

from frisk_b200 import runtime as R
from frisk_b200 import workloads as W
from oracle import ref

pytestmark = pytest.mark.gpu


def sub_rows(w, rows):
    """The workload restricted to some rows of A (and of C): what the oracle is run on when the
    full problem is too large for a CPU loop."""
    s = W.GemmWorkload(w.name, len(rows), w.N, w.K, w.ab_type, w.c_type, transA=w.transA,
                       transB=w.transB, clear_accum=w.clear_accum, seed=w.seed, B=w.B,
                       scale_b=w.scale_b)
    s.A = np.ascontiguousarray(w.A[:, rows] if w.transA else w.A[rows])
    s.scale_a = None if w.scale_a is None else w.scale_a[rows]
    s.C0 = None if w.C0 is None else w.C0[rows]
    return s


def torch_matmul_fp32(w):
    """torch.matmul on the CPU in fp32 over the exactly decoded operands: the one GEMM arithmetic
    the reference itself ever runs (exp/layout/analyze_bank_conflicts.py:142-143, there on random
    tiles as its timing baseline).  Scales and the C += term are applied in float64 afterwards."""
    import torch

    a = torch.from_numpy(np.ascontiguousarray(w.a_logical(), dtype=np.float32))
    b = torch.from_numpy(np.ascontiguousarray(w.b_logical(), dtype=np.float32))
    c = torch.matmul(a, b).numpy().astype(np.float64)
    if w.scale_a is not None:
        c = c * w.scale_a.astype(np.float64)[:, None] * w.scale_b.astype(np.float64)[None, :]
    if not w.clear_accum and w.C0 is not None:
        c = c + W.decode(w.C0, w.c_type).astype(np.float64)
    return c


METRICS_SEEN = []  # (case, metrics) of every checked result, printed at the end of the session


def run_and_check(w, rows=None, **plan_kw):
    """Runs the workload through the C ABI and compares it with three CPU results: the float64
    product, the fp32 C loop of the oracle and torch.matmul in fp32.  The bound is applied to two
    error metrics: the one with the floor relative to the data behind each output
    (W.max_rel_error with `absdot`), and -- for 16-bit and 8-bit inputs -- the one with the floor
    1e-3 rms(R); fp32 inputs are held to the relative Frobenius error."""
    plan = R.GemmPlan.for_workload(w, **plan_kw)
    info = plan.info
    plan.close()
    out = R.gemm_host(w, **plan_kw)
    got = W.decode(out, w.c_type)
    wo = w
    if rows is not None:
        got = got[rows]
        wo = sub_rows(w, rows)
    want64 = ref.ref_gemm_f64(wo)
    floor = ref.abs_dot(wo)
    oracle = W.decode(ref.ref_gemm(wo), wo.c_type)
    what = f"{w.name} {w.M}x{w.N}x{w.K} via {info['kernel_name']}"
    ok, err, metric = W.check(got, want64, w.ab_type, absdot=floor)
    assert ok, f"{what}: {metric} = {err:.3e} vs float64"
    ok, err, metric = W.check(got, oracle, w.ab_type, absdot=floor)
    assert ok, f"{what}: {metric} = {err:.3e} vs the fp32 oracle"
    ok, err, metric = W.check(got, torch_matmul_fp32(wo), w.ab_type, absdot=floor)
    assert ok, f"{what}: {metric} = {err:.3e} vs torch.matmul (CPU, fp32)"
    bound = W.TOLERANCE[w.ab_type][1]
    m = W.parity_metrics(got, want64, floor, bound)
    METRICS_SEEN.append((what, m))
    if w.ab_type != W.F32:
        if w.K <= 4096:
            assert m["max_rel_rms_floor"] <= bound, f"{what}: rms-floor metric {m['max_rel_rms_floor']:.3e} > {bound}"
        else:
            # Longer sums: an output that cancels to far below rms(R) keeps the fp32 accumulation
            # error of the 8192 products behind it, which can pass 1e-2 of the rms floor.  Such
            # outputs must be rare (at most one in 10^4) and cancellation-sized (under 1 % of a
            # typical output); everywhere else the rms-floor bound holds too.
            assert m["over_bound_rms_floor"] <= 1e-4 and m["over_bound_largest_ref"] <= 1e-2, (what, m)
    return out, info


@pytest.fixture(scope="module", autouse=True)
def report_metrics():
    yield
    print("\nparity metrics (vs float64): case | rel. Frobenius | max rel, rms floor | max rel, data floor | share below rms floor | share over the bound (rms floor)")
    for what, m in METRICS_SEEN:
        print(f"  {what} | {m['rel_frobenius']:.3e} | {m['max_rel_rms_floor']:.3e} | "
              f"{m['max_rel_data_floor']:.3e} | {m['below_rms_floor']:.2e} | {m['over_bound_rms_floor']:.2e}")


# ----------------------------------------------------------------------------- small cases
SMALL = [
    # (workload, (M, N, K), expected kernel)
    ("cfg1", (512, 512, 512), "simt"),
    ("cfg1", (70, 50, 33), "simt"),
    ("cfg1", (1, 1, 1), "simt"),
    ("cfg2", (128, 256, 64), "tcgen05"),
    ("cfg2", (128, 64, 128), "tcgen05"),
    ("cfg2", (256, 512, 512), "tcgen05_pair"),
    ("cfg2", (200, 300, 136), "tcgen05_pair"),
    ("cfg2", (1, 8, 8), "tcgen05"),
    ("cfg5", (128, 256, 64), "tcgen05"),
    ("cfg5", (520, 392, 264), "tcgen05_pair"),
    ("cfg5", (130, 264, 72), "tcgen05_pair"),
    ("cfg4", (128, 256, 128), "tcgen05"),
    ("cfg4", (200, 300, 400), "tcgen05_pair"),
    ("cfg3", (16, 256, 64), "skinny"),
    ("cfg3", (16, 1024, 4096), "skinny"),
    ("cfg3", (5, 1000, 520), "skinny"),
    ("cfg3", (48, 2048, 1024), "skinny"),
    ("cfg3", (64, 512, 256), "skinny"),
]


@pytest.mark.parametrize("name,dims,kernel", SMALL)
def test_small_cases_match_oracle(name, dims, kernel):
    w = W.make_workload(name, *dims)
    _, info = run_and_check(w)
    assert info["kernel_name"] == kernel


@pytest.mark.parametrize("force", ["simt", "tcgen05", "tcgen05_pair"])
@pytest.mark.parametrize("name,dims", [("cfg2", (300, 200, 136)), ("cfg5", (520, 392, 264)),
                                       ("cfg4", (256, 256, 256))])
def test_every_kernel_family_agrees(name, dims, force):
    w = W.make_workload(name, *dims)
    _, info = run_and_check(w, force_kernel=force)
    assert info["kernel_name"] == force


def test_tile_width_and_stage_overrides():
    w = W.make_workload("cfg2", 384, 640, 320)
    for tile_n in (64, 128, 256):
        for stages in (1, 2, 3, 0):  # 1 is raised to 2: the pipeline needs two stages
            _, info = run_and_check(w, tile_n=tile_n, stages=stages, force_kernel="tcgen05")
            assert info["tile_n"] == tile_n and info["stages"] >= 2
    _, info = run_and_check(w, num_ctas=3, force_kernel="tcgen05")
    assert info["num_ctas"] == 3
    w = W.make_workload("cfg3", 16, 2048, 2048)
    for ctas in (1, 7, 0):
        run_and_check(w, num_ctas=ctas)


@pytest.mark.parametrize("ab", [W.F32, W.F16, W.BF16])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_all_storage_orders(ab, ta, tb):
    rng = np.random.default_rng(11)
    M, N, K = 136, 264, 200
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = (rng.standard_normal((K, N)) * 0.1).astype(np.float32)
    w = W.GemmWorkload("orders", M, N, K, ab, ab, transA=ta, transB=tb,
                       A=np.ascontiguousarray(W.encode(a, ab).T if ta else W.encode(a, ab)),
                       B=np.ascontiguousarray(W.encode(b, ab).T if tb else W.encode(b, ab)))
    _, info = run_and_check(w)
    assert info["kernel_name"] == ("simt" if ab == W.F32 else "tcgen05_pair")  # M = 136 > 128


@pytest.mark.parametrize("name,dims", [("cfg1", (96, 80, 64)), ("cfg2", (256, 256, 128)),
                                       ("cfg3", (16, 512, 512)), ("cfg4", (128, 256, 256))])
def test_accumulate_into_c(name, dims):
    w = W.make_workload(name, *dims)
    rng = np.random.default_rng(5)
    w.clear_accum = False
    w.C0 = W.encode(rng.standard_normal((w.M, w.N)).astype(np.float32), w.c_type)
    run_and_check(w)


def test_mixed_output_types_and_padded_leading_dimensions():
    rng = np.random.default_rng(9)
    M, N, K = 130, 200, 96
    for ct in (W.F32, W.F16, W.BF16):
        w = W.make_workload("cfg5", M, N, K)
        w.c_type = ct
        run_and_check(w)
    # leading dimensions larger than the rows: lda = K + 8, ldb = N + 16, ldc = N + 24
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal((K, N)).astype(np.float32)
    A = np.zeros((M, K + 8), np.uint16)
    B = np.zeros((K, N + 16), np.uint16)
    A[:, :K] = W.bf16_encode(a)
    B[:, :N] = W.bf16_encode(b)
    Cbuf = np.full((M, N + 24), 0x7FC0, np.uint16)  # NaN canaries in the padding
    plan = R.GemmPlan(M, N, K, W.BF16, lda=K + 8, ldb=N + 16, ldc=N + 24)
    assert plan.info["kernel_name"] == "tcgen05_pair"  # M = 130 > 128
    plan.run_host(A, B, Cbuf)
    plan.close()
    assert (Cbuf[:, N:] == 0x7FC0).all(), "the kernel wrote outside its columns"
    w = W.GemmWorkload("ld", M, N, K, W.BF16, W.BF16, A=W.bf16_encode(a), B=W.bf16_encode(b))
    ok, err, _ = W.check(W.bf16_decode(Cbuf[:, :N]), ref.ref_gemm_f64(w), W.BF16, absdot=ref.abs_dot(w))
    assert ok, err


@pytest.mark.parametrize("M,N,K,ab,ta,tb,pad_a,pad_b,want", [
    (300, 5000, 700, W.BF16, False, False, 0, 0, "tcgen05_pair"),   # K = 700: 1400-byte rows of A
    (260, 333, 264, W.F16, False, True, 3, 5, "tcgen05_pair"),      # both pitches odd, B stored [N, K]
    (100, 520, 137, W.BF16, True, False, 1, 0, "tcgen05"),          # A stored [K, M], 202-byte rows
    (16, 4096, 1000, W.F16, False, True, 0, 1, "skinny"),           # few rows on repacked weights
    (256, 384, 200, W.E4M3, False, True, 0, 0, "tcgen05_pair"),     # 8-bit: 200-byte rows
])
def test_odd_row_pitches_run_on_the_tensor_cores_after_a_repack(M, N, K, ab, ta, tb, pad_a, pad_b, want):
    """Operands whose row pitch is not a multiple of 16 bytes are copied into the workspace at a
    padded pitch and run on the tensor cores; the bits equal those of the same values handed over
    in buffers with 16-byte pitches, and the oracle's tolerance holds."""
    rng = np.random.default_rng(M + N + K)
    fp8 = ab in (W.E4M3, W.E5M2)
    ct = W.BF16 if fp8 else ab
    a = (rng.standard_normal((M, K)) * (4.0 if fp8 else 1.0)).astype(np.float32)
    b = (rng.standard_normal((K, N)) * (4.0 if fp8 else K ** -0.5)).astype(np.float32)
    Aq, Bq = W.encode(a, ab), W.encode(b, ab)
    As = np.ascontiguousarray(Aq.T) if ta else Aq
    Bs = np.ascontiguousarray(Bq.T) if tb else Bq
    sa = (rng.uniform(0.5, 2.0, M) / 448.0).astype(np.float32) if fp8 else None
    sb = (rng.uniform(0.5, 2.0, N) / 448.0).astype(np.float32) if fp8 else None
    es = W.ELEM_SIZE[ab]

    def padded(x, extra):   # the same rows at a pitch `extra` elements longer, canaries in the padding
        out = np.full((x.shape[0], x.shape[1] + extra), 0x7F if es == 1 else 0x7E01, x.dtype if es == 1 else np.uint16)
        out[:, :x.shape[1]] = x.view(out.dtype)
        return out

    def run(A, B):
        plan = R.GemmPlan(M, N, K, ab, ct, transA=ta, transB=tb, lda=A.shape[1], ldb=B.shape[1], scales=fp8)
        out = np.zeros((M, N), W.storage_numpy_dtype(ct))
        plan.run_host(A, B, out, sa, sb)
        info = plan.info
        plan.close()
        return out, info

    odd_a, odd_b = padded(As, pad_a), padded(Bs, pad_b)
    assert (odd_a.shape[1] * es) % 16 or (odd_b.shape[1] * es) % 16
    got, info = run(odd_a, odd_b)
    assert info["kernel_name"] == want and info["cuda_core_reason"] == 0
    n_odd = int(bool((odd_a.shape[1] * es) % 16)) + int(bool((odd_b.shape[1] * es) % 16))
    # the same values at 16-byte pitches: no repack, the same kernel, the same bits
    q = 16 // es
    even, info0 = run(padded(As, -As.shape[1] % q), padded(Bs, -Bs.shape[1] % q))
    assert info0["kernel_name"] == want and info["launches"] == info0["launches"] + n_odd
    assert np.array_equal(got, even)
    w = W.GemmWorkload("odd", M, N, K, ab, ct, transA=ta, transB=tb, A=As, B=Bs, scale_a=sa, scale_b=sb)
    ok, err, metric = W.check(W.decode(got, ct), ref.ref_gemm_f64(w), ab, absdot=ref.abs_dot(w))
    assert ok, f"{metric} = {err}"


def test_guard_bands_around_c_and_workspace_stay_untouched():
    torch = pytest.importorskip("torch")
    dev = torch.device("cuda:0")
    for name, dims in (("cfg2", (200, 300, 136)), ("cfg3", (16, 1000, 520)), ("cfg1", (70, 50, 33))):
        w = W.make_workload(name, *dims)
        plan = R.GemmPlan.for_workload(w)
        cs = W.ELEM_SIZE[w.c_type]
        guard = 4096
        cbuf = torch.full((guard * 2 + w.M * w.N * cs,), 0xAB, dtype=torch.uint8, device=dev)
        wsbuf = torch.full((guard * 2 + max(plan.workspace_bytes, 16),), 0xCD, dtype=torch.uint8, device=dev)
        A = torch.from_numpy(np.ascontiguousarray(w.A).view(np.uint8).reshape(-1)).to(dev)
        B = torch.from_numpy(np.ascontiguousarray(w.B).view(np.uint8).reshape(-1)).to(dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        ws_ptr = wsbuf.data_ptr() + guard
        rc = R.lib().frisk_b200_gemm_run(plan._h, A.data_ptr(), B.data_ptr(), cbuf.data_ptr() + guard,
                                         None, None, ws_ptr, plan.workspace_bytes, status.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        R.check_status(status)
        assert (cbuf[:guard] == 0xAB).all() and (cbuf[-guard:] == 0xAB).all()
        assert (wsbuf[:guard] == 0xCD).all() and (wsbuf[guard + plan.workspace_bytes:] == 0xCD).all()
        got = cbuf[guard:guard + w.M * w.N * cs].cpu().numpy().view(W.storage_numpy_dtype(w.c_type))
        ok, err, _ = W.check(W.decode(got.reshape(w.M, w.N), w.c_type), ref.ref_gemm_f64(w), w.ab_type,
                             absdot=ref.abs_dot(w))
        assert ok, err
        plan.close()


def test_run_argument_errors_on_device():
    torch = pytest.importorskip("torch")
    w = W.make_workload("cfg3", 16, 512, 512)
    plan = R.GemmPlan.for_workload(w)
    dev = torch.device("cuda:0")
    buf = torch.zeros(16 * 512 * 512, dtype=torch.uint8, device=dev)
    L = R.lib()
    # split plan without a workspace / with a short one
    assert L.frisk_b200_gemm_run(plan._h, buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), None, None,
                                 None, 0, None, None) == -4
    assert L.frisk_b200_gemm_run(plan._h, buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), None, None,
                                 buf.data_ptr(), 16, None, None) == -4
    plan.close()
    w = W.make_workload("cfg4", 128, 128, 128)
    plan = R.GemmPlan.for_workload(w)
    assert L.frisk_b200_gemm_run(plan._h, buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), None, None,
                                 None, 0, None, None) == -1  # scales requested but missing
    plan.close()


def test_misaligned_pointers_take_the_cuda_core_kernel():
    torch = pytest.importorskip("torch")
    dev = torch.device("cuda:0")
    w = W.make_workload("cfg5", 128, 128, 128)
    plan = R.GemmPlan.for_workload(w)
    assert plan.info["kernel_name"] == "tcgen05"
    A = torch.zeros(w.A.size * 2 + 64, dtype=torch.uint8, device=dev)
    A[2:2 + w.A.size * 2] = torch.from_numpy(w.A.view(np.uint8).reshape(-1)).to(dev)  # 2-byte offset
    B = torch.from_numpy(w.B.view(np.uint8).reshape(-1)).to(dev)
    Cd = torch.zeros(w.M * w.N * 2, dtype=torch.uint8, device=dev)
    plan.run(A.data_ptr() + 2, B, Cd)
    torch.cuda.synchronize()
    got = W.bf16_decode(Cd.cpu().numpy().view(np.uint16).reshape(w.M, w.N))
    ok, err, _ = W.check(got, ref.ref_gemm_f64(w), W.BF16, absdot=ref.abs_dot(w))
    assert ok, err
    # the slow run is counted and noted, not silent
    assert plan.refresh_info()["cuda_core_runs"] == 1 and plan.info["kernel_name"] == "tcgen05"
    assert b"not 16-byte aligned" in R.lib().frisk_b200_last_error()
    plan.close()


@pytest.mark.parametrize("M,N,K,ct,clear,ldx", [
    (512, 512, 512, W.F32, True, 0),     # the fp32 configuration
    (64, 128, 96, W.F32, False, 4),      # three slices, C +=, padded pitches
    (96, 64, 32, W.BF16, True, 0),       # one slice, bf16 C
])
def test_fp32_pipelined_cuda_core_kernel_gives_the_generic_kernels_bits(M, N, K, ct, clear, ldx):
    """fp32 problems without edges (rows of 32, columns of 64, K of 32, 16-byte aligned row-major
    A and B) run on the cp.async-pipelined CUDA-core kernel; it adds the same products in the same
    order as the generic kernel, which the same problem takes when A sits 4 bytes off the 16-byte
    grid.  Both must give the same bits, and the oracle's."""
    torch = pytest.importorskip("torch")
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(M + N + K)
    a = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    c0 = rng.uniform(-1, 1, (M, N)).astype(np.float32)
    lda, ldb = K + ldx, N + ldx
    Ah = np.zeros((M, lda), np.float32); Ah[:, :K] = a
    Bh = np.zeros((K, ldb), np.float32); Bh[:, :N] = b
    w = W.GemmWorkload("f32-pipe", M, N, K, W.F32, ct, clear_accum=clear, A=a, B=b,
                       C0=None if clear else W.encode(c0, ct))
    plan = R.GemmPlan(M, N, K, W.F32, ct, lda=lda, ldb=ldb, clear_accum=clear)
    assert plan.info["kernel_name"] == "simt" and plan.info["tile_m"] == 32
    Bd = torch.from_numpy(Bh).to(dev)
    abuf = torch.zeros(M * lda + 4, dtype=torch.float32, device=dev)
    outs = []
    for off in (0, 1):   # aligned: pipelined kernel; one float further: the generic one
        abuf.zero_()
        Ad = abuf[off:off + M * lda].view(M, lda)
        Ad.copy_(torch.from_numpy(Ah))
        Cd = torch.from_numpy(np.ascontiguousarray(w.C0 if not clear else W.encode(np.zeros((M, N), np.float32), ct))
                              .view(np.int32 if ct == W.F32 else np.int16)).to(dev)
        plan.run(Ad, Bd, Cd)
        torch.cuda.synchronize()
        outs.append(Cd.cpu().numpy().view(W.storage_numpy_dtype(ct)))
    plan.close()
    assert np.array_equal(outs[0], outs[1])
    got = W.decode(outs[0], ct)
    # (a 16-bit C is held to the 16-bit bound: its last rounding is what the error is then)
    ok, err, metric = W.check(got, ref.ref_gemm_f64(w), ct, absdot=ref.abs_dot(w))
    assert ok, (metric, err)


def test_stream_k_workspace_may_be_shared_and_dirty():
    """The workspace is scratch: two stream-K plans with different slot sizes run alternately on
    ONE buffer, and a buffer handed back full of other bytes, give the same bits as private,
    zero-filled buffers (the arrival counters behind the slots are cleared on every run)."""
    torch = pytest.importorskip("torch")
    dev = torch.device("cuda:0")
    w1 = W.make_workload("cfg3", 16, 512, 4096)            # two tiles: stream-K
    w2 = W.make_workload("cfg3", 24, 4096, 2048, seed=9)   # forced grid: stream-K
    p1 = R.GemmPlan.for_workload(w1)
    p2 = R.GemmPlan.for_workload(w2, num_ctas=37)
    assert p1.workspace_bytes > 0 and p2.workspace_bytes > 0 and p1.workspace_bytes != p2.workspace_bytes
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    bufs = {}
    for w in (w1, w2):
        bufs[w.seed, "A"] = torch.from_numpy(w.A.view(np.int16)).to(dev)
        bufs[w.seed, "B"] = torch.from_numpy(w.B.view(np.int16)).to(dev)

    def run(plan, w, ws):
        out = torch.full((w.M, w.N), 0x7FC0, dtype=torch.int16, device=dev)
        plan.run(bufs[w.seed, "A"], bufs[w.seed, "B"], out, None, None, ws, status)
        R.check_status(status)
        return out.cpu().numpy()

    want1 = run(p1, w1, torch.zeros(p1.workspace_bytes, dtype=torch.uint8, device=dev))
    want2 = run(p2, w2, torch.zeros(p2.workspace_bytes, dtype=torch.uint8, device=dev))
    shared = torch.zeros(max(p1.workspace_bytes, p2.workspace_bytes), dtype=torch.uint8, device=dev)
    for _ in range(3):
        assert np.array_equal(run(p1, w1, shared), want1)
        assert np.array_equal(run(p2, w2, shared), want2)
    shared.fill_(0xCD)   # what a caching allocator may hand back
    assert np.array_equal(run(p1, w1, shared), want1)
    shared.fill_(0xCD)
    assert np.array_equal(run(p2, w2, shared), want2)
    ok, err, _ = W.check(W.bf16_decode(want1.view(np.uint16)), ref.ref_gemm_f64(w1), W.BF16, absdot=ref.abs_dot(w1))
    assert ok, err
    p1.close()
    p2.close()


def test_status_word_maps_to_device_timeout():
    """The host side of the bounded waits: a status word a kernel ORed a code into comes back as
    FRISK_ERR_DEVICE_TIMEOUT with the word in the error text.  The word is set from the host here;
    no kernel is made to give up."""
    torch = pytest.importorskip("torch")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    R.check_status(status)
    status.fill_(0x5)
    with pytest.raises(R.FriskError) as e:
        R.check_status(status)
    assert e.value.code == -6 and "0x5" in str(e.value)
    assert R.lib().frisk_b200_check_status(None, None) == 0   # no status word: nothing to report


def _tight_host_buffer(rows, ld, row_elems, dtype, fill):
    """A host array of exactly (rows - 1) * ld + row_elems elements that ENDS at a page boundary
    followed by an unreadable page: reading one element past the last row's elements faults."""
    import ctypes
    import mmap

    page = mmap.PAGESIZE
    n = (rows - 1) * ld + row_elems
    nbytes = n * np.dtype(dtype).itemsize
    pages = -(-nbytes // page)
    m = mmap.mmap(-1, (pages + 1) * page)
    base = ctypes.addressof(ctypes.c_char.from_buffer(m))
    libc = ctypes.CDLL(None, use_errno=True)
    assert libc.mprotect(ctypes.c_void_p(base + pages * page), ctypes.c_size_t(page), 0) == 0
    arr = np.frombuffer(m, dtype=dtype, count=n, offset=pages * page - nbytes)
    view = np.lib.stride_tricks.as_strided(arr, (rows, row_elems), (ld * arr.itemsize, arr.itemsize))
    view[...] = fill
    return m, arr, view


def test_host_buffers_sized_to_the_last_element_are_enough():
    """Leading dimensions larger than the rows, host buffers of (rows - 1) * ld + row length
    elements (the BLAS convention) placed so that any read past their end faults: the host-buffer
    call reads and writes only the elements of each row."""
    rng = np.random.default_rng(21)
    M, N, K = 136, 200, 96
    lda, ldb, ldc = K + 8, N + 16, N + 24
    a = W.bf16_encode(rng.standard_normal((M, K)).astype(np.float32))
    b = W.bf16_encode(rng.standard_normal((K, N)).astype(np.float32))
    c0 = W.bf16_encode(rng.standard_normal((M, N)).astype(np.float32))
    keep = [_tight_host_buffer(M, lda, K, np.uint16, a), _tight_host_buffer(K, ldb, N, np.uint16, b),
            _tight_host_buffer(M, ldc, N, np.uint16, c0)]
    (_, A, _), (_, B, _), (_, Cbuf, Cview) = keep
    plan = R.GemmPlan(M, N, K, W.BF16, lda=lda, ldb=ldb, ldc=ldc, clear_accum=False)
    rc = R.lib().frisk_b200_gemm_run_host(plan._h, A.ctypes.data, B.ctypes.data, Cbuf.ctypes.data, None, None)
    assert rc == 0
    plan.close()
    w = W.GemmWorkload("tight", M, N, K, W.BF16, W.BF16, A=a, B=b, clear_accum=False, C0=c0)
    ok, err, _ = W.check(W.bf16_decode(np.ascontiguousarray(Cview)), ref.ref_gemm_f64(w), W.BF16,
                         absdot=ref.abs_dot(w))
    assert ok, err


# ----------------------------------------------------------------------------- exact properties
@pytest.mark.parametrize("name,dims", [("cfg2", (512, 768, 1024)), ("cfg5", (512, 768, 1024)),
                                       ("cfg4", (512, 512, 1024)), ("cfg1", (200, 136, 300))])
def test_exact_properties(name, dims):
    w = W.make_workload(name, *dims)
    base = R.gemm_host(w)
    # bit-identical on a second run (no atomics in these kernels)
    assert np.array_equal(base, R.gemm_host(w))
    # permuting the rows of A permutes the rows of C bit-exactly
    perm = np.random.default_rng(1).permutation(w.M)
    w2 = W.make_workload(name, *dims)
    w2.A = np.ascontiguousarray(w.A[perm])
    if w2.scale_a is not None:
        w2.scale_a = w.scale_a[perm]
    assert np.array_equal(R.gemm_host(w2), base[perm])
    # doubling A doubles C exactly (power-of-two scaling commutes with rounding; not for fp16
    # outputs, whose subnormal results round on a fixed grid, nor for the saturating e4m3 inputs)
    if name in ("cfg1", "cfg5"):
        w3 = W.make_workload(name, *dims)
        w3.A = W.encode(W.decode(w.A, w.ab_type) * 2.0, w.ab_type)
        got = W.decode(R.gemm_host(w3), w.c_type)
        assert np.array_equal(got, 2.0 * W.decode(base, w.c_type))
    # appending zero columns to K changes nothing
    pad = 64
    w4 = W.make_workload(name, *dims)
    w4.K = w.K + pad
    za = np.zeros((w.M, pad), w.A.dtype)
    w4.A = np.ascontiguousarray(np.concatenate([w.A, za], axis=1))
    if w.transB:
        w4.B = np.ascontiguousarray(np.concatenate([w.B, np.zeros((w.N, pad), w.B.dtype)], axis=1))
    else:
        w4.B = np.ascontiguousarray(np.concatenate([w.B, np.zeros((pad, w.N), w.B.dtype)], axis=0))
    assert np.array_equal(R.gemm_host(w4), base)


# ----------------------------------------------------------------------------- full configurations
def sampled_rows(M, n=48, seed=7):
    n = min(n, M)
    return np.sort(np.random.default_rng(seed).choice(M, n, replace=False))


def test_cfg1_full_fp32_512():
    w = W.make_workload("cfg1")
    out, info = run_and_check(w)
    assert info["kernel_name"] == "simt"
    assert W.rel_frobenius(out, ref.ref_gemm(w)) <= 1e-4


@pytest.mark.parametrize("name", ["cfg2", "cfg3"])
def test_full_size_configs_on_sampled_rows(name):
    w = W.make_workload(name)
    run_and_check(w, rows=sampled_rows(w.M))


def test_cfg4_full_size_fp8_on_sampled_rows():
    w = W.make_workload("cfg4", 2048, 8192, 8192)  # full N and K, a quarter of the rows
    run_and_check(w, rows=sampled_rows(w.M))


def test_cfg5_shard_and_bf16_8192_on_sampled_rows():
    # one rank's share of cfg5 at 8 GPUs (8192 rows) is the bf16 8192^3 problem with cfg5's data
    w = W.make_workload("cfg5", 8192, 8192, 8192)
    out, _ = run_and_check(w, rows=sampled_rows(w.M))
    # the shards of a row-split product are exactly the rows of the unsplit product
    row0, rows = R.shard_rows(w.M, 8, 3)
    ws = W.GemmWorkload("cfg5-shard", rows, w.N, w.K, W.BF16, W.BF16, B=w.B,
                        A=np.ascontiguousarray(w.A[row0:row0 + rows]))
    assert np.array_equal(R.gemm_host(ws), out[row0:row0 + rows])


def test_cfg5_full_m_on_device_generated_data():
    """All 65536 rows once (A 1 GiB, C 1 GiB): inputs drawn on the device, rows sampled back."""
    torch = pytest.importorskip("torch")
    dev = torch.device("cuda:0")
    M, N, K = 65536, 8192, 8192
    g = torch.Generator(device=dev).manual_seed(4)
    A = torch.randn(M, K, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    B = (torch.randn(K, N, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    Cd = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    plan = R.GemmPlan(M, N, K, W.BF16)
    plan.run(A, B, Cd, status=status)
    R.check_status(status)
    rows = sampled_rows(M, 32)
    idx = torch.from_numpy(rows).to(dev)
    w = W.GemmWorkload("cfg5-dev", len(rows), N, K, W.BF16, W.BF16,
                       A=A[idx].view(torch.uint16).cpu().numpy(), B=B.view(torch.uint16).cpu().numpy())
    got = W.bf16_decode(Cd[idx].view(torch.uint16).cpu().numpy())
    ok, err, metric = W.check(got, ref.ref_gemm_f64(w), W.BF16, absdot=ref.abs_dot(w))
    assert ok, f"{metric} = {err}"
    plan.close()


def test_module_built_with_the_ir_builder_executes():
    """The reference's flow end to end: build frisk.gemm through the builder, then run it."""
    import frisk as F

    w = W.make_workload("cfg2", 256, 384, 192)
    h = F.create_session()
    f16 = h.builder.get_f16_ty()
    tys = [h.memref_type((w.M, w.K), f16), h.memref_type((w.K, w.N), f16), h.memref_type((w.M, w.N), f16)]
    _, entry = h.new_kernel("k", tys)
    h.create_gemm(*[entry.get_argument(i) for i in range(3)], trans_b=True, clear_accum=True)
    calls = F.find_gemms(h.module, "k")
    assert len(calls) == 1 and (calls[0].M, calls[0].N, calls[0].K, calls[0].transB) == (256, 384, 192, True)
    out = np.zeros((w.M, w.N), np.float16)
    F.run(h.module, "k", [w.A, w.B, out])
    ok, err, _ = W.check(out.astype(np.float32), ref.ref_gemm_f64(w), W.F16, absdot=ref.abs_dot(w))
    assert ok, err
    # operands that are not GLOBAL kernel arguments are refused, not silently skipped
    h2 = F.create_session()
    _, e2 = h2.new_kernel("k", [h2.memref_type((128, 64), f16, space=F.MemorySpace.SHARED),
                                h2.memref_type((64, 128), f16, space=F.MemorySpace.SHARED),
                                h2.memref_type((128, 128), f16, space=F.MemorySpace.LOCAL)])
    h2.create_gemm(*[e2.get_argument(i) for i in range(3)])
    with pytest.raises(R.FriskError):
        F.find_gemms(h2.module, "k")


@pytest.mark.parametrize("fp8,dt", [("e4m3fn", W.E4M3), ("e5m2", W.E5M2)])
def test_fp8_gemm_with_scale_operands_built_through_the_ir_builder_executes(fp8, dt):
    """cfg4's form written as IR: 8-bit float A and B (both K-inner), bf16 C, the two fp32 scale
    vectors as the additional fourth and fifth operands of frisk.gemm, bound as kernel arguments.
    Both 8-bit element types the reference's builder names (ffi/ir.cpp:411-414)."""
    import frisk as F

    w = W.make_workload("cfg4", 256, 384, 512)
    if dt == W.E5M2:   # the same values on the other grid
        w.A, w.B, w.ab_type = (W.encode(W.decode(w.A, W.E4M3), dt), W.encode(W.decode(w.B, W.E4M3), dt), dt)
    h = F.create_session()
    f32 = h.builder.get_f32_ty()
    tys = [h.memref_type((w.M, w.K), fp8), h.memref_type((w.K, w.N), fp8),
           h.memref_type((w.M, w.N), "bf16"), h.memref_type((w.M,), f32), h.memref_type((w.N,), f32)]
    _, entry = h.new_kernel("k", tys)
    a = [entry.get_argument(i) for i in range(5)]
    h.builder.create_gemm_op(a[0], a[1], a[2], False, True, True, a[3], a[4])
    (call,) = F.find_gemms(h.module, "k")
    assert (call.arg_scale_a, call.arg_scale_b, call.ab_type, call.c_type) == (3, 4, dt, W.BF16)
    out = np.zeros((w.M, w.N), np.uint16)
    F.run(h.module, "k", [w.A, w.B, out, w.scale_a, w.scale_b])
    assert np.array_equal(out, R.gemm_host(w))
    ok, err, _ = W.check(W.bf16_decode(out), ref.ref_gemm_f64(w), dt, absdot=ref.abs_dot(w))
    assert ok, err


# ----------------------------------------------------------------------------- few-row plans
# Shapes chosen so that every form of the few-row plan runs: clusters of 8, 4 and 2 on 256- and
# 128-row tiles, the stream-K fallback (too few tiles, or a forced grid), ragged N and K, every
# input type, K-inner and N-inner weights, C += and scales.
FEW_ROWS = [
    # (M, N, K, ab, transB, clear_accum, plan options)
    (16, 4096, 2048, W.BF16, False, True, {}),
    (16, 2048, 2048, W.F16, False, True, {}),
    (33, 8192, 512, W.BF16, False, True, {}),
    (64, 8192, 256, W.F16, True, True, {}),       # weights stored [N, K]
    (1, 1000, 520, W.BF16, False, True, {}),      # ragged N and K
    (7, 2304, 1096, W.F16, False, False, {}),     # C += A x B
    (48, 4096, 1024, W.E4M3, True, True, {}),     # scales
    (16, 512, 4096, W.BF16, False, True, {}),     # stream-K: two tiles
    (16, 4096, 2048, W.BF16, False, True, {"num_ctas": 37}),  # stream-K: forced grid
    (24, 4096, 2048, W.F16, False, False, {"num_ctas": 148}),
    (100, 4096, 1024, W.BF16, False, True, {}),   # more than 64 rows: 128-column tiles of B
    (128, 8192, 512, W.F16, True, False, {}),
    (96, 512, 2048, W.BF16, False, True, {"force_kernel": "skinny"}),  # ... and their stream-K form
    (128, 2048, 1024, W.E4M3, True, True, {}),
    (32, 4096, 1024, W.E5M2, True, True, {}),     # the other 8-bit float: scales, clusters
    (16, 512, 4096, W.E5M2, True, False, {}),     # ... stream-K, C +=
]


@pytest.mark.parametrize("M,N,K,ab,tb,clear,opts", FEW_ROWS)
def test_few_row_plans_match_oracle(M, N, K, ab, tb, clear, opts):
    rng = np.random.default_rng(M * 131 + N + K)
    fp8 = ab in (W.E4M3, W.E5M2)
    a = (rng.standard_normal((M, K)) * (1.0 if not fp8 else 4.0)).astype(np.float32)
    b = (rng.standard_normal((K, N)) * (0.05 if not fp8 else 4.0)).astype(np.float32)
    ct = W.BF16 if fp8 else ab
    sa = sb = None
    if fp8:
        sa = (rng.uniform(0.5, 2.0, M) / 448.0).astype(np.float32)
        sb = (rng.uniform(0.5, 2.0, N) / 448.0).astype(np.float32)
    Bq = W.encode(b, ab)
    w = W.GemmWorkload("few-rows", M, N, K, ab, ct, transB=tb, clear_accum=clear,
                       A=W.encode(a, ab), B=np.ascontiguousarray(Bq.T) if tb else Bq,
                       scale_a=sa, scale_b=sb,
                       C0=None if clear else W.encode(rng.standard_normal((M, N)).astype(np.float32), ct))
    out, info = run_and_check(w, **opts)
    assert info["kernel_name"] == "skinny"
    # summation order is fixed by the plan, not by which CTA finishes first
    assert np.array_equal(out, R.gemm_host(w, **opts))


@pytest.mark.parametrize("M,N,K,ab,ct,ta,tb,clear", [
    (300, 104, 200, W.BF16, W.BF16, False, False, True),    # 128-column tiles
    (260, 520, 136, W.F16, W.F32, False, True, False),      # fp32 C, C += A x B
    (512, 768, 640, W.E4M3, W.BF16, False, True, True),     # scales
    (520, 392, 272, W.E5M2, W.F16, False, True, False),     # e5m2 inputs, scales, fp16 C +=
    (384, 1024, 2048, W.BF16, W.F16, True, False, True),    # A stored [K, M]
    (1000, 1000, 1000, W.F16, W.F16, False, False, False),  # ragged everywhere
])
def test_cta_pair_kernel_variants_match_oracle(M, N, K, ab, ct, ta, tb, clear):
    rng = np.random.default_rng(M + 7 * N + 13 * K)
    big = ab in (W.E4M3, W.E5M2)
    a = (rng.standard_normal((M, K)) * (4.0 if big else 1.0)).astype(np.float32)
    b = (rng.standard_normal((K, N)) * (4.0 if big else K ** -0.5)).astype(np.float32)
    sa = (rng.uniform(0.5, 2.0, M) / 448.0).astype(np.float32) if big else None
    sb = (rng.uniform(0.5, 2.0, N) / 448.0).astype(np.float32) if big else None
    Aq, Bq = W.encode(a, ab), W.encode(b, ab)
    w = W.GemmWorkload("pair", M, N, K, ab, ct, transA=ta, transB=tb, clear_accum=clear,
                       A=np.ascontiguousarray(Aq.T) if ta else Aq,
                       B=np.ascontiguousarray(Bq.T) if tb else Bq, scale_a=sa, scale_b=sb,
                       C0=None if clear else W.encode(rng.standard_normal((M, N)).astype(np.float32), ct))
    out, info = run_and_check(w)
    assert info["kernel_name"] == "tcgen05_pair"
    out1, info1 = run_and_check(w, force_kernel="tcgen05")
    assert info1["kernel_name"] == "tcgen05"
    assert np.array_equal(out, out1)  # same k order, same fp32 accumulation: same bits
    if ab == W.E5M2:   # ... and the CUDA-core kernel decodes the same 8-bit format
        _, info2 = run_and_check(w, force_kernel="simt")
        assert info2["kernel_name"] == "simt"


@pytest.mark.parametrize("M,N,K,ab,ct,ta,tb,clear", [
    (512, 512, 4096, W.BF16, W.BF16, False, False, True),     # 128 x 128 tiles, clusters of 8
    (256, 256, 8192, W.F16, W.F32, False, True, False),       # 128 x 64 tiles, fp32 C +=
    (1024, 1024, 12288, W.BF16, W.F16, True, False, True),    # A stored [K, M]; 128 x 256 tiles
    (2048, 128, 4096, W.F16, W.F16, False, False, True),      # one tile column, 256-row tiles
    (300, 200, 4104, W.BF16, W.BF16, False, False, False),    # ragged everywhere, C +=
    (129, 1000, 8192, W.E4M3, W.BF16, False, True, True),     # scales in the split epilogue
    (128, 128, 4096, W.BF16, W.BF16, False, False, True),     # two tiles: stream-K, workspace
])
def test_k_split_plans_without_the_swap_match_oracle(M, N, K, ab, ct, ta, tb, clear):
    """Few tiles of C against a long K: the planner splits K over clusters (or stream-K) of the
    one-CTA kernel instead of leaving most SMs idle.  Same oracle, same tolerances; the summation
    order is fixed by the plan, so two runs give the same bits."""
    rng = np.random.default_rng(M + 7 * N + 13 * K)
    big = ab in (W.E4M3, W.E5M2)
    a = (rng.standard_normal((M, K)) * (4.0 if big else 1.0)).astype(np.float32)
    b = (rng.standard_normal((K, N)) * (4.0 if big else K ** -0.5)).astype(np.float32)
    sa = (rng.uniform(0.5, 2.0, M) / 448.0).astype(np.float32) if big else None
    sb = (rng.uniform(0.5, 2.0, N) / 448.0).astype(np.float32) if big else None
    Aq, Bq = W.encode(a, ab), W.encode(b, ab)
    w = W.GemmWorkload("k-split", M, N, K, ab, ct, transA=ta, transB=tb, clear_accum=clear,
                       A=np.ascontiguousarray(Aq.T) if ta else Aq,
                       B=np.ascontiguousarray(Bq.T) if tb else Bq, scale_a=sa, scale_b=sb,
                       C0=None if clear else W.encode(rng.standard_normal((M, N)).astype(np.float32), ct))
    def run(**kw):
        plan = R.GemmPlan.for_workload(w, **kw)
        info = plan.info
        plan.close()
        return R.gemm_host(w, **kw), info

    out, info = run(k_split=1)
    assert info["kernel_name"] == "tcgen05" and info["split_k"] == 1 and info["swap_ab"] == 0, info
    assert np.array_equal(out, R.gemm_host(w, k_split=1))
    floor = ref.abs_dot(w)
    for other in (ref.ref_gemm_f64(w), W.decode(ref.ref_gemm(w), ct), torch_matmul_fp32(w)):
        ok, err, metric = W.check(W.decode(out, ct), other, ab, absdot=floor)
        assert ok, (metric, err)
    whole, info_w = run(force_kernel="tcgen05")   # the same problem as whole tiles
    assert info_w["split_k"] == 0
    ok, err, metric = W.check(W.decode(out, ct), W.decode(whole, ct), ab, absdot=floor)
    assert ok, (metric, err)


@pytest.mark.parametrize("M,N,K,ab,ct,ta,tb,clear,auto", [
    (512, 512, 32768, W.BF16, W.BF16, False, False, True, True),    # 4 tiles x 18 parts: the plan's own choice
    (1024, 1024, 12288, W.F16, W.F16, True, False, False, True),    # A stored [K, M]; C +=
    (300, 200, 4104, W.BF16, W.BF16, False, False, False, False),   # ragged tiles, ragged last K part, C +=
    (129, 1000, 8192, W.E4M3, W.BF16, False, True, True, False),    # scales applied by the sum
    (256, 130, 2048, W.F16, W.F32, False, True, False, False),      # fp32 C +=, 128-wide tiles, odd N
    (520, 264, 2320, W.E5M2, W.BF16, False, True, True, False),     # six tiles, two unequal K parts
])
def test_k_planes_plans_match_oracle(M, N, K, ab, ct, ta, tb, clear, auto):
    """K planes: the CTA-pair kernel takes one work item per (tile, K part), writes fp32 partial
    tiles into the workspace, and a second launch sums the planes, in their order, into C (scales,
    += C and the cast happen there).  Same oracle, same tolerances, same bits on every run."""
    rng = np.random.default_rng(M + 7 * N + 13 * K)
    big = ab in (W.E4M3, W.E5M2)
    a = (rng.standard_normal((M, K)) * (4.0 if big else 1.0)).astype(np.float32)
    b = (rng.standard_normal((K, N)) * (4.0 if big else K ** -0.5)).astype(np.float32)
    sa = (rng.uniform(0.5, 2.0, M) / 448.0).astype(np.float32) if big else None
    sb = (rng.uniform(0.5, 2.0, N) / 448.0).astype(np.float32) if big else None
    Aq, Bq = W.encode(a, ab), W.encode(b, ab)
    w = W.GemmWorkload("k-planes", M, N, K, ab, ct, transA=ta, transB=tb, clear_accum=clear,
                       A=np.ascontiguousarray(Aq.T) if ta else Aq,
                       B=np.ascontiguousarray(Bq.T) if tb else Bq, scale_a=sa, scale_b=sb,
                       C0=None if clear else W.encode(rng.standard_normal((M, N)).astype(np.float32), ct))
    kw = {} if auto else {"k_split": 2}
    plan = R.GemmPlan.for_workload(w, **kw)
    info, ws = plan.info, plan.workspace_bytes
    plan.close()
    assert (info["kernel_name"], info["split_k"], info["launches"]) == ("tcgen05_pair", 1, 2), info
    assert ws >= 2 * M * N * 4
    out = R.gemm_host(w, **kw)
    assert np.array_equal(out, R.gemm_host(w, **kw))
    floor = ref.abs_dot(w)
    for other in (ref.ref_gemm_f64(w), W.decode(ref.ref_gemm(w), ct), torch_matmul_fp32(w)):
        ok, err, metric = W.check(W.decode(out, ct), other, ab, absdot=floor)
        assert ok, (metric, err)
    whole = R.gemm_host(w, k_split=-1)   # the same problem as whole tiles
    ok, err, metric = W.check(W.decode(out, ct), W.decode(whole, ct), ab, absdot=floor)
    assert ok, (metric, err)


@pytest.mark.parametrize("M,N,K,ab,ct,ta,tb,clear,auto,ctas", [
    (512, 512, 4096, W.BF16, W.BF16, False, False, True, True, 64),     # 8 tiles x 4 pairs: the plan's own choice
    (384, 384, 8192, W.F16, W.F32, False, True, False, True, 48),       # fp32 C +=, B stored [N, K]
    (1024, 1024, 4104, W.BF16, W.BF16, True, False, True, True, 128),   # two pairs per cluster, A stored [K, M], ragged K
    (300, 200, 2056, W.BF16, W.F16, False, False, False, False, 32),    # ragged tiles, C +=
    (512, 500, 4096, W.E4M3, W.BF16, False, True, True, False, 64),     # scales in the fold
    (260, 128, 8192, W.E5M2, W.BF16, False, True, True, False, 16),     # one tile column, mostly padding rows
])
def test_k_split_over_cta_pairs_of_a_cluster_matches_oracle(M, N, K, ab, ct, ta, tb, clear, auto, ctas):
    """K split over the CTA pairs of a cluster: every pair multiplies one K part of a 256 x 128 tile
    with two-SM MMAs, the partial tiles meet through distributed shared memory and each CTA adds
    the images of the rows it owns in pair order.  One launch, no workspace, the same bits on
    every run; same oracle and tolerances as every other plan."""
    rng = np.random.default_rng(M + 7 * N + 13 * K)
    big = ab in (W.E4M3, W.E5M2)
    a = (rng.standard_normal((M, K)) * (4.0 if big else 1.0)).astype(np.float32)
    b = (rng.standard_normal((K, N)) * (4.0 if big else K ** -0.5)).astype(np.float32)
    sa = (rng.uniform(0.5, 2.0, M) / 448.0).astype(np.float32) if big else None
    sb = (rng.uniform(0.5, 2.0, N) / 448.0).astype(np.float32) if big else None
    Aq, Bq = W.encode(a, ab), W.encode(b, ab)
    w = W.GemmWorkload("pair-clusters", M, N, K, ab, ct, transA=ta, transB=tb, clear_accum=clear,
                       A=np.ascontiguousarray(Aq.T) if ta else Aq,
                       B=np.ascontiguousarray(Bq.T) if tb else Bq, scale_a=sa, scale_b=sb,
                       C0=None if clear else W.encode(rng.standard_normal((M, N)).astype(np.float32), ct))
    def plan_of(kw):
        plan = R.GemmPlan.for_workload(w, **kw)
        info, ws = plan.info, plan.workspace_bytes
        plan.close()
        return info, ws

    # `ctas`: the plan on a device that places every cluster at once (checked per plan with the
    # occupancy query: B200s differ in how many SMs each GPC has left).  Where this device cannot,
    # the plan falls back -- to two pairs per cluster when forced, to other forms otherwise -- and
    # the test runs whatever cluster form exists here.
    kw = {} if auto else {"k_split": 3}
    info, ws = plan_of(kw)
    if not (info["kernel_name"] == "tcgen05_pair" and info["split_k"] and info["launches"] == 1):
        kw = {"k_split": 3}
        info, ws = plan_of(kw)
        if not (info["kernel_name"] == "tcgen05_pair" and info["split_k"] and info["launches"] == 1):
            pytest.skip("this device places no cluster shape of the plan")
    tiles = -(-M // 256) * -(-N // 128)
    assert (info["tile_n"], ws) == (128, 0) and info["num_ctas"] in (4 * tiles, 8 * tiles), info
    assert info["num_ctas"] <= ctas
    out = R.gemm_host(w, **kw)
    assert np.array_equal(out, R.gemm_host(w, **kw))
    floor = ref.abs_dot(w)
    for other in (ref.ref_gemm_f64(w), W.decode(ref.ref_gemm(w), ct), torch_matmul_fp32(w)):
        ok, err, metric = W.check(W.decode(out, ct), other, ab, absdot=floor)
        assert ok, (metric, err)
    whole = R.gemm_host(w, k_split=-1)   # the same problem as whole tiles
    ok, err, metric = W.check(W.decode(out, ct), W.decode(whole, ct), ab, absdot=floor)
    assert ok, (metric, err)


@pytest.mark.parametrize("ldc_extra,c_off", [(24, 0), (3, 0), (24, 2)])
def test_k_planes_keep_to_their_columns_and_their_workspace(ldc_extra, c_off):
    """The sum launch of a K-planes plan writes C's N columns and nothing else -- at a padded pitch
    that allows vector stores, at an odd one, and from a base off the 16-byte grid -- and the two
    launches stay inside the workspace the plan asked for."""
    torch = pytest.importorskip("torch")
    dev = torch.device("cuda:0")
    M, N, K = 300, 200, 2048
    rng = np.random.default_rng(77 + ldc_extra + c_off)
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = (rng.standard_normal((K, N)) * K ** -0.5).astype(np.float32)
    c0 = rng.standard_normal((M, N)).astype(np.float32)
    w = W.GemmWorkload("planes-ld", M, N, K, W.BF16, W.BF16, clear_accum=False, A=W.bf16_encode(a),
                       B=W.bf16_encode(b), C0=W.bf16_encode(c0))
    ldc = N + ldc_extra
    plan = R.GemmPlan(M, N, K, W.BF16, ldc=ldc, clear_accum=False, k_split=2)
    assert (plan.info["kernel_name"], plan.info["launches"]) == ("tcgen05_pair", 2)
    guard = 4096
    ws_bytes = plan.workspace_bytes
    cbuf = torch.full((guard + M * ldc,), 0x7FC0, dtype=torch.int16, device=dev)   # NaN canaries
    cview = cbuf[guard // 2 + c_off: guard // 2 + c_off + M * ldc].view(M, ldc)
    cview[:, :N] = torch.from_numpy(w.C0.view(np.int16)).to(dev)
    wsbuf = torch.full((guard * 2 + ws_bytes,), 0xCD, dtype=torch.uint8, device=dev)
    A = torch.from_numpy(w.A.view(np.int16)).to(dev)
    B = torch.from_numpy(w.B.view(np.int16)).to(dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = R.lib().frisk_b200_gemm_run(plan._h, A.data_ptr(), B.data_ptr(), cview.data_ptr(), None, None,
                                     wsbuf.data_ptr() + guard, ws_bytes, status.data_ptr(),
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    R.check_status(status)
    plan.close()
    nan16 = np.int16(0x7FC0)
    flat = cbuf.cpu().numpy()
    body = flat[guard // 2 + c_off: guard // 2 + c_off + M * ldc].reshape(M, ldc)
    assert (flat[:guard // 2 + c_off] == nan16).all() and (flat[guard // 2 + c_off + M * ldc:] == nan16).all()
    assert (body[:, N:] == nan16).all(), "the sum wrote outside C's columns"
    assert (wsbuf[:guard] == 0xCD).all() and (wsbuf[guard + ws_bytes:] == 0xCD).all()
    got = W.bf16_decode(np.ascontiguousarray(body[:, :N]).view(np.uint16))
    ok, err, metric = W.check(got, ref.ref_gemm_f64(w), W.BF16, absdot=ref.abs_dot(w))
    assert ok, (metric, err)


def test_planner_choices_over_seeded_random_problems_match_the_oracle():
    """Whatever the planner picks -- whole tiles, CTA pairs, few-row clusters, stream-K, K-split
    without the swap, repacked operands, CUDA cores -- the result is the oracle's.  48 seeded
    problems: every input type and storage order, odd sizes and pitches, C += and scales."""
    import random
    rnd = random.Random(20)
    seen = {}
    for case in range(48):
        ab = rnd.choice([W.F32, W.F16, W.BF16, W.BF16, W.E4M3, W.E5M2])
        fp8 = ab in (W.E4M3, W.E5M2)
        ct = W.BF16 if fp8 else rnd.choice([ab, ab, W.F32]) if ab != W.F32 else W.F32
        M = rnd.choice([1, 5, 16, 48, 100, 128, 129, 200, 256, 300, 520, 1000])
        N = rnd.choice([8, 72, 128, 200, 256, 520, 1000, 2048, 4100])
        K = rnd.choice([8, 72, 136, 520, 1000, 3072, 4104, 8192])
        ta, tb = rnd.random() < 0.25, rnd.random() < 0.5
        if fp8 and rnd.random() < 0.8:
            ta, tb = False, True
        clear = rnd.random() < 0.7
        rng = np.random.default_rng(1000 + case)
        a = (rng.standard_normal((M, K)) * (4.0 if fp8 else 1.0)).astype(np.float32)
        b = (rng.standard_normal((K, N)) * (4.0 if fp8 else K ** -0.5)).astype(np.float32)
        Aq, Bq = W.encode(a, ab), W.encode(b, ab)
        w = W.GemmWorkload(f"fuzz{case}", M, N, K, ab, ct, transA=ta, transB=tb, clear_accum=clear,
                           A=np.ascontiguousarray(Aq.T) if ta else Aq,
                           B=np.ascontiguousarray(Bq.T) if tb else Bq,
                           scale_a=(rng.uniform(0.5, 2.0, M) / 448.0).astype(np.float32) if fp8 else None,
                           scale_b=(rng.uniform(0.5, 2.0, N) / 448.0).astype(np.float32) if fp8 else None,
                           C0=None if clear else W.encode(rng.standard_normal((M, N)).astype(np.float32), ct))
        plan = R.GemmPlan.for_workload(w)
        info = plan.info
        plan.close()
        out = R.gemm_host(w)
        ok, err, metric = W.check(W.decode(out, ct), ref.ref_gemm_f64(w), ab, absdot=ref.abs_dot(w))
        what = (info["kernel_name"], info["split_k"], info["launches"])
        assert ok, f"case {case}: {M}x{N}x{K} types {ab}->{ct} trans {ta},{tb} clear {clear} via {what}: {metric} = {err:.3e}"
        seen[what] = seen.get(what, 0) + 1
    kinds = {k[0] for k in seen}
    assert {"simt", "tcgen05", "tcgen05_pair", "skinny"} <= kinds, seen
    assert any(k[0] == "tcgen05" and k[1] for k in seen), seen          # K-split without the swap
    assert any(k[2] > 1 and k[0] not in ("tf32x3",) for k in seen), seen   # a repacked operand


def test_back_to_back_dependent_launches_see_each_others_results():
    """The tensor-core kernels are launched with programmatic stream serialization (their set-up may
    overlap the previous kernel's tail).  A chain in which every GEMM reads what the one before
    wrote, launched without any synchronisation, must give the bits of the same chain run one
    step at a time: CTA-pair kernel -> one-CTA kernel -> cluster few-row plan -> stream-K few-row
    plan -> CUDA-core kernel."""
    torch = pytest.importorskip("torch")
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(11)
    bf = torch.bfloat16
    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g, device=dev) * scale).to(bf)
    K = 512
    x0 = rnd(512, K)
    w = [rnd(K, K, scale=K ** -0.5) for _ in range(3)]
    w_wide = rnd(K, 4096, scale=K ** -0.5)
    w_narrow = rnd(4096, 512, scale=4096 ** -0.5)
    w_f32 = torch.randn(512, 96, generator=g, device=dev) * 512 ** -0.5
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    steps = []  # (plan, A, B, C)
    def add(M, N, Kd, a, b, ab=W.BF16, ct=W.BF16, **kw):
        plan = R.GemmPlan(M, N, Kd, ab, ct, **kw)
        out = torch.empty(M, N, device=dev, dtype={W.BF16: bf, W.F32: torch.float32}[ct])
        ws = torch.zeros(max(plan.workspace_bytes, 16), dtype=torch.uint8, device=dev)
        steps.append((plan, a, b, out, ws))
        return out
    y1 = add(512, K, K, x0, w[0])                              # CTA-pair kernel
    y2 = add(512, K, K, y1, w[1], force_kernel="tcgen05")      # one-CTA kernel
    y3 = add(512, K, K, y2, w[2])
    y4 = add(16, 4096, K, y3[:16], w_wide)                     # few rows: clusters
    y5 = add(16, 512, 4096, y4, w_narrow)                      # few rows: stream-K (two tiles)
    y5f = torch.empty(16, 512, device=dev, dtype=torch.float32)
    kinds = [s[0].info["kernel_name"] for s in steps]
    assert kinds == ["tcgen05_pair", "tcgen05", "tcgen05_pair", "skinny", "skinny"], kinds
    f32_plan = R.GemmPlan(16, 96, 512, W.F32, W.F32)           # CUDA-core kernel on the chain's end
    y6 = torch.empty(16, 96, device=dev, dtype=torch.float32)

    def run_chain(sync):
        for plan, a, b, out, ws in steps:
            plan.run(a, b, out, None, None, ws, status)
            if sync:
                torch.cuda.synchronize()
        y5f.copy_(y5)  # a torch kernel in between, then the fp32 GEMM
        f32_plan.run(y5f, w_f32, y6, None, None, None, status)
        torch.cuda.synchronize()
        R.check_status(status)
        return [t.clone() for t in (y1, y2, y3, y4, y5, y6)]

    want = run_chain(sync=True)
    for t in (y1, y2, y3, y4, y5, y6):
        t.zero_()
    for _ in range(3):
        got = run_chain(sync=False)
        for a, b in zip(got, want):
            assert torch.equal(a, b)
    assert float(want[5].abs().max()) > 0
    for plan, *_ in steps:
        plan.close()
    f32_plan.close()


def test_runs_are_capturable_in_a_cuda_graph_and_replay_with_new_inputs():
    """Every launch of the library is stream-ordered work on the caller's stream, so a chain of GEMMs
    can be captured into a CUDA graph once and replayed: CTA-pair kernel with the row fold in its
    epilogue (two launches) -> few-row cluster plan -> few-row stream-K plan (a memset and a launch)
    -> 3xTF32 plan (three launches) -> K planes (the pair kernel and the sum of the planes).  The
    replay must give the bits of the same chain launched
    directly, also after the inputs' contents have changed."""
    torch = pytest.importorskip("torch")
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(23)
    bf = torch.bfloat16
    K = 512

    def rnd(*shape, scale=1.0, dtype=bf):
        return (torch.randn(*shape, generator=g, device=dev) * scale).to(dtype)

    x0 = rnd(512, K)
    w0, w_wide, w_narrow = rnd(K, K, scale=K ** -0.5), rnd(K, 4096, scale=K ** -0.5), rnd(4096, 512, scale=4096 ** -0.5)
    a32, b32 = rnd(512, 1024, dtype=torch.float32), rnd(1024, 1024, scale=1 / 32, dtype=torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    y1 = torch.empty(512, K, device=dev, dtype=bf)
    rowmax = torch.empty(512, device=dev, dtype=bf)
    y2 = torch.empty(16, 4096, device=dev, dtype=bf)
    y3 = torch.empty(16, 512, device=dev, dtype=bf)
    y4 = torch.empty(512, 1024, device=dev, dtype=torch.float32)
    w_deep = rnd(4096, 256, scale=4096 ** -0.5)
    x5 = torch.empty(512, 4096, device=dev, dtype=bf)   # 32 copies of y2, written inside the chain
    y5 = torch.empty(512, 256, device=dev, dtype=bf)
    plans = [R.GemmPlan(512, K, K, W.BF16, row_reduce="max"), R.GemmPlan(16, 4096, K, W.BF16),
             R.GemmPlan(16, 512, 4096, W.BF16), R.GemmPlan(512, 1024, 1024, W.F32, W.F32, force_kernel="tf32x3"),
             R.GemmPlan(512, 256, 4096, W.BF16, k_split=2)]
    assert [p.info["kernel_name"] for p in plans] == ["tcgen05_pair", "skinny", "skinny", "tf32x3", "tcgen05_pair"]
    assert plans[4].info["launches"] == 2 and plans[4].workspace_bytes > 0
    assert plans[1].workspace_bytes == 0 and plans[2].workspace_bytes > 0   # clusters, then stream-K
    wss = [torch.zeros(max(p.workspace_bytes, 256), dtype=torch.uint8, device=dev) for p in plans]

    def chain(stream):
        plans[0].run_ex(x0, w0, y1, workspace=wss[0], status=status, stream=stream, row_reduce_dst=rowmax)
        plans[1].run(y1[:16], w_wide, y2, None, None, wss[1], status, stream)
        plans[2].run(y2, w_narrow, y3, None, None, wss[2], status, stream)
        plans[3].run(a32, b32, y4, None, None, wss[3], status, stream)
        x5.view(32, 16, 4096).copy_(y2)
        plans[4].run(x5, w_deep, y5, None, None, wss[4], status, stream)

    outs = (y1, rowmax, y2, y3, y4, y5)
    chain(torch.cuda.current_stream().cuda_stream)          # also loads every kernel before the capture
    torch.cuda.synchronize()
    want = [t.clone() for t in outs]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        chain(torch.cuda.current_stream().cuda_stream)
    for t in outs:
        t.zero_()
    graph.replay()
    torch.cuda.synchronize()
    R.check_status(status)
    for got, ref_t in zip(outs, want):
        assert torch.equal(got, ref_t)
    # new contents in the same buffers: the replay computes on what is there now
    x0.copy_(rnd(512, K))
    a32.copy_(rnd(512, 1024, dtype=torch.float32))
    graph.replay()
    torch.cuda.synchronize()
    replayed = [t.clone() for t in outs]
    chain(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    R.check_status(status)
    for got, ref_t in zip(replayed, outs):
        assert torch.equal(got, ref_t)
    assert not torch.equal(replayed[0], want[0])
    for p in plans:
        p.close()


# ----------------------------------------------------------------------------- fp32 on tensor cores
@pytest.mark.parametrize("M,N,K,ta,tb,clear", [
    (512, 512, 512, False, False, True),       # cfg1's shape, forced onto the 3xTF32 plan
    (1000, 776, 520, False, True, True),       # ragged tiles, K-inner B
    (384, 1024, 2052, True, False, False),     # A stored [K, M], C += A x B
    (260, 520, 1096, True, True, True),
    (64, 2048, 1024, False, False, True),      # few rows: the one-CTA whole-tile kernel
    (2048, 2048, 2048, False, False, True),    # large enough for the plan to choose it itself
])
def test_fp32_on_tensor_cores_keeps_fp32_accuracy(M, N, K, ta, tb, clear):
    """3xTF32: A = A_hi + A_lo, B = B_hi + B_lo in tf32, three products accumulated in fp32.  The
    bound is the fp32 one (relative Frobenius error <= 1e-4); what is reached is 4e-7 at K = 512
    and 5e-6 at K = 2052 (the tensor core's fp32 accumulation over 3K products), and the largest
    element error stays below 1e-5 of the data behind it (a single-pass tf32 product would sit
    near 5e-4)."""
    rng = np.random.default_rng(M + N + K)
    a = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    w = W.GemmWorkload("fp32-tc", M, N, K, W.F32, W.F32, transA=ta, transB=tb, clear_accum=clear,
                       A=np.ascontiguousarray(a.T) if ta else a, B=np.ascontiguousarray(b.T) if tb else b,
                       C0=None if clear else rng.standard_normal((M, N)).astype(np.float32))
    forced = {} if 2.0 * M * N * K >= 1e9 else dict(force_kernel="tf32x3")
    out, info = run_and_check(w, **forced)
    assert info["kernel_name"] == "tf32x3"
    want = ref.ref_gemm_f64(w)
    assert W.rel_frobenius(out, want) <= 1e-5
    assert float(np.max(np.abs(out - want) / ref.abs_dot(w))) <= 1e-5
    assert np.array_equal(out, R.gemm_host(w, **forced))          # same bits on a second run
    simt, info2 = run_and_check(w, force_kernel="simt")
    assert info2["kernel_name"] == "simt"
    assert W.rel_frobenius(out, simt) <= 1e-5
