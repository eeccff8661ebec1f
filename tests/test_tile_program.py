"""The tiled matrix product around frisk.gemm (tmp/ir.mlir:1-17 of the reference) is recognised
and lifted to one whole-problem GEMM; everything that is not exactly that product is refused."""
import numpy as np
import pytest

import frisk as F
from frisk_b200 import runtime as R, workloads as W
from tile_programs import build_tiled_matmul


def test_sketch_program_prints_like_the_reference_and_lifts():
    m = build_tiled_matmul(1024, 1024, 1024, 128, 128, 32)  # the sizes of the reference's sketch
    assert m.verify(), m.verify_message()
    text = str(m)
    assert "frisk.parallel (%arg3, %arg4) = (8, 8), threads = 128" in text
    assert "frisk.copy %arg0[%arg3 * 128, %arg5 * 32], %0[0, 0]" in text
    assert "frisk.copy %2[0, 0], %arg2[%arg3 * 128, %arg4 * 128]" in text
    t = F.ir.frisk.lift_tiled_gemm(m.get_kernel("matmul"))
    assert (t["M"], t["N"], t["K"]) == (1024, 1024, 1024)
    assert (t["arg_a"], t["arg_b"], t["arg_c"]) == (0, 1, 2)
    assert t["clear_accum"] is True and t["tile"] == [128, 128, 32] and t["grid"] == [8, 8]
    assert str(t["ab_type"]) == "f16" and str(t["c_type"]) == "f16"
    (call,) = F.find_gemms(m, "matmul")
    assert (call.M, call.N, call.K, call.ab_type, call.c_type) == (1024, 1024, 1024, W.F16, W.F16)
    assert not call.transA and not call.transB and call.clear_accum


@pytest.mark.parametrize("dims,tile,dtype,acc,kstep", [
    ((512, 768, 256), (64, 128, 32), "bf16", True, 4),    # C tile loaded first: C += A x B
    ((256, 256, 512), (256, 64, 64), "fp32", False, 1),
    ((128, 384, 96), (128, 128, 32), "fp16", False, 32),  # loop variable counts elements of K
])
def test_variants_lift(dims, tile, dtype, acc, kstep):
    m = build_tiled_matmul(*dims, *tile, dtype=dtype, accumulate=acc, kstep=kstep)
    assert m.verify(), m.verify_message()
    (call,) = F.find_gemms(m, "matmul")
    assert (call.M, call.N, call.K) == dims and call.clear_accum == (not acc)
    assert call.ab_type == {"fp16": W.F16, "bf16": W.BF16, "fp32": W.F32}[dtype]


@pytest.mark.parametrize("tweak,reason", [
    ("fill_one", "filled with zero"),
    ("no_init", "neither cleared nor loaded"),
    ("no_store", "copy of the result"),
    ("a_rows_follow_bx", "A tile rows must start at by"),
    ("k_gap", "consecutive slices"),
    ("c_swapped", "C tiles must land"),
    ("grid_short", "cover A exactly"),
    ("extra_fill", "unexpected frisk.fill in the k loop"),
    ("gemm_clears", "must accumulate"),
    ("gemm_trans_b", "must not transpose"),
    ("gemm_scaled", "must not carry scale operands"),
])
def test_everything_else_is_refused_with_the_reason(tweak, reason):
    m = build_tiled_matmul(512, 512, 256, 128, 128, 32, tweak=tweak)
    with pytest.raises(ValueError, match=reason):
        F.ir.frisk.lift_tiled_gemm(m.get_kernel("matmul"))
    with pytest.raises(R.FriskError, match="not a tiled matrix product"):
        F.find_gemms(m, "matmul")


def test_tiled_matmul_with_a_row_reduce_of_the_accumulator_lifts_to_a_fused_plan():
    """One tile column (TN = N): a tile row holds whole rows of C, so the program's reduce of the
    accumulator tile over its columns is a reduce of C over dim 1 and rides in the GEMM's epilogue."""
    from frisk_b200 import execute as X
    m = build_tiled_matmul(512, 256, 128, 128, 256, 32, dtype="bf16", row_reduce=("max", True))
    assert m.verify(), m.verify_message()
    t = F.ir.frisk.lift_tiled_gemm(m.get_kernel("matmul"))
    assert (t["M"], t["N"], t["K"], t["arg_r"], t["reduce_kind"], t["reduce_clear"]) == (512, 256, 128, 3, "max", True)
    gemm, red = X.find_gemms(m, "matmul")
    assert isinstance(gemm, X.GemmCall) and red == X.ReduceCall((512, 256), 1, W.BF16, "max", True, 2, 3)
    # read back from text, the same program lifts the same way
    t2 = F.ir.frisk.lift_tiled_gemm(F.parse_module(str(m)).get_kernel("matmul"))
    assert {k: t2[k] for k in ("M", "N", "K", "arg_r", "reduce_kind")} == {k: t[k] for k in ("M", "N", "K", "arg_r", "reduce_kind")}
    for kw, reason in ((dict(N=512), "one tile column"), (dict(tweak="reduce_dim0"), "dim = 1"),
                       (dict(tweak="reduce_rows_off"), "by \\* TM")):
        kw = dict(kw)
        mm = build_tiled_matmul(512, kw.pop("N", 256), 128, 128, 256, 32, dtype="bf16", row_reduce=("add", True), **kw)
        with pytest.raises(ValueError, match=reason):
            F.ir.frisk.lift_tiled_gemm(mm.get_kernel("matmul"))


@pytest.mark.gpu
@pytest.mark.parametrize("kind,clear", [("max", True), ("add", False)])
def test_tiled_matmul_with_row_reduce_folds_in_the_epilogue(kind, clear):
    from frisk_b200 import execute as X
    from oracle import ref
    M, N, K = 512, 256, 384
    m = build_tiled_matmul(M, N, K, 128, 256, 32, dtype="bf16", row_reduce=(kind, clear))
    w = W.make_workload("cfg5", M, N, K)
    c = np.zeros((M, N), np.uint16)
    init = W.encode(np.random.default_rng(3).standard_normal(M).astype(np.float32), W.BF16)
    r = init.copy()
    F.run(m, "matmul", [w.A, w.B, c, r])
    assert X.LAST_RUN == [("gemm+reduce", "tcgen05_pair")]
    ok, err, metric = W.check(W.decode(c, W.BF16), ref.ref_gemm_f64(w), W.BF16, absdot=ref.abs_dot(w))
    assert ok, (metric, err)
    want, mag = ref.ref_reduce(c, 1, W.BF16, kind, clear, init)
    err = np.abs(W.decode(r, W.BF16).astype(np.float64) - want)
    tol = 0.0 if kind == "max" else 1e-5 * mag + 2.0 ** -7 * np.abs(want)
    assert (err <= tol).all(), float(err.max())


def test_reference_flagship_module_is_still_a_whole_problem_gemm():
    # bind_test.py's module (gemm on the kernel arguments inside for / block) is not a tile program
    from test_ir_builder import build_bind_test_module  # the reference script's program
    m = build_bind_test_module()[0]
    red, call = F.find_gemms(m, "test_gemm")  # the script also reduces its first argument
    assert (call.M, call.N, call.K) == (4096, 4096, 4096)
    assert (red.shape, red.dim, red.kind, red.clear, red.arg_src, red.arg_dst) == ((4096, 4096), 1, "max", True, 0, 3)
    with pytest.raises(ValueError, match="not a tiled matrix product"):
        F.ir.frisk.lift_tiled_gemm(m.get_kernel("test_gemm"))


@pytest.mark.gpu
@pytest.mark.parametrize("dims,tile,dtype,acc", [
    ((1024, 1024, 1024), (128, 128, 32), "fp16", False),
    ((512, 768, 256), (64, 128, 32), "bf16", True),
])
def test_lifted_program_runs_and_matches_the_oracle(dims, tile, dtype, acc):
    from oracle import ref
    M, N, K = dims
    ab = {"fp16": W.F16, "bf16": W.BF16}[dtype]
    rng = np.random.default_rng(7)
    a = rng.standard_normal((M, K)).astype(np.float32) * K ** -0.5
    b = rng.standard_normal((K, N)).astype(np.float32)
    c0 = rng.standard_normal((M, N)).astype(np.float32)
    A, B, C = W.encode(a, ab), W.encode(b, ab), W.encode(c0, ab)
    m = build_tiled_matmul(M, N, K, *tile, dtype=dtype, accumulate=acc)
    w = W.GemmWorkload("tiled", M, N, K, ab, ab, A=A, B=B, C0=C.copy() if acc else None,
                       clear_accum=not acc)
    F.run(m, "matmul", [A, B, C])
    got = W.decode(C, ab)
    ok, err, metric = W.check(got, ref.ref_gemm_f64(w), ab, absdot=ref.abs_dot(w))
    assert ok, f"{metric} = {err}"
    # one GEMM over the arguments: the same bits as planning that GEMM directly
    assert np.array_equal(C, R.gemm_host(w))


def gemm_then_row_max(dtype="fp16", dims=(16, 32, 64), kind="max", clear=True):
    """A kernel that multiplies and then takes the row maxima of the product: the two ops of the
    reference's attention sketches (tmp/ir.mlir:80-158) on whole buffers."""
    M, N, K = dims
    h = F.create_session()
    tys = [h.memref_type((M, K), dtype), h.memref_type((K, N), dtype), h.memref_type((M, N), dtype),
           h.memref_type((M,), dtype)]
    _, entry = h.new_kernel("scores_max", tys)
    h.create_gemm(entry.get_argument(0), entry.get_argument(1), entry.get_argument(2), clear_accum=True)
    h.builder.create_reduce_op(entry.get_argument(2), entry.get_argument(3), kind, 1, clear)
    return h


def test_reduce_ops_on_kernel_arguments_are_found_in_program_order():
    from frisk_b200 import execute as X
    h = gemm_then_row_max()
    assert h.module.verify()
    for module in (h.module, F.parse_module(str(h.module))):  # as built, and read back from text
        gemm, red = X.find_gemms(module, "scores_max")
        assert isinstance(gemm, X.GemmCall) and (gemm.arg_a, gemm.arg_b, gemm.arg_c) == (0, 1, 2)
        assert red == X.ReduceCall((16, 32), 1, W.F16, "max", True, 2, 3)
    # a reduce of a buffer that is not a kernel argument is refused, not guessed at
    h = F.create_session()
    _, entry = h.new_kernel("local_reduce", [h.memref_type((8,), "fp16")])
    frag = h.alloc_buffer((8, 8), "fp16", space=F.MemorySpace.LOCAL)
    h.builder.create_reduce_op(frag, entry.get_argument(0), "add", 1, True)
    with pytest.raises(R.FriskError, match="frisk.reduce source is not a kernel argument"):
        X.find_gemms(h.module, "local_reduce")


@pytest.mark.gpu
def test_gemm_followed_by_reduce_runs_as_written():
    from oracle import ref
    h = gemm_then_row_max("bf16", (64, 512, 256))
    w = W.make_workload("cfg5", 64, 512, 256)
    c = np.zeros((64, 512), np.uint16)
    rowmax = np.zeros((64,), np.uint16)
    F.run(h.module, "scores_max", [w.A, w.B, c, rowmax])
    ok, err, metric = W.check(W.decode(c, W.BF16), ref.ref_gemm_f64(w), W.BF16, absdot=ref.abs_dot(w))
    assert ok, (metric, err)
    want, _ = ref.ref_reduce(c, 1, W.BF16, "max")  # exact: the maximum of the stored values
    assert np.array_equal(W.decode(rowmax, W.BF16).astype(np.float64), want)
    # the two ops ran as one fused plan: the reduce sits in the gemm's epilogue
    from frisk_b200 import execute as X
    assert X.LAST_RUN == [("gemm+reduce", "tcgen05")]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,dims,kind,clear", [("fp16", (512, 1024, 256), "add", True),
                                                   ("bf16", (300, 520, 136), "max", False),
                                                   ("fp16", (1024, 768, 64), "min", True)])
def test_gemm_then_row_reduce_is_fused_and_matches_the_two_ops(dtype, dims, kind, clear):
    """The pair of ops of the reference's attention sketch (tmp/ir.mlir:112-135: a gemm, then a
    frisk.reduce of its result over dim 1) executed as one fused plan, against the same module's two
    ops restated on the CPU: the product in float64, the reduce on the stored C."""
    from frisk_b200 import execute as X
    from oracle import ref
    M, N, K = dims
    dt = {"fp16": W.F16, "bf16": W.BF16}[dtype]
    h = gemm_then_row_max(dtype, dims, kind, clear)
    rng = np.random.default_rng(M + N)
    w = W.GemmWorkload("scores", M, N, K, dt, dt,
                       A=W.encode(rng.standard_normal((M, K)).astype(np.float32), dt),
                       B=W.encode((rng.standard_normal((K, N)) * K ** -0.5).astype(np.float32), dt))
    c = np.zeros((M, N), W.storage_numpy_dtype(dt))
    init = W.encode(rng.standard_normal(M).astype(np.float32), dt)
    dst = init.copy()
    F.run(h.module, "scores_max", [w.A, w.B, c, dst])
    assert X.LAST_RUN == [("gemm+reduce", "tcgen05_pair")]
    ok, err, metric = W.check(W.decode(c, dt), ref.ref_gemm_f64(w), dt, absdot=ref.abs_dot(w))
    assert ok, (metric, err)
    want, mag = ref.ref_reduce(c, 1, dt, kind, clear, init)
    err = np.abs(W.decode(dst, dt).astype(np.float64) - want)
    ulp = {W.F16: 2.0 ** -10, W.BF16: 2.0 ** -7}[dt]
    tol = 0.0 if kind != "add" else 1e-5 * mag + ulp * np.abs(want)
    assert (err <= tol).all(), float(err.max())
    # fp32 operands have no tensor-core plan: the same program runs as two launches
    h32 = gemm_then_row_max("fp32", (96, 80, 64), kind, True)
    w32 = W.make_workload("cfg1", 96, 80, 64)
    c32, d32 = np.zeros((96, 80), np.float32), np.zeros(96, np.float32)
    F.run(h32.module, "scores_max", [w32.A, w32.B, c32, d32])
    assert X.LAST_RUN == [("gemm", "simt"), ("reduce", "reduce")]
    want, mag = ref.ref_reduce(c32, 1, W.F32, kind)
    assert (np.abs(d32 - want) <= (0.0 if kind != "add" else 1e-5 * mag + 2.0 ** -23 * np.abs(want))).all()


# ---- the tile-by-tile fold of a matrix (the reduce of the reference's online-softmax sketch) ----
from tile_programs import build_tiled_reduce


def test_tiled_reduce_lifts_to_one_whole_buffer_reduce():
    from frisk_b200 import execute as X
    # the sketch's shape (tmp/ir.mlir:22-36): 8192 rows, tiles of 1024 columns, one row per block
    m = build_tiled_reduce(8192, 8192, 1, 1024, kind="max")
    assert m.verify(), m.verify_message()
    text = str(m)
    assert "frisk.parallel (%arg2) = (8192), threads = 128" in text
    assert "frisk.fill %1 {value = 0xFC00 : f16}" in text          # -inf, printed as MLIR prints it
    assert 'frisk.reduce %0, %1 {clear = false, dim = 1 : i64, kind = "max"}' in text
    t = F.ir.frisk.lift_tiled_reduce(m.get_kernel("fold"))
    assert (t["shape"], t["dim"], t["kind"], t["clear"]) == ([8192, 8192], 1, "max", True)
    assert (t["arg_src"], t["arg_dst"], t["tile"], t["grid"]) == (0, 1, [1, 1024], 8192)
    for module in (m, F.parse_module(text)):                        # as built, and read back from text
        assert X.find_gemms(module, "fold") == [X.ReduceCall((8192, 8192), 1, W.F16, "max", True, 0, 1)]
    assert str(F.parse_module(text)) == text


@pytest.mark.parametrize("kw,want", [
    (dict(R=4096, C=256, TR=512, TC=64, dim=0, kind="add", dtype="fp32"), ((4096, 256), 0, W.F32, "add", True)),
    (dict(R=256, C=4096, TR=32, TC=1024, kind="min", dtype="bf16", start="load"), ((256, 4096), 1, W.BF16, "min", False)),
    (dict(R=256, C=4096, TR=32, TC=4096, kind="mul", loop=False, start="reduce_clears"), ((256, 4096), 1, W.F16, "mul", True)),
    (dict(R=64, C=512, TR=64, TC=512, dim=0, kind="max", loop=False, start="fill"), ((64, 512), 0, W.F16, "max", True)),
])
def test_tiled_reduce_variants_lift(kw, want):
    from frisk_b200 import execute as X
    m = build_tiled_reduce(**kw)
    assert m.verify(), m.verify_message()
    assert X.find_gemms(m, "fold") == [X.ReduceCall(*want, 0, 1)]


@pytest.mark.parametrize("tweak,reason", [
    ("grid_short", "cover the source exactly"),
    ("result_off", "must land at block index"),
    ("fill_other", "identity of the reduce kind"),
    ("reduce_clears_in_loop", "only the last tile would count"),
    ("gap", "consecutive tiles"),
    ("extra_fill", "unexpected frisk.fill in the loop"),
    ("no_store", "not copied out"),
])
def test_tiled_reduce_refusals_name_the_reason(tweak, reason):
    m = build_tiled_reduce(256, 4096, 32, 1024, tweak=tweak)
    with pytest.raises(ValueError, match=reason):
        F.ir.frisk.lift_tiled_reduce(m.get_kernel("fold"))
    with pytest.raises(R.FriskError, match="not a tiled reduce"):
        F.find_gemms(m, "fold")


@pytest.mark.gpu
@pytest.mark.parametrize("kw", [
    dict(R=2048, C=4096, TR=1, TC=1024, kind="max", dtype="fp16"),
    dict(R=4096, C=1024, TR=512, TC=64, dim=0, kind="add", dtype="fp32"),
    dict(R=512, C=2048, TR=32, TC=512, kind="min", dtype="bf16", start="load"),
])
def test_tiled_reduce_runs_and_matches_the_oracle(kw):
    from frisk_b200 import execute as X
    from oracle import ref
    dt = {"fp16": W.F16, "bf16": W.BF16, "fp32": W.F32}[kw["dtype"]]
    dim, kind = kw.get("dim", 1), kw["kind"]
    m = build_tiled_reduce(**kw)
    rng = np.random.default_rng(kw["R"] + kw["C"])
    x = W.encode(rng.standard_normal((kw["R"], kw["C"])).astype(np.float32), dt)
    init = W.encode(rng.standard_normal(x.shape[1 - dim]).astype(np.float32), dt)
    dst = init.copy()
    F.run(m, "fold", [x, dst])
    assert X.LAST_RUN == [("reduce", "reduce")]
    clear = kw.get("start", "fill") != "load"
    want, mag = ref.ref_reduce(x, dim, dt, kind, clear, init)
    err = np.abs(W.decode(dst, dt).astype(np.float64) - want)
    ulp = {W.F32: 2.0 ** -23, W.F16: 2.0 ** -10, W.BF16: 2.0 ** -7}[dt]
    tol = 0.0 if kind in ("min", "max") else 1e-5 * mag + ulp * np.abs(want)
    assert (err <= tol).all(), float(err.max())


def test_fills_and_copies_of_kernel_arguments_are_reported_not_silently_dropped():
    """Only gemm and reduce ops are executed; a fill or copy that touches a kernel argument is
    named in a FriskWarning (the reference's flagship module has both next to its gemm)."""
    import warnings
    from frisk_b200 import execute as X
    h = F.create_session()
    _, entry = h.new_kernel("k", [h.memref_type((64, 64), "fp16")] * 3)
    A, B, C = (entry.get_argument(i) for i in range(3))
    h.builder.create_fill_op(C, 1.0, "fp16")          # a program that relies on this fill ...
    h.create_gemm(A, B, C, clear_accum=False)
    (call,) = X.find_gemms(h.module, "k")
    assert not call.clear_accum and X.SKIPPED == [("frisk.fill", (2,))]   # ... is told that it did not run
    import pathlib
    flagship = F.parse_module((pathlib.Path(__file__).parent / "golden" / "bind_test_module.mlir").read_text())
    X.find_gemms(flagship, "test_gemm")
    assert X.SKIPPED == [("frisk.fill", (0,)), ("frisk.copy", (0, 1))]
    # tile programs are made of copies: lifting one reports nothing
    X.find_gemms(build_tiled_matmul(256, 256, 256, 128, 128, 32), "matmul")
    assert X.SKIPPED == []
    X.find_gemms(build_tiled_reduce(256, 4096, 32, 1024), "fold")
    assert X.SKIPPED == []
    # fills of local / shared buffers next to a whole-problem gemm are hints, not reported
    h = F.create_session()
    _, entry = h.new_kernel("k2", [h.memref_type((64, 64), "fp16")] * 3)
    frag = h.alloc_buffer((8, 8), "fp16", space=F.MemorySpace.LOCAL)
    h.builder.create_fill_op(frag, 0.0, "fp16")
    h.create_gemm(*(entry.get_argument(i) for i in range(3)), clear_accum=True)
    X.find_gemms(h.module, "k2")
    assert X.SKIPPED == []


@pytest.mark.gpu
def test_run_warns_about_ops_it_does_not_execute():
    h = F.create_session()
    _, entry = h.new_kernel("k", [h.memref_type((64, 64), "fp16")] * 3)
    A, B, C = (entry.get_argument(i) for i in range(3))
    h.builder.create_fill_op(C, 1.0, "fp16")
    h.create_gemm(A, B, C, clear_accum=True)
    a = W.encode(np.eye(64, dtype=np.float32), W.F16)
    c = np.zeros((64, 64), np.uint16)
    with pytest.warns(F.FriskWarning, match="frisk.fill of argument 2"):
        F.run(h.module, "k", [a, a, c])
    assert np.array_equal(c, a.view(np.uint16))   # identity x identity, fp16 bits
