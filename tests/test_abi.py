"""Host-side checks of the C ABI that need no GPU: every declared symbol is exported, plans pick
the expected kernel family, argument errors map to the documented codes, row sharding and the
layout mapping are right.  No compute call is made here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from frisk_b200 import runtime as R
from frisk_b200 import workloads as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "frisk_b200.h")).read()
    return sorted(set(re.findall(r"\b(frisk_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(R.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/frisk_b200.h but not exported"


def test_version_and_strerror():
    assert "sm_100a" in R.version()
    L = R.lib()
    assert L.frisk_b200_strerror(0) == b"ok"
    for code in range(-9, 0):
        assert L.frisk_b200_strerror(code) not in (b"", b"unknown error")
    assert L.frisk_b200_strerror(-99) == b"unknown error"


@pytest.mark.parametrize("name,kernel", [
    ("cfg1", "simt"), ("cfg2", "tcgen05_pair"), ("cfg3", "skinny"), ("cfg4", "tcgen05_pair"),
    ("cfg5", "tcgen05_pair"), ("bf16_8192", "tcgen05_pair"),
])
def test_plan_picks_kernel_family_for_the_benchmark_configs(name, kernel):
    full = {"cfg1": (512, 512, 512), "cfg2": (4096, 4096, 4096), "cfg3": (16, 8192, 8192),
            "cfg4": (8192, 8192, 8192), "cfg5": (65536, 8192, 8192),
            "bf16_8192": (8192, 8192, 8192)}[name]
    ab = {"cfg1": W.F32, "cfg2": W.F16, "cfg4": W.E4M3}.get(name, W.BF16)
    ct = {"cfg1": W.F32, "cfg2": W.F16}.get(name, W.BF16)
    plan = R.GemmPlan(*full, ab, ct, transB=name in ("cfg2", "cfg4"), scales=name == "cfg4")
    assert plan.info["kernel_name"] == kernel
    if kernel == "skinny":
        assert plan.info["swap_ab"] == 1 and plan.info["split_k"] == 1
        # 32 tiles of 256 columns of B, each owned by a cluster of four CTAs (a K slice each) that
        # sum their partials through distributed shared memory: no workspace
        assert plan.workspace_bytes == 0 and plan.info["num_ctas"] == 128
        assert plan.info["launches"] == 1
        # too few tiles for clusters to cover enough SMs: stream-K, at most 14 CTAs per tile (the
        # reduction sums up to 16 partials), 28 x 2 partial-tile slots of 256 x 16 fp32 and one
        # arrival counter per tile
        sk = R.GemmPlan(16, 512, 4096, ab, ct)
        assert sk.info["kernel_name"] == "skinny" and sk.info["num_ctas"] == 28
        assert sk.workspace_bytes == 28 * 2 * 256 * 16 * 4 + 2 * 4
        sk.close()
    else:
        assert plan.workspace_bytes == 0 and plan.info["launches"] == 1
    if kernel != "simt":
        assert plan.info["smem_bytes"] <= 227 * 1024
        assert plan.info["swizzle_a"] == 128 and plan.info["swizzle_b"] == 128
    plan.close()


def test_odd_row_pitches_are_repacked_not_sent_to_the_cuda_cores():
    """A row pitch that is not a multiple of 16 bytes rules out a tensor map on the caller's buffer:
    the plan keeps the tensor-core kernel and copies that operand into the workspace at a padded
    pitch first (one more launch per repacked operand)."""
    base = R.GemmPlan(100, 104, 104, W.BF16)
    p = R.GemmPlan(100, 104, 104, W.BF16, lda=107)           # 214-byte rows of A
    assert (p.info["kernel_name"], p.info["cuda_core_reason"]) == (base.info["kernel_name"], 0)
    assert p.info["launches"] == base.info["launches"] + 1
    assert p.workspace_bytes == base.workspace_bytes + (100 * 104 * 2 + 255) // 256 * 256
    p.close()
    p = R.GemmPlan(100, 100, 100, W.BF16, lda=101, ldb=100)  # both pitches odd; padded to 104 elements
    assert p.info["kernel_name"] == "tcgen05" and p.info["launches"] == 3
    assert p.workspace_bytes == 2 * ((100 * 104 * 2 + 255) // 256 * 256)
    p.close()
    p = R.GemmPlan(16, 4096, 1000, W.F16, transB=True, ldb=1001)   # a few-row plan on repacked weights
    assert p.info["kernel_name"] == "skinny" and p.info["launches"] == 2
    p.close()
    p = R.GemmPlan(100, 100, 100, W.BF16, lda=101, force_kernel="simt")   # asked for: no repacking
    assert p.info["kernel_name"] == "simt" and p.workspace_bytes == 0 and p.info["launches"] == 1
    p.close()
    base.close()
    p = R.GemmPlan(100, 104, 104, W.BF16)
    assert p.info["kernel_name"] == "tcgen05"
    p.close()
    p = R.GemmPlan(4096, 4096, 4096, W.BF16, band_tiles=4, stages=3)  # tuning overrides are accepted
    assert p.info["kernel_name"] == "tcgen05_pair" and p.info["stages"] == 3
    p.close()
    p = R.GemmPlan(128, 128, 128, W.E4M3, W.BF16, transB=False)  # fp8 MN-major B: CUDA cores
    assert p.info["kernel_name"] == "simt"
    p.close()


def test_k_split_override():
    """desc.k_split: 0 lets the plan decide (few tiles against a long K are split), -1 never splits,
    1 takes the cluster / stream-K form whenever it exists, 2 the K planes of the CTA-pair kernel."""
    auto = R.GemmPlan(512, 512, 65536, W.BF16)
    never = R.GemmPlan(512, 512, 65536, W.BF16, k_split=-1)
    clusters = R.GemmPlan(512, 512, 65536, W.BF16, k_split=1)
    # a deep K on four 256 x 256 tiles: K planes (the small tiles of the cluster form would pull
    # three times the bytes from L2)
    assert (auto.info["split_k"], auto.info["kernel_name"], auto.info["launches"]) == (1, "tcgen05_pair", 2)
    assert auto.workspace_bytes >= 2 * 512 * 512 * 4 and auto.workspace_bytes <= 20 << 20
    assert (clusters.info["split_k"], clusters.info["kernel_name"], clusters.info["swap_ab"]) == (1, "tcgen05", 0)
    assert clusters.info["launches"] == 1 and clusters.workspace_bytes == 0
    for p in (auto, clusters):
        assert p.info["num_ctas"] > 4 * never.info["num_ctas"]
    assert never.info["split_k"] == 0
    # a shallower problem keeps the cluster form: the second launch would cost more than it saves
    small = R.GemmPlan(129, 1000, 8192, W.BF16)
    small_planes = R.GemmPlan(129, 1000, 8192, W.BF16, k_split=2)
    assert (small.info["split_k"], small.info["kernel_name"], small.info["launches"]) == (1, "tcgen05", 1)
    assert (small_planes.info["kernel_name"], small_planes.info["launches"]) == ("tcgen05_pair", 2)
    big = R.GemmPlan(4096, 4096, 4096, W.BF16)
    forced = R.GemmPlan(4096, 4096, 4096, W.BF16, k_split=1)
    no_room = R.GemmPlan(4096, 4096, 4096, W.BF16, k_split=2)   # more tiles than pairs: no planes
    assert big.info["split_k"] == 0 and forced.info["split_k"] == 1 and no_room.info["split_k"] == 0
    for p in (auto, never, clusters, small, small_planes, big, forced, no_room):
        p.close()
    # eight tiles of 256 x 128 against 64 k-blocks: clusters of four CTA pairs, one launch, no
    # workspace (k_split = 3 forces the form, with two pairs per cluster where four do not fit)
    pairs = R.GemmPlan(512, 512, 4096, W.BF16)
    pairs2 = R.GemmPlan(1024, 1024, 4096, W.BF16)   # 32 tiles: two pairs per cluster
    forced4 = R.GemmPlan(256, 256, 4096, W.BF16, k_split=3)
    assert (pairs.info["kernel_name"], pairs.info["split_k"], pairs.info["launches"]) == ("tcgen05_pair", 1, 1)
    assert (pairs.info["num_ctas"], pairs.info["tile_n"], pairs.workspace_bytes) == (64, 128, 0)
    assert (pairs2.info["split_k"], pairs2.info["num_ctas"], pairs2.workspace_bytes) == (1, 128, 0)
    assert (forced4.info["kernel_name"], forced4.info["num_ctas"]) == ("tcgen05_pair", 16)
    # two tiles are not the plan's own choice for this form, nor is a K of 32 k-blocks on 32 tiles
    assert R.GemmPlan(256, 256, 4096, W.BF16).info["kernel_name"] == "tcgen05"
    assert R.GemmPlan(1024, 1024, 2048, W.BF16).info["split_k"] == 0
    for p in (pairs, pairs2, forced4):
        p.close()
    with pytest.raises(R.FriskError) as e:
        R.GemmPlan(512, 512, 512, W.BF16, k_split=4)
    assert e.value.code == -1


def test_forced_pair_split_forms_keep_their_invariants_over_random_shapes():
    """k_split = 2 (K planes) and 3 (K split over the CTA pairs of a cluster) on seeded random
    problems: where the form exists the plan fits the device (an even number of CTAs, at most one
    per SM), K planes ask for one fp32 copy of C per part and launch twice, pair clusters ask for
    nothing and launch once; where it does not, the plan is what k_split = 0 or -1 would give."""
    import random
    rnd = random.Random(7)
    forms = {2: 0, 3: 0}
    for _ in range(120):
        M = rnd.choice([130, 200, 256, 300, 512, 640, 1000, 1024, 2048, 4096])
        N = rnd.choice([72, 128, 200, 256, 520, 1024, 2048, 4104])   # (16-byte pitches: no repack)
        K = rnd.choice([512, 1024, 2064, 4096, 8192, 32768])
        ab = rnd.choice([W.BF16, W.F16, W.E4M3])
        ks = rnd.choice([2, 3])
        kw = dict(transB=True) if ab == W.E4M3 else {}
        p = R.GemmPlan(M, N, K, ab, W.BF16, k_split=ks, scales=ab == W.E4M3, **kw)
        i, ws = p.info, p.workspace_bytes
        p.close()
        if not (i["kernel_name"] == "tcgen05_pair" and i["split_k"]):
            continue
        assert i["num_ctas"] % 2 == 0 and 4 <= i["num_ctas"] <= 148 and i["tile_m"] == 256, (M, N, K, i)
        if ks == 2:
            tiles = -(-M // 256) * -(-N // i["tile_n"])
            parts = i["num_ctas"] // 2 // tiles if i["num_ctas"] // 2 >= tiles else 0
            assert i["launches"] == 2 and ws >= 2 * M * N * 4 and ws <= 20 << 20, (M, N, K, i, ws)
            assert parts == 0 or ws >= parts * M * N * 4
        else:
            tiles = -(-M // 256) * -(-N // 128)
            assert i["launches"] == 1 and ws == 0 and i["tile_n"] == 128, (M, N, K, i)
            assert i["num_ctas"] == tiles * 8 or i["num_ctas"] == tiles * 4
        forms[ks] += 1
    assert forms[2] >= 10 and forms[3] >= 10, forms


def test_plan_info_says_why_a_plan_runs_on_cuda_cores():
    """FRISK_TC_* of include/frisk_b200.h: a plan that resolved to the CUDA-core kernel names the
    rule that kept it off the tensor cores, so a 100x slower run is never a silent one."""
    cases = [
        (dict(ab=W.F32), 1),                                   # FRISK_TC_INPUT_TYPE
        (dict(ab=W.E4M3, ct=W.BF16, transB=False), 4),         # FRISK_TC_FP8_ORDER
        (dict(ab=W.BF16, force_kernel="simt"), 5),             # FRISK_TC_FORCED
    ]
    for kw, reason in cases:
        kw = dict(kw)
        ab, ct = kw.pop("ab"), kw.pop("ct", None)
        p = R.GemmPlan(96, 112, 96, ab, ct, **kw)
        assert p.info["kernel_name"] == "simt" and p.info["cuda_core_reason"] == reason, (kw, p.info)
        assert p.info["cuda_core_runs"] == 0
        p.close()
    p = R.GemmPlan(256, 256, 256, W.BF16)
    assert p.info["cuda_core_reason"] == 0
    p.close()


def test_plan_create_rejects_bad_descriptions():
    for kw in (dict(M=0), dict(K=-1), dict(lda=3), dict(ldc=5), dict(stages=-1), dict(band_tiles=-2)):
        args = dict(M=8, N=8, K=8)
        args.update({k: v for k, v in kw.items() if k in args})
        extra = {k: v for k, v in kw.items() if k not in args}
        with pytest.raises(R.FriskError) as e:
            R.GemmPlan(args["M"], args["N"], args["K"], W.F32, **extra)
        assert e.value.code == -1
    L = R.lib()
    d = R.GemmDesc()
    d.M = d.N = d.K = 8
    d.a_type, d.b_type, d.c_type = W.F16, W.BF16, W.F16  # ffi/ir.cpp:357-359: one element type
    h = C.c_void_p()
    assert L.frisk_b200_gemm_plan_create(C.byref(d), C.byref(h)) == -1
    assert L.frisk_b200_gemm_plan_create(None, C.byref(h)) == -1
    d.b_type = W.F16
    for fp8 in (W.E4M3, W.E5M2):   # 8-bit floats are input types only
        d.c_type = fp8
        assert L.frisk_b200_gemm_plan_create(C.byref(d), C.byref(h)) == -2
    d.a_type = d.b_type = 5        # no such type
    d.c_type = W.F16
    assert L.frisk_b200_gemm_plan_create(C.byref(d), C.byref(h)) == -1
    p5 = R.GemmPlan(512, 512, 512, W.E5M2, W.BF16, transB=True, scales=True)
    assert p5.info["kernel_name"] == "tcgen05_pair" and p5.info["tile_k"] == 128
    p5.close()
    p = R.GemmPlan(100, 100, 100, W.BF16, lda=101, force_kernel="tcgen05")   # odd pitches (B: 200 bytes): both repacked
    assert p.info["kernel_name"] == "tcgen05" and p.info["launches"] == 3
    p.close()


def test_run_without_device_reports_no_device_or_runs():
    import torch

    plan = R.GemmPlan(8, 8, 8, W.F32)
    a = np.zeros((8, 8), np.float32)
    if not torch.cuda.is_available():
        with pytest.raises(R.FriskError) as e:
            plan.run_host(a, a, a.copy())
        assert e.value.code == -7
    L = R.lib()
    assert L.frisk_b200_gemm_run(None, None, None, None, None, None, None, 0, None, None) == -1
    plan.close()


def test_fp32_plans_split_into_tf32_when_large():
    """fp32 inputs: the CUDA-core kernel for small problems (cfg1), three tf32 products on the
    tensor cores from about 1 GFLOP on; the split operands live in the workspace."""
    small = R.GemmPlan(512, 512, 512, W.F32)
    assert small.info["kernel_name"] == "simt" and small.workspace_bytes == 0
    small.close()
    big = R.GemmPlan(4096, 4096, 4096, W.F32)
    assert big.info["kernel_name"] == "tf32x3" and big.info["launches"] == 3
    assert (big.info["tile_m"], big.info["tile_n"], big.info["tile_k"]) == (256, 256, 32)
    assert big.workspace_bytes == 2 * 2 * 4096 * 4096 * 4       # A' and B': two K segments (lo, hi) each
    lay = big.operand_layout(0)
    assert (lay["swizzle_bytes"], lay["box_inner"], lay["k_step_bytes"]) == (128, 32, 32)
    big.close()
    forced = R.GemmPlan(512, 512, 512, W.F32, force_kernel="tf32x3")
    assert forced.info["kernel_name"] == "tf32x3"
    forced.close()
    few = R.GemmPlan(64, 8192, 4096, W.F32)                      # few rows: one-CTA whole tiles
    assert few.info["kernel_name"] == "tf32x3" and few.info["tile_m"] == 128
    few.close()
    odd = R.GemmPlan(4096, 4096, 4095, W.F32)                    # 16380-byte rows: no TMA
    assert odd.info["kernel_name"] == "simt"
    odd.close()
    for kw, code in ((dict(ab=W.BF16), -2), (dict(ab=W.F32, lda=4098), -3), (dict(ab=W.F32, ct=W.BF16), -3)):
        with pytest.raises(R.FriskError) as e:
            R.GemmPlan(4096, 4096, 4096, kw["ab"], kw.get("ct"), force_kernel="tf32x3", lda=kw.get("lda", 0))
        assert e.value.code == code, kw


def test_run_ex_argument_errors():
    """Host-side checks of frisk_b200_gemm_run_ex that come before any device work."""
    L = R.lib()
    plan = R.GemmPlan(256, 256, 256, W.BF16, row_reduce="max")
    tiles_c = 256 // plan.info["tile_n"]
    assert plan.workspace_bytes == 2 * tiles_c * 256 * 4 and plan.info["launches"] == 2   # a fold per row and half tile
    a = R.GemmRunArgs()
    assert L.frisk_b200_gemm_run_ex(plan._h, None) == -1
    assert L.frisk_b200_gemm_run_ex(None, C.byref(a)) == -1
    a.A = a.B = a.C = 256
    a.n_peers = 8                                             # at most seven other GPUs
    assert L.frisk_b200_gemm_run_ex(plan._h, C.byref(a)) == -1
    a.n_peers = 2                                             # ... each with a destination
    a.peer_c[0] = 512
    assert L.frisk_b200_gemm_run_ex(plan._h, C.byref(a)) == -1
    a.n_peers = 0                                             # a fused reduce needs its destination
    assert L.frisk_b200_gemm_run_ex(plan._h, C.byref(a)) == -1
    plan.close()
    for bad in (dict(epilogue=5), dict(epilogue=-1)):
        with pytest.raises(R.FriskError) as e:
            R.GemmPlan(256, 256, 256, W.BF16, **bad)
        assert e.value.code == -1
    d = R.GemmDesc()
    d.M = d.N = d.K = 256
    d.a_type = d.b_type = d.c_type = W.BF16
    d.row_reduce = 5
    h = C.c_void_p()
    assert L.frisk_b200_gemm_plan_create(C.byref(d), C.byref(h)) == -1
    # the whole-tile epilogue keeps 16 KiB of staging behind the pipeline stages, whichever way it
    # stores (its element-wise path uses the area too): six stages of 32 KiB for the CTA-pair kernel
    p2, p1 = R.GemmPlan(4096, 4096, 4096, W.BF16, epilogue=2), R.GemmPlan(4096, 4096, 4096, W.BF16, epilogue=1)
    assert (p2.info["stages"], p1.info["stages"]) == (6, 6)
    assert p2.info["smem_bytes"] <= 226 * 1024
    p1.close()
    p2.close()
    # TMA stores take two staging buffers per warp (32 KiB) and still leave six stages
    p4 = R.GemmPlan(4096, 4096, 4096, W.BF16, epilogue=4)
    assert p4.info["kernel_name"] == "tcgen05_pair" and p4.info["stages"] == 6
    assert p2.info["smem_bytes"] + 16 * 1024 == p4.info["smem_bytes"] <= 226 * 1024
    p4.close()
    # peer buffers: argument errors need no device
    assert L.frisk_b200_peer_alloc(0, C.byref(h), C.create_string_buffer(64)) == -1
    assert L.frisk_b200_peer_open(None, C.byref(h)) == -1
    assert L.frisk_b200_peer_close(None) == 0 and L.frisk_b200_peer_free(None) == 0
    tf = C.c_double()
    assert L.frisk_b200_measure_mma_peak(W.BF16, 1, 33, 1, C.byref(tf), None) == -1   # k_blocks % 32
    assert L.frisk_b200_measure_mma_peak(9, 1, 64, 1, C.byref(tf), None) == -2


@pytest.mark.parametrize("M,P", [(65536, 1), (65536, 2), (65536, 4), (65536, 8), (10, 3), (7, 8), (0, 4)])
def test_shard_rows_partitions_every_row_once(M, P):
    covered = []
    for r in range(P):
        row0, rows = R.shard_rows(M, P, r)
        covered.extend(range(row0, row0 + rows))
        assert rows in (M // P, M // P + 1)
    assert covered == list(range(M))
    if M % P == 0 and M:
        assert R.shard_rows(M, P, P - 1) == (M - M // P, M // P)


def test_shard_rows_errors():
    for bad in ((8, 0, 0), (8, 4, 4), (8, 4, -1)):
        with pytest.raises(R.FriskError) as e:
            R.shard_rows(*bad)
        assert e.value.code == -8


def test_planner_invariants_over_random_shapes():
    """Whatever the shape, a plan names a kernel the library has, fits the SM (shared memory,
    pipeline depth, grid) and states its workspace; few-row plans either need no workspace
    (clusters) or the stream-K one."""
    import random
    rnd = random.Random(5)
    seen = set()
    for _ in range(400):
        ab = rnd.choice([W.F32, W.F16, W.BF16, W.E4M3, W.E5M2])
        ct = ab if ab not in (W.E4M3, W.E5M2) else W.BF16
        M = rnd.choice([1, 7, 16, 33, 64, 65, 100, 128, 129, 200, 256, 1000, 4096, 8192])
        N = rnd.choice([8, 64, 104, 256, 512, 1000, 2048, 4096, 8192, 28672])
        K = rnd.choice([8, 64, 72, 520, 1024, 4096, 8192])
        ta, tb = rnd.random() < 0.2, rnd.random() < 0.5
        if ab in (W.E4M3, W.E5M2) and (ta or not tb):
            ta, tb = False, True  # 8-bit inputs run on tensor cores only K-inner
        p = R.GemmPlan(M, N, K, ab, ct, transA=ta, transB=tb, scales=ab in (W.E4M3, W.E5M2))
        i = p.info
        seen.add(i["kernel_name"])
        assert i["kernel_name"] in ("simt", "tcgen05", "tcgen05_pair", "skinny", "tf32x3")
        # operands with an odd row pitch are repacked into the workspace: a launch and a padded copy each
        es = W.ELEM_SIZE[ab]
        repack = 0
        if ab != W.F32 and i["kernel_name"] != "simt":
            for rows, cols in (((K, M) if ta else (M, K)), ((N, K) if tb else (K, N))):
                if cols * es % 16:
                    repack += (rows * (-(-cols * es // 16) * 16) + 255) // 256 * 256
        n_repack = 0 if not repack else sum(1 for c in ((M if ta else K), (K if tb else N)) if c * es % 16)
        planes = i["kernel_name"] == "tcgen05_pair" and i["split_k"] and p.workspace_bytes - repack > 0
        assert i["launches"] == (3 if i["kernel_name"] == "tf32x3" else 2 if planes else 1) + n_repack
        assert i["num_ctas"] >= 1
        own_ws = p.workspace_bytes - repack
        if i["kernel_name"] == "tf32x3":   # fp32 in and out, at least about a GFLOP, TMA-able rows
            assert ab == W.F32 and 2.0 * M * N * K >= 1e9 and p.workspace_bytes >= 2 * 4 * (M * K + K * N)
        if i["kernel_name"] != "simt":
            assert 2 <= i["stages"] <= 12 and i["smem_bytes"] <= 227 * 1024
            assert i["num_ctas"] <= 148 and i["tile_k"] * W.ELEM_SIZE[ab] == 128
        if i["kernel_name"] == "tcgen05_pair":
            assert i["num_ctas"] % 2 == 0 and i["tile_m"] == 256 and M > 128
        if i["kernel_name"] == "skinny":
            assert M <= 128 and N >= 256 and not ta and i["swap_ab"] == 1
            assert i["tile_m"] == (M + 15) // 16 * 16 and i["tile_n"] in (128, 256)
            if own_ws == 0:              # clusters: tiles x a power-of-two cluster size
                tiles = -(-N // i["tile_n"])
                assert i["num_ctas"] % tiles == 0 and i["num_ctas"] // tiles in (2, 4, 8)
            else:                        # stream-K: slots + one counter per tile
                assert own_ws % 4 == 0 and i["num_ctas"] <= 14 * -(-N // i["tile_n"])
        elif i["kernel_name"] == "tcgen05" and i["split_k"]:
            # few tiles against a long K: the K-split forms without the swap
            assert K >= 48 * i["tile_k"] and i["swap_ab"] == 0 and i["tile_m"] in (128, 256)
            tiles = -(-M // i["tile_m"]) * -(-N // i["tile_n"])
            if own_ws == 0:
                assert i["num_ctas"] % tiles == 0 and i["num_ctas"] // tiles in (2, 4, 8)
            else:
                assert own_ws % 4 == 0 and i["num_ctas"] <= 14 * tiles
        elif i["kernel_name"] == "tcgen05_pair" and i["split_k"]:
            tiles = -(-M // 256) * -(-N // i["tile_n"])
            if i["launches"] - n_repack == 2:   # K planes: one fp32 copy of C per K part
                assert own_ws >= 2 * M * N * 4 and i["num_ctas"] % 2 == 0
            else:                               # K split over the pairs of a cluster
                assert own_ws == 0 and i["tile_n"] == 128 and i["num_ctas"] // tiles in (4, 8)
                assert K >= 32 * i["tile_k"]
        elif i["kernel_name"] != "tf32x3":
            assert own_ws == 0 and not i["split_k"]
        p.close()
    assert seen == {"simt", "tcgen05", "tcgen05_pair", "skinny", "tf32x3"}


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    """No CPU fallback: without libfrisk_b200.so every entry point raises, nothing computes."""
    monkeypatch.setattr(R, "LIB_PATH", str(tmp_path / "libfrisk_b200.so"))
    monkeypatch.setattr(R, "_lib", None)
    try:
        with pytest.raises(R.FriskError, match="missing"):
            R.GemmPlan(8, 8, 8, W.F32)
        with pytest.raises(R.FriskError, match="missing"):
            R.gemm_host(W.make_workload("cfg1", 8, 8, 8))
    finally:
        monkeypatch.undo()


def test_reduce_plans_cover_the_reduced_dimension_exactly_once():
    """frisk_b200_reduce_info is host arithmetic (it assumes 148 SMs when no device is visible):
    the pieces tile the reduced dimension, the workspace holds one fp32 per piece and output
    element, and the workspace query covers both alignments of the source."""
    rng = np.random.default_rng(0)
    shapes = [((8192, 8192), 1), ((8192, 8192), 0), ((1, 1 << 26), 1), ((4, 8, 16), 1), ((0, 8), 1),
              ((5, 0), 1), ((3, 7, 0), 1)]
    for _ in range(200):
        rank = int(rng.integers(1, 4))
        shape = tuple(int(rng.choice([1, 2, 3, 5, 8, 16, 33, 100, 1000, 4096, 70001])) for _ in range(rank))
        if np.prod(shape, dtype=np.int64) > 1 << 34:
            continue
        shapes.append((shape, int(rng.integers(0, rank))))
    for shape, dim in shapes:
        for dtype in (W.F32, W.F16, W.BF16):
            d = R.reduce_desc(shape, dim, dtype, "max")
            need = R.reduce_workspace_bytes(d)
            for aligned in (True, False):
                info = R.reduce_info(d, aligned)
                empty = d.outer == 0 or d.inner == 0
                assert info["launches"] == (0 if empty else 2 if info["chunks"] > 1 else 1)
                assert info["lines"] == int(d.inner == 1)
                assert info["chunks"] >= 1 and info["chunk_len"] >= 1
                if not empty:
                    assert info["chunks"] * info["chunk_len"] >= d.extent
                    assert (info["chunks"] - 1) * info["chunk_len"] < max(d.extent, 1)
                    assert info["ctas"] >= 1
                want_ws = d.outer * info["chunks"] * d.inner * 4 if info["chunks"] > 1 else 0
                assert info["workspace_bytes"] == want_ws <= need
                if not aligned and d.inner != 1:
                    assert info["vector"] == 1
    assert R.reduce_info(R.reduce_desc((8192, 8192), 1, W.F16, "max")) == dict(
        lines=1, vector=8, chunks=1, launches=1, chunk_len=8192, ctas=1024, workspace_bytes=0)
    with pytest.raises(R.FriskError) as e:
        R.reduce_info(R.reduce_desc((4, 4), 1, W.E4M3, "add"))
    assert e.value.code == -2
    bad = R.reduce_desc((4, 4), 1, W.F32, "add")
    bad.kind = 9
    with pytest.raises(R.FriskError) as e:
        R.reduce_info(bad)
    assert e.value.code == -1
