"""Layout mapping and cost model against the reference's pinned outputs: the shared-memory maps
GemmOp::inferLayout printed for five cases (tmp/log_12_18, evaluated point-wise as functions), the
swizzle selection rule of FriskOps.cpp:589-618, and the bank statistics of
exp/layout/result/log_12_23."""
import json
import os

import pytest

import frisk as F
from frisk_b200 import runtime as R
from frisk_b200 import workloads as W

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def eval_map(text, d0, d1):
    """Evaluates the results of a printed affine map '(d0, d1) -> (e0, e1, ...)' at a point."""
    body = text.split("->", 1)[1].strip()
    assert body[0] == "(" and body[-1] == ")"
    py = body[1:-1].replace("floordiv", "//").replace("mod", "%")
    return list(eval("(" + py + ",)", {"d0": d0, "d1": d1}))


def golden_cases():
    gold = json.load(open(os.path.join(GOLDEN, "layouts.json")))
    out = []
    for case in gold["cases"]:
        for operand, lay in case["layouts"].items():
            if lay["kind"] == "Layout":  # shared-memory operands (fragments are register layouts)
                out.append((case["name"], case["target"], operand, lay))
    return out


@pytest.mark.parametrize("name,target,operand,lay", golden_cases(),
                         ids=[f"{c[0]}-{c[2]}" for c in golden_cases()])
def test_shared_layout_maps_equal_reference_pointwise(name, target, operand, lay):
    rows, cols = lay["shape"]
    h = F.create_session()
    f16 = h.builder.get_f16_ty()
    tys = [h.memref_type((128, 64), f16, space=F.MemorySpace.SHARED),
           h.memref_type((64, 128), f16, space=F.MemorySpace.SHARED),
           h.memref_type((128, 128), f16, space=F.MemorySpace.LOCAL)]
    _, entry = h.new_kernel(name, tys)
    g = h.create_gemm(*[entry.get_argument(i) for i in range(3)])
    attr = g.infer_shared_layout(operand, hopper=target == "sm_90")
    amap = F.frisk.layout_index_map(attr)
    assert amap.get_num_results() == 3
    tma = R.layout_to_tma(rows, cols, 16, k_inner=(operand == "A"))
    assert tma["swizzle_bytes"] == 128 and tma["reference_layout"] == "full_bank"
    span = tma["swizzle_bytes"]
    for i in range(rows):
        for j in range(0, cols, 3):
            want = eval_map(lay["index"], i, j)
            assert amap.evaluate([i, j]) == want
            tc, ts, index = want
            # the same element where TMA puts it: one box per column atom, 8-row atoms inside
            off = R.swizzled_offset(i, j, rows, cols, 16, span)
            assert off == tc * rows * span + ts * 8 * span + index * 2


@pytest.mark.parametrize("bits", [8, 16, 32])
def test_swizzle_selection_rule_and_descriptor_fields(bits):
    vec = 128 // bits
    es = bits // 8
    for cont, sw, name, ltype in ((vec * 8, 128, "full_bank", 2), (vec * 16, 128, "full_bank", 2),
                                  (vec * 4, 64, "half_bank", 4), (vec * 12, 64, "half_bank", 4),
                                  (vec * 2, 32, "quarter_bank", 6), (vec * 3, 0, "linear", 0)):
        for k_inner in (True, False):
            p = R.layout_to_tma(64, cont, bits, k_inner)
            assert (p["swizzle_bytes"], p["reference_layout"], p["umma_layout_type"]) == (sw, name, ltype)
            assert p["umma_major"] == (0 if k_inner else 1)
            span = sw or 16
            assert p["box_inner"] * es == span and p["box_outer"] == 64
            assert p["num_boxes"] * span == cont * es
            assert p["stride_byte_offset"] == 8 * span
            if k_inner:
                assert p["k_step_bytes"] == 32
            else:
                assert p["k_step_bytes"] == (32 // es) * span and p["leading_byte_offset"] == 64 * span
    with pytest.raises(R.FriskError) as e:
        R.layout_to_tma(64, vec + 1, bits, True)  # the reference returns no layout either
    assert e.value.code == -3
    with pytest.raises(R.FriskError):
        R.layout_to_tma(64, 64, 64, True)  # f64 has no tcgen05 operand type
    with pytest.raises(R.FriskError):
        R.layout_to_tma(512, 64, 16, True)  # more rows than a TMA box holds


def test_kernel_operand_layouts_are_the_mapped_ones():
    """The mapper's answers for the tile shapes the kernels stage, as literals."""
    a = R.layout_to_tma(128, 64, 16, True)    # A tile 128 x 64 bf16, K-major
    assert (a["swizzle_bytes"], a["num_boxes"], a["box_inner"], a["box_outer"]) == (128, 1, 64, 128)
    assert (a["stride_byte_offset"], a["k_step_bytes"]) == (1024, 32)
    b = R.layout_to_tma(64, 256, 16, False)   # B tile 64 (K) x 256 (N) bf16, N contiguous
    assert (b["num_boxes"], b["box_inner"], b["box_outer"]) == (4, 64, 64)
    assert (b["leading_byte_offset"], b["stride_byte_offset"], b["k_step_bytes"]) == (8192, 1024, 2048)
    f8 = R.layout_to_tma(256, 128, 8, True)   # e4m3 B tile 256 x 128, K-major
    assert (f8["swizzle_bytes"], f8["box_inner"], f8["k_step_bytes"]) == (128, 128, 32)


@pytest.mark.parametrize("dims,ab,kw,tiles", [
    # (M, N, K), input type, plan options, ((rows, cols, k_inner) of the staged A-role / B-role tile)
    ((8192, 8192, 8192), W.BF16, {}, ((128, 64, True), (64, 128, False))),            # pair: half of B per CTA
    ((4096, 4096, 4096), W.F16, dict(transB=True), ((128, 64, True), (128, 64, True))),
    ((8192, 8192, 8192), W.E4M3, dict(transB=True, c_type=W.BF16, scales=True), ((128, 128, True), (128, 128, True))),
    ((384, 1024, 2048), W.BF16, dict(transA=True), ((64, 128, False), (64, 64, False))),    # A stored [K, M]; 128-wide tiles
    ((128, 512, 256), W.BF16, dict(force_kernel="tcgen05"), ((128, 64, True), (64, 256, False))),
    ((16, 8192, 8192), W.BF16, {}, ((64, 256, False), (16, 64, True))),               # few rows: weights first
    ((64, 8192, 256), W.F16, dict(transB=True), ((256, 64, True), (64, 64, True))),
])
def test_plans_stage_exactly_what_the_layout_mapper_says(dims, ab, kw, tiles):
    """The plan's TMA boxes and UMMA descriptors come from frisk_b200_layout_to_tma: for every
    operand of every kernel family the plan reports the mapper's answer for the staged tile, and
    the 64-bit descriptor base the kernel runs on is that answer bit for bit."""
    kw = dict(kw)
    plan = R.GemmPlan(*dims, ab, kw.pop("c_type", None), **kw)
    bits = 8 * W.ELEM_SIZE[ab]
    for operand, (rows, cols, k_inner) in enumerate(tiles):
        got = plan.operand_layout(operand)
        want = R.layout_to_tma(rows, cols, bits, k_inner)
        for key, value in want.items():
            assert got[key] == value, (operand, key, got[key], value)
        assert got["swizzle_bytes"] == 128 == plan.info["swizzle_a"] == plan.info["swizzle_b"]
        d = got["umma_desc_base"]
        assert (d >> 16) & 0x3FFF == want["leading_byte_offset"] // 16
        assert (d >> 32) & 0x3FFF == want["stride_byte_offset"] // 16
        assert (d >> 46) & 1 == 1 and (d >> 61) & 7 == want["umma_layout_type"] == 2
        assert d & 0x3FFF == 0                       # the start address is added per stage
        # the copies of a stage cover the tile: the mapper's boxes, or (a K-major half of B in the
        # CTA-pair kernel, so that a half-width item can load half of it) two boxes of half the rows
        assert got["tma_boxes_per_stage"] in (want["num_boxes"], 2 * want["num_boxes"])
    plan.close()
    p = R.GemmPlan(64, 64, 64, W.F32)
    with pytest.raises(R.FriskError):
        p.operand_layout(0)   # the CUDA-core kernel stages nothing by TMA
    p.close()


def test_swizzled_offsets_are_a_permutation_of_the_tile():
    for mode in (0, 32, 64, 128, R.SWIZZLE_128B_ATOM_32B, R.SWIZZLE_128B_ATOM_64B):
        rows, cols, bits = 16, 128, 16
        offs = {R.swizzled_offset(i, j, rows, cols, bits, mode) for i in range(rows) for j in range(cols)}
        assert offs == set(range(0, rows * cols * 2, 2))
    assert R.swizzled_offset(0, 128, 16, 128, 16, 128) == -1
    assert R.swizzled_offset(0, 0, 16, 100, 16, 128) == -1  # row not a multiple of the span


def test_bank_model_reproduces_reference_statistics():
    gold = json.load(open(os.path.join(GOLDEN, "bank_stats.json")))
    lv = gold["config"]["lane_vector"]
    checked = 0
    for lay in gold["layouts"]:
        if "bank_stats" not in lay or lay["operand"] == "C":
            continue
        rows, cols = lay["shape"]
        ours = R.bank_conflicts(rows, cols, lay["element_bits"], 128, lv)
        base = R.bank_conflicts(rows, cols, lay["element_bits"], 0, lv)
        for got, want in ((ours, lay["bank_stats"]), (base, lay["baseline_row_major"])):
            assert got["samples"] == want["samples"]
            assert got["max_conflict"] == want["max_conflict"]
            assert got["avg_max_conflict"] == pytest.approx(want["avg_max_conflict"])
        checked += 1
    assert checked == 2


def test_bank_model_blackwell_modes_and_distinct_word_counting():
    # counting distinct 4-byte words per bank (what the hardware serialises on): a 512-byte warp
    # request over a swizzled or a linear 128-byte-row tile needs 4 wavefronts, the minimum
    for mode in (0, 32, 64, 128, R.SWIZZLE_128B_ATOM_32B, R.SWIZZLE_128B_ATOM_64B):
        st = R.bank_conflicts(128, 64, 16, mode, 8, distinct_words_only=True)
        assert st["samples"] == 32 and st["max_conflict"] == 4
    with pytest.raises(R.FriskError):
        R.bank_conflicts(128, 60, 16, 128, 8)


def test_access_patterns_tell_the_swizzle_modes_apart():
    """The reference's model walks row-major windows only, which every layout serves without
    conflicts.  The two patterns a swizzle exists for -- a chunk column (every lane another row,
    the same 16-byte chunk: the ldmatrix / UMMA operand fetch, and the staged epilogue's writes)
    and row pieces (consecutive lanes along a row: the staged epilogue's read-back) -- separate
    the modes.  Tile: 32 rows x 128 bytes, the staging area of one epilogue warp."""
    col = {m: R.bank_conflicts_access(32, 64, 16, m, R.ACCESS_CHUNK_COLUMN) for m in
           (0, 32, 64, 128, R.SWIZZLE_128B_ATOM_32B, R.SWIZZLE_128B_ATOM_64B)}
    row = {m: R.bank_conflicts_access(32, 64, 16, m, R.ACCESS_ROW_PIECES) for m in col}
    # plain 128-byte rows: the 8 rows of a quarter warp all start in the same bank -> 8 passes
    assert col[0]["conflict_degree"] == 8.0 and col[0]["max_wavefronts_per_request"] == 32
    assert row[0]["conflict_degree"] == 1.0
    # the three TMA swizzles spread a chunk column over all banks ...
    for m in (32, 64, 128):
        assert col[m]["conflict_degree"] == 1.0 and col[m]["max_wavefronts_per_request"] == 4
    # ... but only the 128-byte one keeps a 128-byte row in one box: the narrower ones cut it
    # into 2 or 4 boxes a multiple of 1 KiB apart, which collide when a row is read back
    assert [row[m]["conflict_degree"] for m in (32, 64, 128)] == [4.0, 2.0, 1.0]
    assert [col[m]["tma_boxes"] for m in (32, 64, 128)] == [4, 2, 1]
    assert [col[m]["global_segment_bytes"] for m in (32, 64, 128)] == [32, 64, 128]
    # the coarser atoms of the 128-byte swizzle move 32 or 64 bytes at a time: fine for accesses
    # of that width, 2- and 4-way conflicts for 16-byte chunk columns
    assert col[R.SWIZZLE_128B_ATOM_32B]["conflict_degree"] == 2.0
    assert col[R.SWIZZLE_128B_ATOM_64B]["conflict_degree"] == 4.0
    assert row[R.SWIZZLE_128B_ATOM_32B]["conflict_degree"] == 1.0
    # so the one mode that is conflict-free both ways, with the fewest copies and the longest
    # global segments, is the 128-byte swizzle: what the plans and the staged epilogue use
    best = min(col, key=lambda m: (col[m]["conflict_degree"] * row[m]["conflict_degree"], col[m]["tma_boxes"] or 99))
    assert best == 128
    # the operand tiles of the kernels, fetched by chunk columns: conflict-free in the mapped mode
    for rows, cols, bits in ((128, 64, 16), (256, 128, 8), (64, 128, 16)):
        mode = R.layout_to_tma(rows, cols, bits, True)["swizzle_bytes"]
        assert R.bank_conflicts_access(rows, cols, bits, mode, R.ACCESS_CHUNK_COLUMN)["conflict_degree"] == 1.0
    with pytest.raises(R.FriskError):
        R.bank_conflicts_access(32, 60, 16, 128, R.ACCESS_CHUNK_COLUMN)   # rows are not whole chunks
    with pytest.raises(R.FriskError):
        R.bank_conflicts_access(32, 64, 16, 128, 7)


def test_accumulator_layout_on_sm100_is_the_tensor_memory_map():
    """Addition: where the reference gives C a register fragment (mma.sync / wgmma ownership,
    FriskOps.cpp:304-347), tcgen05 keeps the accumulator in tensor memory: tile row r in lane r,
    column c in column c; tcgen05.ld.32x32b gives thread r its row, columns as registers."""
    h = F.create_session()
    f16 = h.builder.get_f16_ty()
    tys = [h.memref_type((128, 64), f16, space=F.MemorySpace.SHARED),
           h.memref_type((64, 256), f16, space=F.MemorySpace.SHARED),
           h.memref_type((128, 256), f16, space=F.MemorySpace.LOCAL)]
    _, entry = h.new_kernel("acc", tys)
    g = h.create_gemm(*[entry.get_argument(i) for i in range(3)])
    attr = g.infer_accumulator_layout_sm100(128, 256)
    assert str(attr) == ("#frisk.layout<[128, 256], affine_map<(d0, d1) -> (d1)>, "
                         "affine_map<(d0, d1) -> (d0)>, 1>")
    index = F.frisk.layout_index_map(attr)
    for r, c in ((0, 0), (5, 17), (127, 255)):
        assert index.evaluate([r, c]) == [c]   # register j of thread r holds column j
    with pytest.raises(ValueError):
        g.infer_accumulator_layout_sm100(64, 256)
    with pytest.raises(ValueError):
        g.infer_accumulator_layout_sm100(128, 260)
