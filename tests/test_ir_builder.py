"""The IR-builder surface (``import frisk as F``) against the reference's pinned outputs:
the module text of test/python/bind_test.py (tmp/log_11_18), attribute and module prints of
test_pass/attr_test.cpp (tmp/log_12_18), plus the flows of helper_test.py and map_expr_test.py
and the error conventions of ffi/ir.cpp."""
import json
import os
import subprocess
import sys

import pytest

import frisk as F

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden")
# a checkout of the reference beside this repository, when there is one (else those tests skip)
REFERENCE = os.environ.get("FRISK_REFERENCE_ROOT", os.path.normpath(os.path.join(HERE, "..", "..", "reference")))


def build_bind_test_module():
    """The construction sequence of the reference's flagship script (bind_test.py:3-60)."""
    context = F.context()
    F.frisk.load_dialects(context)
    builder = F.builder(context)
    module = builder.create_module()
    module.context = context
    dtype = builder.get_f16_ty()
    mem_type = builder.get_memref_ty(dtype, [4096, 4096], F.AffineMap(), F.MemorySpace.GLOBAL)
    mem2_type = builder.get_memref_ty(dtype, [4096], F.AffineMap(), F.MemorySpace.GLOBAL)
    kernel_type = builder.get_kernel_ty([mem_type, mem_type, mem_type, mem2_type])
    kernel = builder.create_kernel_op(module, "test_gemm", kernel_type)
    module.push_back(kernel)
    entry1 = kernel.add_entry_block()
    builder.set_insertion_point_to_start(entry1)
    parallel = builder.create_parallel_op([8, 8], 128)
    entry2 = parallel.add_entry_block()
    builder.set_insertion_point_to_start(entry2)
    vals = [entry1.get_argument(i) for i in range(4)]
    builder.create_alloc_buffer_op([128, 32], "fp16", F.MemorySpace.SHARED, 1024)
    builder.create_alloc_buffer_op([32, 128], "fp16", F.MemorySpace.SHARED, 1024)
    builder.create_alloc_buffer_op([128, 128], "fp16", F.MemorySpace.LOCAL)
    seen = {}

    def for_body(b, iv):
        builder.create_fill_op(vals[0], 0.0, "fp16")
        builder.create_reduce_op(vals[0], vals[3], "max", 1, True)
        seen["copy"] = builder.create_copy_op(vals[0], vals[1], [iv, iv], [iv, iv])

        def block_body(b2, ivs):
            seen["ivs"] = len(ivs)
            seen["gemm"] = b2.create_gemm_op(vals[0], vals[1], vals[2])

        seen["block"] = builder.create_block_op([128, 128], block_body)

    seen["for"] = builder.create_for_op(0, 128, 1, for_body)
    return module, kernel, parallel, seen


def test_bind_test_module_text_matches_reference_log():
    module, *_ = build_bind_test_module()
    want = open(os.path.join(GOLDEN, "bind_test_module.mlir")).read().rstrip("\n")
    assert str(module) == want
    assert module.verify()


def test_op_accessors_on_the_bind_test_module():
    module, kernel, parallel, seen = build_bind_test_module()
    assert kernel.get_num_arguments() == 4 and str(kernel.arg(3).get_type()) == "memref<4096xf16, 1>"
    with pytest.raises(IndexError):
        kernel.arg(4)
    assert parallel.get_grid() == [8, 8] and parallel.get_thread_num() == 128
    assert parallel.get_grid_dim() == 2 and len(parallel.get_ivs()) == 2
    f = seen["for"]
    assert (f.get_lower_bound(), f.get_upper_bound(), f.get_step()) == (0, 128, 1)
    assert str(f.get_induction_var()) == "%arg6"
    blk = seen["block"]
    assert blk.get_block_ranges() == [128, 128] and blk.get_iteration_num() == 128 * 128
    assert seen["ivs"] == 2
    cp = seen["copy"]
    assert cp.get_src_extents() == [4096, 4096] and cp.get_dst_extents() == [4096, 4096]
    assert cp.get_src_affine_map().is_identity() and len(cp.get_src_indices()) == 2
    g = seen["gemm"]
    assert g.get_attrs() == {"M": 4096, "N": 4096, "K": 4096, "transA": False, "transB": False,
                             "clear_accum": False, "policy": "Square"}
    assert str(g.get_matrix_C()) == "%arg2" and len(g.get_all_matrix()) == 3
    names = []
    module.walk(lambda op: names.append(op.get_name()))
    assert names[-1] == "builtin.module" and names.count("frisk.gemm") == 1
    assert module.get_kernel("test_gemm") is not None and module.get_kernel("nope") is None
    assert F.frisk.GemmOp.from_operation(g.get_operation()) is not None


def test_helper_flow():
    """helper_test.py:4-23."""
    helper = F.create_session()
    f16 = helper.builder.get_f16_ty()
    a_ty = helper.memref_type((128, 64), f16, space=F.MemorySpace.SHARED)
    b_ty = helper.memref_type((64, 128), f16, space=F.MemorySpace.SHARED)
    c_ty = helper.memref_type((128, 128), f16, space=F.MemorySpace.LOCAL)
    kernel, entry = helper.new_kernel("helper_demo", [a_ty, b_ty, c_ty])
    args = [entry.get_argument(i) for i in range(3)]
    helper.create_gemm(args[0], args[1], args[2])
    scratch = helper.alloc_buffer((32, 32), "fp16", space=F.MemorySpace.SHARED, alignment=64)
    assert "memref" in str(scratch.get_type())
    assert str(scratch.get_type()) == "memref<32x32xf16, 3>"
    assert kernel.verify() and helper.module.verify()
    text = str(helper.module)
    assert "frisk.kernel @helper_demo(memref<128x64xf16, 3>, memref<64x128xf16, 3>, memref<128x128xf16>)" in text
    assert '%0 = frisk.alloc_buffer {scope = "shared", alignment = 64} -> memref<32x32xf16, 3>' in text


def test_attr_test_module_and_attribute_prints():
    gold = json.load(open(os.path.join(GOLDEN, "layouts.json")))
    prints = gold["attr_prints"]
    for space in ("Local", "Global", "Shared"):
        assert str(F.frisk.enum_attr("memory_space", space)) in prints
    for pol in ("Square", "FullRow", "FullCol"):
        assert str(F.frisk.enum_attr("gemm_warp_policy", pol)) in prints
    ctx = F.context()
    b = F.builder(ctx)
    d0, d1 = b.get_affine_dim_expr(0), b.get_affine_dim_expr(1)
    lay = F.frisk.layout_attr([4, 4], F.AffineMap.get(2, 0, [d0 * 4 + d1], ctx))
    assert str(lay) in prints
    # the sm80_ss case of attr_test.cpp:159-232: module with a target attribute, gemm with a
    # thread-count attribute
    case = gold["cases"][0]
    helper = F.create_session()
    helper.module.set_str_attr("frisk.target", case["target"])
    f16 = helper.builder.get_f16_ty()
    tys = [helper.memref_type((128, 64), f16, space=F.MemorySpace.SHARED),
           helper.memref_type((64, 128), f16, space=F.MemorySpace.SHARED),
           helper.memref_type((128, 128), f16, space=F.MemorySpace.LOCAL)]
    kernel, entry = helper.new_kernel(case["name"], tys)
    g = helper.create_gemm(*[entry.get_argument(i) for i in range(3)])
    g.set_attr("frisk.threads", helper.builder.get_int64_attr(128))
    assert str(helper.module) == case["module"]


def test_map_expr_flow():
    """map_expr_test.py:3-25; expected strings follow MLIR's simplification and printing rules."""
    context = F.context()
    builder = F.builder(context)
    dim0 = builder.get_affine_dim_expr(0)
    symbol = builder.get_affine_symbol_expr(0)
    cst0 = builder.get_affine_constant_expr(0)
    cst5 = builder.get_affine_constant_expr(5)
    expr = dim0 * cst5 + symbol + cst0
    assert str(expr) == "d0 * 5 + s0"
    assert expr.get_kind() == F.AffineExprKind.Add
    expr2 = F.get_affine_binary_op_expr(expr.get_kind(), expr, expr)
    assert str(expr2) == "(d0 * 5 + s0) * 2"
    binary = expr2.as_binary()
    assert str(binary.get_lhs()) == "d0 * 5 + s0" and str(binary.get_rhs()) == "2"
    assert expr2.as_dim() is None and dim0.as_dim().get_position() == 0
    amap = F.AffineMap.get(1, 1, [expr2], context)
    assert str(amap) == "(d0)[s0] -> ((d0 * 5 + s0) * 2)"
    assert str(amap.get_result(0)) == str(amap.get_results()[0])
    assert amap.get_num_dims() == 1 and amap.get_num_symbols() == 1 and amap.get_num_inputs() == 2


def test_affine_printing_and_simplification_rules():
    ctx = F.context()
    b = F.builder(ctx)
    d0, d1, s0 = b.get_affine_dim_expr(0), b.get_affine_dim_expr(1), b.get_affine_symbol_expr(0)
    assert str(d0 - d1) == "d0 - d1"
    assert str(d0 - 3) == "d0 - 3"
    assert str(d0 + d1 * -4) == "d0 - d1 * 4"
    assert str(-d0) == "-d0"
    assert str((d0 + d1) * 2) == "(d0 + d1) * 2"
    assert str(d0.floor_div(8).floor_div(8)) == "(d0 floordiv 8) floordiv 8"
    assert str((d0 % 8).floor_div(2)) == "(d0 mod 8) floordiv 2"
    assert str(3 + d0) == "d0 + 3" and str(s0 + d0) == "d0 + s0"
    assert str((d0 + 2) + 3) == "d0 + 5" and str((d0 * 2) * 3) == "d0 * 6"
    assert str(d0 * 1) == "d0" and str(d0 + 0) == "d0" and str(d0 * 0) == "0"
    assert str((d0 * 8).floor_div(4)) == "d0 * 2" and str((d0 * 8) % 4) == "0"
    assert str((d0 * 8 + d1) % 4) == "d1 mod 4"
    assert (d0 * 4).get_largest_known_divisor() == 4 and (d0 * 4).is_multiple_of(2)
    assert d0.is_function_of_dim(0) and not d0.is_function_of_dim(1)
    assert (d0 + s0).is_function_of_symbol(0) and s0.is_symbolic_or_constant()
    assert (d0 * 3).is_pure_affine() and not (d0 * d1).is_pure_affine()
    m = F.AffineMap.get(2, 0, [d0 * 4 + d1, d1.floor_div(2)], ctx)
    assert m.evaluate([3, 5]) == [17, 2]
    assert F.AffineMap.get_multi_dim_identity_map(3, ctx).is_identity()
    assert F.AffineMap.get_permutation_map([1, 0], ctx).is_permutation()
    assert not F.AffineMap() and F.AffineMap.get(ctx).is_empty()
    assert str(F.AffineMap.get_constant_map(7, ctx)) == "() -> (7)"


def test_types_and_memory_spaces():
    ctx = F.context()
    b = F.builder(ctx)
    f16 = b.get_f16_ty()
    assert str(b.get_bf16_ty()) == "bf16" and str(b.get_f8e4m3fn_ty()) == "f8E4M3FN"
    g = b.get_memref_ty(f16, [4, 8])  # defaults: identity layout, GLOBAL (ffi/ir.cpp:256)
    assert str(g) == "memref<4x8xf16, 1>" and g.get_memory_space() == F.MemorySpace.GLOBAL
    l = b.get_memref_ty(f16, [4, 8], F.AffineMap(), F.MemorySpace.LOCAL)
    assert str(l) == "memref<4x8xf16>" and l.get_memory_space() == F.MemorySpace.LOCAL
    d0, d1 = b.get_affine_dim_expr(0), b.get_affine_dim_expr(1)
    t = b.get_memref_ty(f16, [4, 8], F.AffineMap.get(2, 0, [d1, d0], ctx), F.MemorySpace.SHARED)
    assert str(t) == "memref<4x8xf16, affine_map<(d0, d1) -> (d1, d0)>, 3>"
    assert g.get_rank() == 2 and g.get_shape() == [4, 8] and g.get_elem_width() == 16
    assert g.get_element_ty().is_f16() and g.get_layout_map().is_identity()
    assert int(F.MemorySpace.GLOBAL) == 1 and int(F.MemorySpace.SHARED) == 3 and int(F.MemorySpace.LOCAL) == 0
    assert F.GLOBAL == F.MemorySpace.GLOBAL  # exported values
    assert str(b.get_ranked_tensor_ty(f16, [2, 3])) == "tensor<2x3xf16>"
    assert str(b.get_function_ty([f16], [f16])) == "(f16) -> f16"


def _kernel_with_args(types):
    helper = F.create_session()
    kernel, entry = helper.new_kernel("k", types(helper))
    return helper, [entry.get_argument(i) for i in range(entry.get_num_arguments())]


def test_create_gemm_op_error_conventions():
    """ffi/ir.cpp:327-359: ValueError for non-memref operands, wrong rank, shape mismatch,
    mixed element types."""
    def tys(h):
        f16, f32 = h.builder.get_f16_ty(), h.builder.get_f32_ty()
        return [h.memref_type((8, 4), f16), h.memref_type((4, 16), f16), h.memref_type((8, 16), f16),
                h.memref_type((5, 16), f16), h.memref_type((8, 16), f32), h.memref_type((8,), f16),
                h.memref_type((8, 4), "e4m3fn"), h.memref_type((4, 16), "e4m3fn"),
                h.memref_type((8, 16), "bf16")]
    h, a = _kernel_with_args(tys)
    h.create_gemm(a[0], a[1], a[2])
    with pytest.raises(ValueError, match="inner dimensions"):
        h.create_gemm(a[0], a[3], a[2])
    with pytest.raises(ValueError, match="C shape"):
        h.create_gemm(a[0], a[1], a[3])
    with pytest.raises(ValueError, match="matching element types"):
        h.create_gemm(a[0], a[1], a[4])
    with pytest.raises(ValueError, match="rank-2"):
        h.create_gemm(a[5], a[1], a[2])
    with pytest.raises(ValueError, match="memref"):
        h.create_gemm(h.builder.get_f32(1.0), a[1], a[2])
    # extension: e4m3 inputs with a bf16 C (the reference cannot express an fp8 GEMM at all)
    g = h.create_gemm(a[6], a[7], a[8], trans_b=True)
    assert g.get_attrs()["transB"] is True and h.module.verify()


def test_gemm_scale_operands_extension():
    """Additive: an 8-bit float gemm may carry per-row / per-column fp32 scale vectors as a fourth
    and fifth operand; the reference's three-operand form prints exactly as before."""
    def tys(h):
        f32 = h.builder.get_f32_ty()
        return [h.memref_type((8, 4), "e4m3fn"), h.memref_type((4, 16), "e4m3fn"),
                h.memref_type((8, 16), "bf16"), h.memref_type((8,), f32), h.memref_type((16,), f32),
                h.memref_type((9,), f32), h.memref_type((8, 4), h.builder.get_f16_ty()),
                h.memref_type((4, 16), h.builder.get_f16_ty()), h.memref_type((8, 16), h.builder.get_f16_ty())]
    h, a = _kernel_with_args(tys)
    g = h.builder.create_gemm_op(a[0], a[1], a[2], False, True, True, a[3], a[4])
    assert g.get_scale_A().id() == a[3].id() and g.get_scale_B().id() == a[4].id()
    assert len(list(g.get_all_matrix())) == 3
    assert h.module.verify(), h.module.verify_message()
    text = str(h.module)
    assert "frisk.gemm(%arg0, %arg1, %arg2, %arg3, %arg4) {" in text
    assert text.rstrip().count("memref<8xf32, 1>, memref<16xf32, 1>") >= 1
    plain = h.builder.create_gemm_op(a[0], a[1], a[2])
    assert plain.get_scale_A() is None and plain.get_scale_B() is None
    with pytest.raises(ValueError, match="together"):
        h.builder.create_gemm_op(a[0], a[1], a[2], False, False, False, a[3])
    with pytest.raises(ValueError, match="matching length"):
        h.builder.create_gemm_op(a[0], a[1], a[2], False, False, False, a[5], a[4])
    with pytest.raises(ValueError, match="8-bit float"):
        h.builder.create_gemm_op(a[6], a[7], a[8], False, False, False, a[3], a[4])


def test_other_builder_errors():
    ctx = F.context()
    b = F.builder(ctx)
    with pytest.raises(ValueError):
        b.create_alloc_buffer_op([4], "int7")
    with pytest.raises(ValueError):
        b.create_alloc_buffer_op([4], "fp16", F.MemorySpace.SHARED, -8)
    with pytest.raises(ValueError):
        b.get_float_attr(1.0, "fp128")
    h = F.create_session()
    f16 = h.builder.get_f16_ty()
    _, entry = h.new_kernel("k", [h.memref_type((4, 4), f16), h.memref_type((4, 4), f16)])
    a0, a1 = entry.get_argument(0), entry.get_argument(1)
    with pytest.raises(IndexError):
        entry.arg(2)
    d0 = h.builder.get_affine_dim_expr(0)
    one_map = F.AffineMap.get(1, 0, [d0], h.context)
    with pytest.raises(ValueError):  # one map without the other (the reference aborts here)
        h.builder.create_copy_op(a0, a1, [], [], one_map)
    op = h.builder.create_alloc_buffer_op([4, 4], "bf16", F.MemorySpace.LOCAL)
    assert op.get_num_results() == 1
    with pytest.raises(IndexError):
        F.OpState.get_result(op, 1)
    with pytest.raises(IndexError):
        F.OpState.get_region(op, 0)


def test_verifiers_reject_what_the_reference_rejects():
    h = F.create_session()
    f16, f32 = h.builder.get_f16_ty(), h.builder.get_f32_ty()
    _, entry = h.new_kernel("k", [h.memref_type((8, 4), f16), h.memref_type((8,), f16),
                                  h.memref_type((4,), f16)])
    src, dst_ok, dst_bad = (entry.get_argument(i) for i in range(3))
    h.builder.create_reduce_op(src, dst_ok, "max", 1)
    assert h.module.verify()
    h.builder.create_reduce_op(src, dst_bad, "max", 1)
    assert not h.module.verify() and "non-reduced dimension" in h.module.verify_message()
    h2 = F.create_session()
    _, e2 = h2.new_kernel("k", [h2.memref_type((8, 4), f16)])
    h2.builder.create_fill_op(e2.get_argument(0), 1.0, "fp32")  # value type != element type
    assert not h2.module.verify()
    h3 = F.create_session()
    _, e3 = h3.new_kernel("k", [h3.memref_type((8, 4), f16)])
    h3.builder.create_reduce_op(e3.get_argument(0), e3.get_argument(0), "median", 0)
    assert not h3.module.verify()


def test_sibling_regions_reuse_ssa_numbers_like_mlir():
    h = F.create_session()
    f16 = h.builder.get_f16_ty()
    _, entry = h.new_kernel("k", [h.memref_type((4, 4), f16)])
    names = []
    for _ in range(2):
        h.builder.create_for_op(0, 4, 2, lambda b, iv: names.append(str(iv)))
    text = str(h.module)
    assert text.count("frisk.for %arg1 = 0 to 4 step = 2 {") == 2
    assert names == ["%arg1", "%arg1"]


def test_constants_and_functions_print():
    ctx = F.context()
    b = F.builder(ctx)
    mod = b.create_module()
    fty = b.get_function_ty([b.get_f32_ty()], [b.get_f32_ty()])
    fn = b.get_or_insert_function(mod, "f", fty)
    mod.push_back(fn)
    entry = fn.add_entry_block()
    b.set_insertion_point_to_start(entry)
    c = b.get_int64(5)
    x = b.get_f32(1.5)
    b.ret([fn.arg(0)])
    assert mod.has_function("f") and mod.get_function("f").get_num_arguments() == 1
    text = str(mod)
    assert "func.func @f(%arg0: f32) -> f32 {" in text
    assert "%c5_i64 = arith.constant 5 : i64" in text
    assert "%cst = arith.constant 1.500000e+00 : f32" in text
    assert "return %arg0 : f32" in text
    assert str(c) == "%c5_i64" and str(x) == "%cst"
    assert c.get_defining_op().is_constant_op()
    t = b.get_f32_tensor([2.0, 2.0], [2])
    assert t.get_defining_op().to_constant_op().get_splat_float_value() == 2.0


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "test", "python")),
                    reason="the reference checkout is not on this machine")
@pytest.mark.parametrize("script", ["bind_test.py", "helper_test.py", "map_expr_test.py"])
def test_reference_scripts_run_unmodified(script):
    env = dict(os.environ, PYTHONPATH=os.path.dirname(HERE))
    out = subprocess.run([sys.executable, os.path.join(REFERENCE, "test", "python", script)],
                         capture_output=True, text=True, env=env, timeout=120)
    assert out.returncode == 0, out.stderr
    if script == "bind_test.py":
        want = open(os.path.join(GOLDEN, "bind_test_module.mlir")).read().rstrip("\n")
        assert out.stdout.rstrip("\n") == want
