"""The textual form read back: modules printed by the reference itself (fixtures made from its
logs tmp/log_11_18 and tmp/log_12_18 by tests/golden/make_golden.py) and by this package parse to
modules that print to the same text, verify, and execute."""
import json
import os

import numpy as np
import pytest

import frisk as F
from frisk_b200 import runtime as R, workloads as W
from tile_programs import build_tiled_matmul

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def reference_texts():
    out = [("bind_test", open(os.path.join(GOLDEN, "bind_test_module.mlir")).read())]
    for case in json.load(open(os.path.join(GOLDEN, "layouts.json")))["cases"]:
        out.append((case["name"], case["module"]))
    return out


@pytest.mark.parametrize("name,text", reference_texts(), ids=[n for n, _ in reference_texts()])
def test_modules_printed_by_the_reference_round_trip(name, text):
    m = F.parse_module(text)
    assert str(m).strip() == text.strip()
    assert m.verify(), m.verify_message()


def test_reference_flagship_text_yields_its_gemm():
    text = open(os.path.join(GOLDEN, "bind_test_module.mlir")).read()
    _reduce, call = F.find_gemms(F.parse_module(text), "test_gemm")
    assert (call.M, call.N, call.K, call.ab_type) == (4096, 4096, 4096, W.F16)
    assert (call.arg_a, call.arg_b, call.arg_c) == (0, 1, 2) and not call.clear_accum


@pytest.mark.parametrize("kw", [
    dict(dims=(1024, 1024, 1024), tile=(128, 128, 32)),
    dict(dims=(512, 768, 256), tile=(64, 128, 32), dtype="bf16", accumulate=True, kstep=4),
])
def test_tiled_program_text_round_trips_and_lifts(kw):
    m = build_tiled_matmul(*kw["dims"], *kw["tile"], **{k: v for k, v in kw.items() if k not in ("dims", "tile")})
    text = str(m)
    back = F.parse_module(text)
    assert str(back) == text and back.verify()
    assert F.find_gemms(back, "matmul") == F.find_gemms(m, "matmul")


def test_other_constructs_round_trip():
    text = """module attributes {frisk.target = "sm_100a"} {
  frisk.kernel @k(memref<8x4xf8E4M3FN, 1>, memref<4x16xf8E4M3FN, 1>, memref<8x16xbf16, 1>, memref<8xf32, 1>, memref<16xf32, 1>, memref<16x8xf16, affine_map<(d0, d1) -> (d1, d0)>, 1>) {
    frisk.gemm(%arg0, %arg1, %arg2, %arg3, %arg4) {K = 4 : i64, M = 8 : i64, N = 16 : i64, clear_accum = true, policy = #frisk<gemm_warp_policy Square>, transA = false, transB = true} : memref<8x4xf8E4M3FN, 1>, memref<4x16xf8E4M3FN, 1>, memref<8x16xbf16, 1>, memref<8xf32, 1>, memref<16xf32, 1>
    frisk.for %arg6 = 2 to 10 step = 2 {
      frisk.block (%arg7) to (16) {
        %0 = frisk.alloc_buffer {scope = "shared", alignment = 128} -> memref<4x4xbf16, 3>
        frisk.copy %arg2[%arg6 floordiv 2, (%arg7 mod 4) * 4 + symbol(%arg6)], %0[0, 0] {src_extents = [4, 4], dst_extents = [4, 4]}  : memref<8x16xbf16, 1>, memref<4x4xbf16, 3>
        frisk.fill %0 {value = -1.500000e+00 : bf16} : memref<4x4xbf16, 3>
      }
    }
    frisk.reduce %arg2, %arg4 {clear = false, dim = 0 : i64, kind = "sum"} : memref<8x16xbf16, 1>, memref<16xf32, 1>
  }
}"""
    m = F.parse_module(text)
    assert str(m).strip() == text
    call, red = F.find_gemms(m, "k")
    assert (call.arg_scale_a, call.arg_scale_b, call.transB, call.clear_accum) == (3, 4, True, True)
    assert (red.kind, red.dim, red.clear, red.arg_src, red.arg_dst) == ("sum", 0, False, 2, 4)
    assert not m.verify()  # "sum" is not a reduce kind and the element types differ: run() would refuse


@pytest.mark.parametrize("text,what", [
    ("module {\n  frisk.kernel @k(memref<4x4xf16, 1>) {\n    frisk.fill %arg1 {value = 0.000000e+00 : f16} : memref<4x4xf16, 1>\n  }\n}",
     r"line 3, column \d+: use of undefined value %arg1"),
    ("module {\n  frisk.kernel @k(memref<4x4xq16, 1>) {\n  }\n}", r"line 2, .*unknown type 'q16'"),
    ("module {\n  frisk.kernel @k(memref<4x4xf16, 1>) {\n    frisk.fill %arg0 {value = 0.000000e+00 : f16} : memref<4x8xf16, 1>\n  }\n}",
     "operand types do not match"),
    ("module {\n  frisk.kernel @k() {\n    frisk.softmax\n  }\n}", "operation 'frisk.softmax' is not read back"),
    ("module {\n  frisk.kernel @k() {\n  }\n} trailing", "text after the module"),
    ("module {\n  frisk.kernel @k() {\n", "expected"),
])
def test_unreadable_text_is_refused_with_line_and_column(text, what):
    with pytest.raises(ValueError, match=what):
        F.parse_module(text)


@pytest.mark.gpu
def test_module_text_executes():
    from oracle import ref
    # a whole-problem gemm written as text, the way the reference prints one
    w = W.make_workload("cfg2", 256, 384, 192)
    text = f"""module {{
  frisk.kernel @k(memref<256x192xf16, 1>, memref<192x384xf16, 1>, memref<256x384xf16, 1>) {{
    frisk.gemm(%arg0, %arg1, %arg2) {{K = 192 : i64, M = 256 : i64, N = 384 : i64, clear_accum = true, policy = #frisk<gemm_warp_policy Square>, transA = false, transB = true}} : memref<256x192xf16, 1>, memref<192x384xf16, 1>, memref<256x384xf16, 1>
  }}
}}"""
    out = np.zeros((w.M, w.N), np.float16)
    F.run(text, "k", [w.A, w.B, out])
    assert np.array_equal(out.view(np.uint16), R.gemm_host(w).view(np.uint16))
    ok, err, _ = W.check(out.astype(np.float32), ref.ref_gemm_f64(w), W.F16, absdot=ref.abs_dot(w))
    assert ok, err
    # the tiled program, through its text
    m = build_tiled_matmul(512, 512, 256, 128, 128, 32, dtype="bf16")
    rng = np.random.default_rng(3)
    A = W.encode(rng.standard_normal((512, 256)).astype(np.float32), W.BF16)
    B = W.encode(rng.standard_normal((256, 512)).astype(np.float32) * 0.05, W.BF16)
    C = np.zeros((512, 512), np.uint16)
    F.run(str(m), "matmul", [A, B, C])
    wl = W.GemmWorkload("text", 512, 512, 256, W.BF16, W.BF16, A=A, B=B)
    assert np.array_equal(C, R.gemm_host(wl))
