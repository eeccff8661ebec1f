"""Running the ``frisk.gemm`` and ``frisk.reduce`` ops of a module: the step the reference stops
short of.

Four forms are executed, all through libfrisk_b200 on the buffers bound to the kernel arguments:

* a ``frisk.reduce`` whose source and destination are kernel arguments in the GLOBAL memory space:
  one whole-buffer reduce per op, in program order with the gemms (so a gemm followed by a row
  maximum of its result runs as written);

* a ``frisk.gemm`` whose operands are kernel arguments in the GLOBAL memory space (what the
  reference's flagship script emits: test/python/bind_test.py:53, captured in tmp/log_11_18:12):
  one whole-problem GEMM per op;
* the tiled matrix product the reference sketches in tmp/ir.mlir:1-17 -- a ``frisk.parallel`` grid
  whose body allocates tiles, clears (or loads) the accumulator tile, runs a ``frisk.for`` over K of
  two ``frisk.copy`` and a ``frisk.gemm`` on the tiles, and copies the accumulator out.  The
  program is checked to be exactly that product (``frisk_ffi.ir.frisk.lift_tiled_gemm``) and run as
  ONE GEMM over the kernel's arguments: tile sizes, staging and grid are the B200 back end's own
  choice, so the copy / fill / for / parallel ops are recognised, not interpreted one by one;
* the tile-by-tile fold of a matrix -- a one-dimensional ``frisk.parallel`` grid whose body walks a
  row (or column) block of a GLOBAL argument in tiles, ``frisk.reduce``-ing each tile into a
  rank-1 accumulator buffer, as the reference's online-softmax sketch does for its row maximum
  (tmp/ir.mlir:22-36) -- recognised the same way (``lift_tiled_reduce``) and run as ONE
  whole-buffer reduce.

A gemm or reduce on anything but kernel arguments, outside those two tile programs, is refused
with the reason; there is no CPU path.

Only ``frisk.gemm`` and ``frisk.reduce`` are executed, each once, in program order.  The loops,
blocks, fills and copies that the reference's flagship script wraps around its whole-problem gemm
(test/python/bind_test.py:29-53: the gemm sits inside parallel / for / block ops and next to a fill
and a copy of the same kernel arguments) are builder exercises, not a meaning this back end could
execute; they are not run.  A ``frisk.fill`` or ``frisk.copy`` that touches a kernel argument is
therefore reported: ``run`` raises a ``FriskWarning`` naming every such op (``SKIPPED`` lists them),
so that a program which relies on, say, clearing C with a fill before an accumulating gemm does not
go wrong silently -- fill or copy the bound buffers on the host instead.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import runtime as R
from . import workloads as W
from .frisk_ffi import ir


@dataclass
class GemmCall:
    M: int
    N: int
    K: int
    ab_type: int
    c_type: int
    transA: bool
    transB: bool
    clear_accum: bool
    arg_a: int  # kernel argument indices of A, B, C
    arg_b: int
    arg_c: int
    arg_scale_a: Optional[int] = None  # ... and of the scale vectors of an 8-bit float gemm
    arg_scale_b: Optional[int] = None


@dataclass
class ReduceCall:
    shape: tuple
    dim: int
    dtype: int
    kind: str
    clear: bool
    arg_src: int
    arg_dst: int


class FriskWarning(UserWarning):
    """An op of the kernel that touches a kernel argument was not executed."""


# fills and copies of kernel arguments the last `find_gemms` walked past: (op name, argument indices)
SKIPPED: List[tuple] = []


def _dtype_of(ty) -> int:
    s = str(ty)
    table = {"f32": W.F32, "f16": W.F16, "bf16": W.BF16, "f8E4M3FN": W.E4M3, "f8E5M2": W.E5M2}
    if s not in table:
        raise R.FriskError(-2, f"element type {s} has no GEMM kernel")
    return table[s]


def find_gemms(module, kernel_name: str) -> list:
    """The executable ops of the kernel in program order: GemmCall and ReduceCall records."""
    kernel = module.get_kernel(kernel_name)
    if kernel is None:
        raise KeyError(f"no frisk.kernel named {kernel_name!r} in the module")
    args = {kernel.arg(i).id(): i for i in range(kernel.get_num_arguments())}
    calls: list = []
    del SKIPPED[:]

    def visit(op):
        if op.get_name() in ("frisk.fill", "frisk.copy"):
            touched = [args[v.id()] for v in (op.get_operand(i) for i in range(op.get_num_operands()))
                       if v.id() in args]
            if touched:
                SKIPPED.append((op.get_name(), tuple(touched)))
            return
        r = op.to_reduce_op()
        if r is not None:
            src, dst = r.get_src_memref(), r.get_dst_memref()
            for name, v in (("source", src), ("destination", dst)):
                if v.id() not in args or v.get_type().get_memory_space() != ir.MemorySpace.GLOBAL:
                    raise R.FriskError(-2, f"frisk.reduce {name} is not a kernel argument in GLOBAL memory: "
                                           "only whole-buffer reduces are executed")
            ty = src.get_type()
            dtype = _dtype_of(ty.get_element_ty())
            if dtype in (W.E4M3, W.E5M2):
                raise R.FriskError(-2, "frisk.reduce has no kernel for 8-bit floats")
            calls.append(ReduceCall(tuple(ty.get_shape()), r.get_reduce_dim(), dtype, r.get_kind(),
                                    r.get_clear(), args[src.id()], args[dst.id()]))
            return
        g = op.to_gemm_op()
        if g is None:
            return
        vals = [g.get_matrix_A(), g.get_matrix_B(), g.get_matrix_C()]
        idx = []
        for name, v in zip("ABC", vals):
            if v.id() not in args:
                raise R.FriskError(-2, f"frisk.gemm operand {name} is not a kernel argument: only "
                                       "whole-problem GEMMs on global buffers are executed")
            space = v.get_type().get_memory_space()
            if space != ir.MemorySpace.GLOBAL:
                raise R.FriskError(-2, f"frisk.gemm operand {name} must live in GLOBAL memory")
            idx.append(args[v.id()])
        for name, v in (("scale_a", g.get_scale_A()), ("scale_b", g.get_scale_B())):
            if v is None:
                idx.append(None)
            elif v.id() not in args:
                raise R.FriskError(-2, f"frisk.gemm operand {name} is not a kernel argument")
            else:
                idx.append(args[v.id()])
        a = g.get_attrs()
        ta, tc = vals[0].get_type(), vals[2].get_type()
        calls.append(GemmCall(a["M"], a["N"], a["K"], _dtype_of(ta.get_element_ty()),
                              _dtype_of(tc.get_element_ty()), a["transA"], a["transB"],
                              a["clear_accum"], *idx))

    try:
        kernel.get_region(0).front().walk(visit)
    except R.FriskError as whole_problem_error:
        # not whole-problem gemms on kernel arguments: the kernel has to be the tiled product
        try:
            t = ir.frisk.lift_tiled_gemm(kernel)
        except ValueError as e:
            # ... or the tile-by-tile fold of a matrix (no gemm in it)
            try:
                r = ir.frisk.lift_tiled_reduce(kernel)
            except ValueError as e2:
                raise R.FriskError(-2, f"{whole_problem_error}; and the kernel is {e}; and {e2}") from None
            del SKIPPED[:]
            return [ReduceCall(tuple(r["shape"]), r["dim"], _dtype_of(r["type"]), r["kind"], r["clear"],
                               r["arg_src"], r["arg_dst"])]
        del SKIPPED[:]   # in a lifted tile program the copies ARE the program
        lifted = [GemmCall(t["M"], t["N"], t["K"], _dtype_of(t["ab_type"]), _dtype_of(t["c_type"]),
                           False, False, t["clear_accum"], t["arg_a"], t["arg_b"], t["arg_c"])]
        if "arg_r" in t:  # the tile program folds the accumulator's rows: a reduce of C behind the gemm
            lifted.append(ReduceCall((t["M"], t["N"]), 1, _dtype_of(t["c_type"]), t["reduce_kind"],
                                     t["reduce_clear"], t["arg_c"], t["arg_r"]))
        return lifted
    return calls


# What the last `run` launched, in order: ("gemm" | "gemm+reduce" | "reduce", kernel family).
LAST_RUN: List[tuple] = []


def parse_module(text: str):
    """Reads a module from its textual form (``str(module)``, a ``.mlir`` file written by this
    package or printed by the reference) into a fresh context; ``ValueError`` names line and
    column of what cannot be read."""
    ctx = ir.context()
    ir.frisk.load_dialects(ctx)
    module = ir.frisk.parse_module(text, ctx)
    module.context = ctx
    return module


def run(module, kernel_name: str, buffers: Sequence[np.ndarray], *, scale_a: Optional[np.ndarray] = None,
        scale_b: Optional[np.ndarray] = None, plan_options: Optional[Dict] = None) -> None:
    """Executes every ``frisk.gemm`` and ``frisk.reduce`` of the kernel (a module, or its text) on host buffers (one per kernel argument, raw
    storage bits in the memory order the op's trans flags state).  C buffers are updated in
    place.  Raises when the CUDA library or a device is missing: there is no CPU path."""
    if isinstance(module, str):  # the textual form
        module = parse_module(module)
    if not module.verify():
        raise R.FriskError(-1, "module does not verify: " + module.verify_message())
    del LAST_RUN[:]
    calls = find_gemms(module, kernel_name)
    if SKIPPED:
        what = ", ".join(f"{name} of argument{'s' if len(a) > 1 else ''} {', '.join(map(str, a))}" for name, a in SKIPPED)
        warnings.warn(f"not executed (only frisk.gemm and frisk.reduce run): {what}", FriskWarning, stacklevel=2)
    skip = set()
    for i, call in enumerate(calls):
        if i in skip:
            continue
        if isinstance(call, ReduceCall):
            src = np.ascontiguousarray(buffers[call.arg_src])
            dst = buffers[call.arg_dst]
            if not dst.flags["C_CONTIGUOUS"]:
                raise ValueError("the destination buffer must be C-contiguous (it is written in place)")
            if tuple(src.shape) != call.shape:
                raise ValueError(f"the source buffer has shape {tuple(src.shape)}, the op says {call.shape}")
            R.reduce_host(src, dst, call.dim, call.dtype, call.kind, call.clear)
            LAST_RUN.append(("reduce", "reduce"))
            continue
        sa, sb = scale_a, scale_b
        if sa is None and call.arg_scale_a is not None:  # scale vectors bound as kernel arguments
            sa = np.ascontiguousarray(buffers[call.arg_scale_a], dtype=np.float32)
            sb = np.ascontiguousarray(buffers[call.arg_scale_b], dtype=np.float32)
        kw = dict(transA=call.transA, transB=call.transB, clear_accum=call.clear_accum,
                  scales=sa is not None, **(plan_options or {}))
        # A frisk.reduce over the columns of the C this gemm has just written (the row maximum /
        # row sum after the first gemm of the reference's attention sketch, tmp/ir.mlir:112-135)
        # runs inside the gemm's epilogue, when a whole-tile tensor-core plan exists for it.
        plan, fused = None, None
        nxt = calls[i + 1] if i + 1 < len(calls) else None
        if (isinstance(nxt, ReduceCall) and nxt.arg_src == call.arg_c and nxt.dim == 1
                and nxt.shape == (call.M, call.N) and nxt.dtype == call.c_type
                and nxt.arg_dst not in (call.arg_a, call.arg_b, call.arg_c)):
            try:
                plan = R.GemmPlan(call.M, call.N, call.K, call.ab_type, call.c_type,
                                  row_reduce=nxt.kind, row_reduce_clear=nxt.clear, **kw)
                fused = nxt
                skip.add(i + 1)
            except R.FriskError as e:
                if e.code != -2:
                    raise
        if plan is None:
            plan = R.GemmPlan(call.M, call.N, call.K, call.ab_type, call.c_type, **kw)
        try:
            a = np.ascontiguousarray(buffers[call.arg_a])
            b = np.ascontiguousarray(buffers[call.arg_b])
            c = buffers[call.arg_c]
            if not c.flags["C_CONTIGUOUS"]:
                raise ValueError("the C buffer must be C-contiguous (it is written in place)")
            dst = None
            if fused is not None:
                dst = buffers[fused.arg_dst]
                if not dst.flags["C_CONTIGUOUS"] or dst.size != call.M:
                    raise ValueError("the reduce destination must be a C-contiguous buffer of M elements")
            plan.run_host(a, b, c, sa, sb, dst)
            LAST_RUN.append(("gemm+reduce" if fused else "gemm", plan.info["kernel_name"]))
        finally:
            plan.close()
