"""Session helpers with the names and signatures of the reference's python/frisk/common/utils.py
(create_context / create_session at :18-35, FriskHelper at :38-163), on top of the MLIR-free
``frisk_ffi`` module.  ``bf16`` is accepted wherever the reference takes a dtype string."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple, Union

from ..frisk_ffi import ir

DTypeLike = Union[str, "ir.type"]
ShapeLike = Sequence[int]

__all__ = ["create_context", "create_session", "FriskHelper"]

_TYPE_GETTERS = {
    "fp16": "get_f16_ty", "bf16": "get_bf16_ty", "fp32": "get_f32_ty", "fp64": "get_f64_ty",
    "int64": "get_int64_ty", "e4m3fn": "get_f8e4m3fn_ty", "e5m2": "get_f8e5m2_ty",
}


def create_context(*, load_dialects: bool = True, disable_multithreading: bool = True):
    """A context with the frisk dialect registered (single-threaded by default, as upstream)."""
    ctx = ir.context()
    if disable_multithreading:
        ctx.disable_multithreading()
    if load_dialects:
        ir.frisk.load_dialects(ctx)
    return ctx


def create_session(*, load_dialects: bool = True, disable_multithreading: bool = True) -> "FriskHelper":
    return FriskHelper.create(load_dialects=load_dialects,
                              disable_multithreading=disable_multithreading)


@dataclass
class FriskHelper:
    """Context + builder + module in one object, with shorthands for the common ops."""

    context: "ir.context"
    builder: "ir.builder"
    module: "ir.module"

    @classmethod
    def create(cls, *, load_dialects: bool = True, disable_multithreading: bool = True) -> "FriskHelper":
        ctx = create_context(load_dialects=load_dialects,
                             disable_multithreading=disable_multithreading)
        builder = ir.builder(ctx)
        module = builder.create_module()
        module.context = ctx  # harmless here (handles keep the context alive), kept for parity
        return cls(ctx, builder, module)

    # -- types ---------------------------------------------------------------------------
    def memref_type(self, shape: ShapeLike, dtype: DTypeLike = "fp16", *,
                    space=ir.MemorySpace.GLOBAL, layout: Optional["ir.AffineMap"] = None):
        element = self._as_type(dtype)
        amap = layout if layout is not None else ir.AffineMap()
        return self.builder.get_memref_ty(element, [int(d) for d in shape], amap, space)

    # -- ops -----------------------------------------------------------------------------
    def new_kernel(self, name: str, arg_types: Sequence["ir.type"]) -> Tuple["ir.KernelOp", "ir.block"]:
        kernel_type = self.builder.get_kernel_ty(list(arg_types))
        kernel = self.builder.create_kernel_op(self.module, name, kernel_type)
        self.module.push_back(kernel)
        entry = kernel.add_entry_block()
        self.builder.set_insertion_point_to_start(entry)
        return kernel, entry

    def alloc_buffer(self, shape: ShapeLike, dtype: DTypeLike = "fp16", *,
                     space=ir.MemorySpace.LOCAL, alignment: int = 0):
        op = self.builder.create_alloc_buffer_op(list(shape), self._as_dtype_str(dtype), space, alignment)
        return ir.OpState.get_result(op, 0)

    def create_gemm(self, A, B, C, *, trans_a: bool = False, trans_b: bool = False,
                    clear_accum: bool = False):
        return self.builder.create_gemm_op(A, B, C, trans_a, trans_b, clear_accum)

    # -- conveniences ----------------------------------------------------------------------
    def ensure_insertion_block(self):
        block = self.builder.get_insertion_block()
        if block is not None:
            return block
        new_block = self.builder.new_block()
        self.module.get_region(0).push_back(new_block)
        self.builder.set_insertion_point_to_start(new_block)
        return new_block

    def dump(self, msg: Optional[str] = None) -> None:
        if msg:
            print(msg)
        print(self.module)

    # -- internals -------------------------------------------------------------------------
    def _as_type(self, dtype: DTypeLike):
        if isinstance(dtype, ir.type):
            return dtype
        getter = _TYPE_GETTERS.get(dtype.lower())
        if getter is None:
            raise ValueError(f"Unsupported dtype '{dtype}'.")
        return getattr(self.builder, getter)()

    def _as_dtype_str(self, dtype: DTypeLike) -> str:
        if isinstance(dtype, str):
            return dtype
        for name, test in (("fp16", "is_f16"), ("bf16", "is_bf16"), ("fp32", "is_f32"), ("fp64", "is_f64")):
            if getattr(dtype, test)():
                return name
        raise ValueError("Unsupported MLIR type for allocation helper.")
