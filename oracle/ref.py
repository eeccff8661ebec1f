"""Python face of the CPU oracle (oracle/frisk_ref_gemm.c).  TEST INFRASTRUCTURE ONLY.

PARITY UNPINNED for numerics: the reference has no GEMM arithmetic to compare with (see the
header of frisk_ref_gemm.c).  The storage codecs are pinned against numpy / ml_dtypes / torch in
tests/test_oracle.py, and the C loop against an independent numpy float64 product.

Only tests/, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` import this.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Optional

import numpy as np

from frisk_b200 import workloads as W

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_build", "libfrisk_ref.so")


class RefDesc(C.Structure):
    _fields_ = [
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("ab_type", C.c_int32), ("c_type", C.c_int32),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
        ("transA", C.c_int32), ("transB", C.c_int32), ("clear_accum", C.c_int32),
        ("use_scales", C.c_int32), ("acc64", C.c_int32),
    ]


def build(force: bool = False) -> str:
    """Compiles the C restatement with the Makefile beside it."""
    src = os.path.join(_HERE, "frisk_ref_gemm.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "clean", "all"])
    return LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        L = C.CDLL(LIB_PATH)
        vp = C.c_void_p
        L.frisk_ref_gemm_rows.argtypes = [C.POINTER(RefDesc), vp, vp, vp, vp, vp, C.c_int64,
                                          C.c_int64, C.c_int]
        L.frisk_ref_gemm_rows.restype = C.c_int
        L.frisk_ref_max_threads.restype = C.c_int
        for name, arg, res in (("frisk_ref_decode_f16", C.c_uint16, C.c_float),
                               ("frisk_ref_decode_bf16", C.c_uint16, C.c_float),
                               ("frisk_ref_decode_e4m3", C.c_uint8, C.c_float),
                               ("frisk_ref_decode_e5m2", C.c_uint8, C.c_float),
                               ("frisk_ref_encode_bf16", C.c_float, C.c_uint16),
                               ("frisk_ref_encode_f16", C.c_float, C.c_uint16)):
            f = getattr(L, name)
            f.argtypes = [arg]
            f.restype = res
        _lib = L
    return _lib


def max_threads() -> int:
    return int(lib().frisk_ref_max_threads())


def ref_gemm(w: W.GemmWorkload, rows: Optional[tuple[int, int]] = None, acc64: bool = False,
             num_threads: int = 0, out: Optional[np.ndarray] = None) -> np.ndarray:
    """Oracle result for a workload as raw storage bits of C ([M, N]; only `rows` are filled)."""
    d = RefDesc()
    d.M, d.N, d.K = w.M, w.N, w.K
    d.ab_type, d.c_type = w.ab_type, w.c_type
    d.lda = w.M if w.transA else w.K
    d.ldb = w.K if w.transB else w.N
    d.ldc = w.N
    d.transA, d.transB = int(w.transA), int(w.transB)
    d.clear_accum = int(w.clear_accum)
    d.use_scales = int(w.scale_a is not None)
    d.acc64 = int(acc64)
    if out is None:
        out = np.zeros((w.M, w.N), dtype=W.storage_numpy_dtype(w.c_type))
        if not w.clear_accum and w.C0 is not None:
            out[...] = w.C0
    a = np.ascontiguousarray(w.A)
    b = np.ascontiguousarray(w.B)
    sa = None if w.scale_a is None else np.ascontiguousarray(w.scale_a, dtype=np.float32)
    sb = None if w.scale_b is None else np.ascontiguousarray(w.scale_b, dtype=np.float32)
    m0, m1 = rows if rows is not None else (0, w.M)
    rc = lib().frisk_ref_gemm_rows(C.byref(d), a.ctypes.data, b.ctypes.data, out.ctypes.data,
                                   None if sa is None else sa.ctypes.data,
                                   None if sb is None else sb.ctypes.data, m0, m1, num_threads)
    if rc != 0:
        raise ValueError("frisk_ref_gemm_rows rejected its arguments")
    return out


def ref_gemm_f64(w: W.GemmWorkload, rows: Optional[np.ndarray] = None) -> np.ndarray:
    """Independent numpy float64 product on the decoded inputs (no final cast)."""
    a = w.a_logical().astype(np.float64)
    b = w.b_logical().astype(np.float64)
    if rows is not None:
        a = a[rows]
    c = a @ b
    if w.scale_a is not None:
        sa = w.scale_a.astype(np.float64)
        c = c * (sa[rows] if rows is not None else sa)[:, None] * w.scale_b.astype(np.float64)[None, :]
    if not w.clear_accum and w.C0 is not None:
        c0 = W.decode(w.C0, w.c_type).astype(np.float64)
        c = c + (c0[rows] if rows is not None else c0)
    return c


def abs_dot(w: W.GemmWorkload, rows: Optional[np.ndarray] = None) -> np.ndarray:
    """sum_k |A[m,k]| |B[k,n]| (times |scales|): the magnitude of the data behind each output,
    used as the floor of the relative-error metric."""
    a = np.abs(w.a_logical().astype(np.float64))
    b = np.abs(w.b_logical().astype(np.float64))
    if rows is not None:
        a = a[rows]
    s = a @ b
    if w.scale_a is not None:
        sa = np.abs(w.scale_a.astype(np.float64))
        s = s * (sa[rows] if rows is not None else sa)[:, None] * np.abs(w.scale_b.astype(np.float64))[None, :]
    if not w.clear_accum and w.C0 is not None:
        c0 = np.abs(W.decode(w.C0, w.c_type).astype(np.float64))
        s = s + (c0[rows] if rows is not None else c0)
    return s


def ref_reduce(src: np.ndarray, dim: int, dtype: int, kind: str, clear: bool = True,
               dst0: Optional[np.ndarray] = None) -> tuple[np.ndarray, np.ndarray]:
    """``frisk.reduce`` restated (op: include/Dialect/Frisk/IR/FriskOps.td:413-443; shape and kind
    rules: lib/Dialect/Frisk/IR/FriskOps.cpp:1734-1767): dst = (clear ? identity : dst) (op) the
    fold of `src` (raw storage bits) over `dim`, computed in float64 on the exactly decoded
    elements.  Returns (result as float64 without the final cast, sum of magnitudes folded --
    the scale an error of a sum is measured against).  min / max skip NaN like fminf / fmaxf
    folded from the identity.
    PARITY UNPINNED: the reference never executes this op and holds no expected values for it."""
    x = W.decode(np.asarray(src), dtype).astype(np.float64)
    fold = {"add": np.add, "mul": np.multiply, "min": np.fmin, "max": np.fmax}[kind]
    ident = {"add": 0.0, "mul": 1.0, "min": np.inf, "max": -np.inf}[kind]
    out = fold.reduce(x, axis=dim, initial=ident)
    mag = np.abs(x).sum(axis=dim) if kind == "add" else np.abs(out)
    if not clear:
        d0 = W.decode(np.asarray(dst0), dtype).astype(np.float64).reshape(out.shape)
        out = fold(d0, out)
        mag = mag + np.abs(d0) if kind == "add" else np.abs(out)
    return out, mag
