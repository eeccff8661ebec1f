"""ctypes binding of libfrisk_b200.so -- the execution side of ``frisk.gemm``.

The reference's Python surface can only build and print IR (its ``create_gemm_op`` is at
ffi/ir.cpp:322-366; nothing below it executes).  This module is the part a user calls to run the
op: ``plan`` turns a GEMM description (or a ``frisk.gemm`` op found in a module) into a
``GemmPlan``; ``GemmPlan.run`` launches it on device pointers, ``GemmPlan.run_host`` on numpy
arrays.  There is no CPU fallback: when the shared library is missing every entry point raises.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import numpy as np

from . import workloads as W

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfrisk_b200.so")

KERNEL_NAMES = {0: "simt", 1: "tcgen05", 2: "skinny", 3: "tcgen05_pair", 4: "tf32x3"}


class FriskError(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = code
        super().__init__(what)


class GemmDesc(C.Structure):
    _fields_ = [
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("a_type", C.c_int32), ("b_type", C.c_int32), ("c_type", C.c_int32),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
        ("transA", C.c_int32), ("transB", C.c_int32),
        ("clear_accum", C.c_int32), ("scale_mode", C.c_int32),
        ("force_kernel", C.c_int32), ("tile_n", C.c_int32), ("stages", C.c_int32),
        ("num_ctas", C.c_int32), ("band_tiles", C.c_int32),
        ("epilogue", C.c_int32), ("row_reduce", C.c_int32), ("row_reduce_clear", C.c_int32),
        ("panel_tiles", C.c_int32), ("l2_hints", C.c_int32), ("k_split", C.c_int32),
    ]


class GemmRunArgs(C.Structure):
    _fields_ = [
        ("A", C.c_void_p), ("B", C.c_void_p), ("C", C.c_void_p),
        ("scale_a", C.c_void_p), ("scale_b", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("device_status", C.c_void_p), ("stream", C.c_void_p),
        ("row_reduce_dst", C.c_void_p), ("n_peers", C.c_int32), ("peer_c", C.c_void_p * 7),
    ]


class PlanInfo(C.Structure):
    _fields_ = [
        ("kernel", C.c_int32), ("tile_m", C.c_int32), ("tile_n", C.c_int32), ("tile_k", C.c_int32),
        ("stages", C.c_int32), ("num_ctas", C.c_int32), ("swap_ab", C.c_int32),
        ("split_k", C.c_int32), ("smem_bytes", C.c_int32), ("launches", C.c_int32),
        ("swizzle_a", C.c_int32), ("swizzle_b", C.c_int32),
        ("cuda_core_reason", C.c_int32), ("cuda_core_runs", C.c_int64),
    ]

    def as_dict(self) -> dict:
        d = {n: int(getattr(self, n)) for n, _ in self._fields_}
        d["kernel_name"] = KERNEL_NAMES.get(d["kernel"], "?")
        return d


class ReduceDesc(C.Structure):
    _fields_ = [("outer", C.c_int64), ("extent", C.c_int64), ("inner", C.c_int64), ("dtype", C.c_int32),
                ("kind", C.c_int32), ("clear", C.c_int32), ("device", C.c_int32)]


class ReduceInfo(C.Structure):
    _fields_ = [("lines", C.c_int32), ("vector", C.c_int32), ("chunks", C.c_int32), ("launches", C.c_int32),
                ("chunk_len", C.c_int64), ("ctas", C.c_int64), ("workspace_bytes", C.c_size_t)]

    def as_dict(self) -> dict:
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


REDUCE_KINDS = {"add": 0, "mul": 1, "min": 2, "max": 3}


class LayoutDesc(C.Structure):
    _fields_ = [("rows", C.c_int64), ("cols", C.c_int64), ("elem_bits", C.c_int32),
                ("k_inner", C.c_int32)]


class TmaParams(C.Structure):
    _fields_ = [
        ("swizzle_bytes", C.c_int32), ("box_inner", C.c_int32), ("box_outer", C.c_int32),
        ("num_boxes", C.c_int32), ("umma_layout_type", C.c_int32), ("umma_major", C.c_int32),
        ("leading_byte_offset", C.c_int32), ("stride_byte_offset", C.c_int32),
        ("k_step_bytes", C.c_int32), ("reference_layout", C.c_char * 24),
    ]

    def as_dict(self) -> dict:
        d = {n: getattr(self, n) for n, _ in self._fields_}
        d["reference_layout"] = d["reference_layout"].decode()
        return d


class BankStats(C.Structure):
    _fields_ = [("avg_max_conflict", C.c_double), ("max_conflict", C.c_int32),
                ("samples", C.c_int32)]


class AccessStats(C.Structure):
    _fields_ = [("requests", C.c_int64), ("wavefronts", C.c_int64), ("ideal_wavefronts", C.c_int64),
                ("conflict_degree", C.c_double), ("max_wavefronts_per_request", C.c_int32),
                ("tma_boxes", C.c_int32), ("global_segment_bytes", C.c_int32)]


ACCESS_CHUNK_COLUMN, ACCESS_ROW_PIECES = 1, 2
SWIZZLE_128B_ATOM_32B = 1032
SWIZZLE_128B_ATOM_64B = 1064

_lib = None


def lib() -> C.CDLL:
    """Loads libfrisk_b200.so (built in-tree by ``python -m frisk_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FriskError(-5, f"{LIB_PATH} is missing: build it with `python -m frisk_b200.build` "
                             "(there is no fallback path)")
    L = C.CDLL(LIB_PATH)
    vp, i32p = C.c_void_p, C.POINTER(C.c_int32)
    L.frisk_b200_gemm_plan_create.argtypes = [C.POINTER(GemmDesc), C.POINTER(vp)]
    L.frisk_b200_gemm_plan_create.restype = C.c_int
    L.frisk_b200_gemm_plan_destroy.argtypes = [vp]
    L.frisk_b200_gemm_plan_destroy.restype = None
    L.frisk_b200_gemm_plan_info.argtypes = [vp, C.POINTER(PlanInfo)]
    L.frisk_b200_gemm_plan_info.restype = C.c_int
    L.frisk_b200_gemm_workspace_bytes.argtypes = [vp, C.POINTER(C.c_size_t)]
    L.frisk_b200_gemm_workspace_bytes.restype = C.c_int
    L.frisk_b200_gemm_run.argtypes = [vp, vp, vp, vp, vp, vp, vp, C.c_size_t, vp, vp]
    L.frisk_b200_gemm_run.restype = C.c_int
    L.frisk_b200_gemm_run_ex.argtypes = [vp, C.POINTER(GemmRunArgs)]
    L.frisk_b200_gemm_run_ex.restype = C.c_int
    L.frisk_b200_peer_alloc.argtypes = [C.c_size_t, C.POINTER(vp), C.c_char_p]
    L.frisk_b200_peer_alloc.restype = C.c_int
    L.frisk_b200_peer_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    L.frisk_b200_peer_open.restype = C.c_int
    L.frisk_b200_peer_close.argtypes = [vp]
    L.frisk_b200_peer_close.restype = C.c_int
    L.frisk_b200_peer_free.argtypes = [vp]
    L.frisk_b200_peer_free.restype = C.c_int
    L.frisk_b200_gemm_run_host.argtypes = [vp, vp, vp, vp, vp, vp]
    L.frisk_b200_gemm_run_host.restype = C.c_int
    L.frisk_b200_gemm_run_host_ex.argtypes = [vp, vp, vp, vp, vp, vp, vp]
    L.frisk_b200_gemm_run_host_ex.restype = C.c_int
    L.frisk_b200_gemm_skinny_static.argtypes = [C.POINTER(GemmDesc), vp, vp, vp, vp, vp, vp, vp]
    L.frisk_b200_gemm_skinny_static.restype = C.c_int
    L.frisk_b200_gemm_skinny_static_capacity.argtypes = []
    L.frisk_b200_gemm_skinny_static_capacity.restype = C.c_size_t
    L.frisk_b200_check_status.argtypes = [vp, vp]
    L.frisk_b200_check_status.restype = C.c_int
    L.frisk_b200_strerror.argtypes = [C.c_int]
    L.frisk_b200_strerror.restype = C.c_char_p
    L.frisk_b200_last_error.argtypes = []
    L.frisk_b200_last_error.restype = C.c_char_p
    L.frisk_b200_shard_rows.argtypes = [C.c_int64, C.c_int, C.c_int, C.POINTER(C.c_int64),
                                        C.POINTER(C.c_int64)]
    L.frisk_b200_shard_rows.restype = C.c_int
    L.frisk_b200_layout_to_tma.argtypes = [C.POINTER(LayoutDesc), C.POINTER(TmaParams)]
    L.frisk_b200_layout_to_tma.restype = C.c_int
    L.frisk_b200_gemm_plan_operand_layout.argtypes = [vp, C.c_int32, C.POINTER(TmaParams),
                                                      C.POINTER(C.c_uint64), C.POINTER(C.c_int32)]
    L.frisk_b200_gemm_plan_operand_layout.restype = C.c_int
    L.frisk_b200_swizzled_offset.argtypes = [C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int32,
                                             C.c_int32]
    L.frisk_b200_swizzled_offset.restype = C.c_int64
    L.frisk_b200_bank_conflicts.argtypes = [C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int32,
                                            C.c_int32, C.POINTER(BankStats)]
    L.frisk_b200_bank_conflicts.restype = C.c_int
    L.frisk_b200_bank_conflicts_access.argtypes = [C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int32,
                                                   C.POINTER(AccessStats)]
    L.frisk_b200_bank_conflicts_access.restype = C.c_int
    L.frisk_b200_reduce_info.argtypes = [C.POINTER(ReduceDesc), C.c_int, C.POINTER(ReduceInfo)]
    L.frisk_b200_reduce_info.restype = C.c_int
    L.frisk_b200_reduce_workspace_bytes.argtypes = [C.POINTER(ReduceDesc), C.POINTER(C.c_size_t)]
    L.frisk_b200_reduce_workspace_bytes.restype = C.c_int
    L.frisk_b200_reduce_run.argtypes = [C.POINTER(ReduceDesc), vp, vp, vp, C.c_size_t, vp]
    L.frisk_b200_reduce_run.restype = C.c_int
    L.frisk_b200_reduce_run_host.argtypes = [C.POINTER(ReduceDesc), vp, vp]
    L.frisk_b200_reduce_run_host.restype = C.c_int
    L.frisk_b200_measure_mma_peak.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                              C.POINTER(C.c_double), C.POINTER(C.c_double)]
    L.frisk_b200_measure_mma_peak.restype = C.c_int
    L.frisk_b200_device_sm_count.argtypes = []
    L.frisk_b200_device_sm_count.restype = C.c_int
    L.frisk_b200_version.argtypes = []
    L.frisk_b200_version.restype = C.c_char_p
    _lib = L
    return L


def _check(rc: int, what: str) -> None:
    if rc != 0:
        L = lib()
        msg = L.frisk_b200_strerror(rc).decode()
        detail = L.frisk_b200_last_error().decode()
        raise FriskError(rc, f"{what}: {msg}" + (f" ({detail})" if detail and rc in (-5, -6) else ""))


def _ptr(x) -> Optional[int]:
    """Device or host address of a torch tensor / numpy array / int / None."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if isinstance(x, np.ndarray):
        return x.ctypes.data
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    raise TypeError(f"cannot take the address of {type(x)}")


class GemmPlan:
    """A planned ``frisk.gemm``.  See include/frisk_b200.h for the operand convention."""

    def __init__(self, M: int, N: int, K: int, ab_type: int, c_type: Optional[int] = None, *,
                 transA: bool = False, transB: bool = False, clear_accum: bool = True,
                 scales: bool = False, lda: int = 0, ldb: int = 0, ldc: int = 0,
                 force_kernel: Optional[str] = None, tile_n: int = 0, stages: int = 0,
                 num_ctas: int = 0, band_tiles: int = 0, epilogue: int = 0,
                 row_reduce: Optional[str] = None, row_reduce_clear: bool = True,
                 panel_tiles: int = 0, l2_hints: int = 0, k_split: int = 0):
        L = lib()
        d = GemmDesc()
        d.M, d.N, d.K = M, N, K
        d.a_type = d.b_type = ab_type
        d.c_type = ab_type if c_type is None else c_type
        d.lda, d.ldb, d.ldc = lda, ldb, ldc
        d.transA, d.transB = int(transA), int(transB)
        d.clear_accum = int(clear_accum)
        d.scale_mode = 1 if scales else 0
        d.force_kernel = 0 if force_kernel is None else 1 + {"simt": 0, "tcgen05": 1, "skinny": 2, "tcgen05_pair": 3, "tf32x3": 4}[force_kernel]
        d.tile_n, d.stages, d.num_ctas, d.band_tiles = tile_n, stages, num_ctas, band_tiles
        d.epilogue = epilogue
        d.row_reduce = 0 if row_reduce is None else 1 + REDUCE_KINDS[row_reduce]
        d.row_reduce_clear = int(row_reduce_clear)
        d.panel_tiles, d.l2_hints, d.k_split = panel_tiles, l2_hints, k_split
        self.desc = d
        self._h = C.c_void_p()
        _check(L.frisk_b200_gemm_plan_create(C.byref(d), C.byref(self._h)), "plan_create")
        info = PlanInfo()
        _check(L.frisk_b200_gemm_plan_info(self._h, C.byref(info)), "plan_info")
        self.info = info.as_dict()
        ws = C.c_size_t()
        _check(L.frisk_b200_gemm_workspace_bytes(self._h, C.byref(ws)), "workspace_bytes")
        self.workspace_bytes = int(ws.value)

    def refresh_info(self) -> dict:
        """Reads the plan's info again (its run counters change as the plan is used)."""
        info = PlanInfo()
        _check(lib().frisk_b200_gemm_plan_info(self._h, C.byref(info)), "plan_info")
        self.info = info.as_dict()
        return self.info

    def operand_layout(self, operand: int) -> dict:
        """The staged tile of operand 0 (UMMA rows) or 1 (UMMA columns) as the plan uses it."""
        lay, desc, boxes = TmaParams(), C.c_uint64(), C.c_int32()
        _check(lib().frisk_b200_gemm_plan_operand_layout(self._h, operand, C.byref(lay), C.byref(desc),
                                                         C.byref(boxes)), "plan_operand_layout")
        out = lay.as_dict()
        out["umma_desc_base"] = int(desc.value)
        out["tma_boxes_per_stage"] = int(boxes.value)
        return out

    @classmethod
    def for_workload(cls, w: W.GemmWorkload, **kw) -> "GemmPlan":
        return cls(w.M, w.N, w.K, w.ab_type, w.c_type, transA=w.transA, transB=w.transB,
                   clear_accum=w.clear_accum, scales=w.scale_a is not None, **kw)

    def close(self) -> None:
        if self._h:
            lib().frisk_b200_gemm_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def run(self, A, B, Cout, scale_a=None, scale_b=None, workspace=None, status=None,
            stream: int = 0) -> None:
        """Asynchronous launch on device buffers (torch CUDA tensors or raw addresses)."""
        ws_bytes = 0
        if workspace is not None:
            ws_bytes = workspace.numel() * workspace.element_size() if hasattr(workspace, "numel") \
                else self.workspace_bytes
        rc = lib().frisk_b200_gemm_run(self._h, _ptr(A), _ptr(B), _ptr(Cout), _ptr(scale_a),
                                       _ptr(scale_b), _ptr(workspace), ws_bytes, _ptr(status),
                                       stream or None)
        _check(rc, "gemm_run")

    def run_ex(self, A, B, Cout, *, scale_a=None, scale_b=None, workspace=None, status=None,
               stream: int = 0, row_reduce_dst=None, peers=()) -> None:
        """``run`` with the destination of a fused row reduce and / or peer copies of C (device
        addresses in other GPUs' memory: where this plan's rows start in each peer's whole C)."""
        a = GemmRunArgs()
        a.A, a.B, a.C = _ptr(A), _ptr(B), _ptr(Cout)
        a.scale_a, a.scale_b = _ptr(scale_a), _ptr(scale_b)
        a.workspace = _ptr(workspace)
        a.workspace_bytes = 0 if workspace is None else (
            workspace.numel() * workspace.element_size() if hasattr(workspace, "numel") else self.workspace_bytes)
        a.device_status = _ptr(status)
        a.stream = stream or None
        a.row_reduce_dst = _ptr(row_reduce_dst)
        a.n_peers = len(peers)
        for i, q in enumerate(peers):
            a.peer_c[i] = _ptr(q)
        _check(lib().frisk_b200_gemm_run_ex(self._h, C.byref(a)), "gemm_run_ex")

    def run_host(self, A: np.ndarray, B: np.ndarray, Cout: np.ndarray,
                 scale_a: Optional[np.ndarray] = None, scale_b: Optional[np.ndarray] = None,
                 row_reduce_dst: Optional[np.ndarray] = None) -> None:
        """Synchronous GEMM on host arrays (copies in, runs, copies C -- and the fused row
        reduce's destination, for a plan that has one -- back)."""
        rc = lib().frisk_b200_gemm_run_host_ex(self._h, _ptr(A), _ptr(B), _ptr(Cout), _ptr(scale_a),
                                               _ptr(scale_b), _ptr(row_reduce_dst))
        _check(rc, "gemm_run_host")


def check_status(status, stream: int = 0) -> None:
    _check(lib().frisk_b200_check_status(_ptr(status), stream or None), "device status")


def gemm_host(w: W.GemmWorkload, **plan_kw) -> np.ndarray:
    """Runs a workload from host buffers and returns C as raw storage bits."""
    plan = GemmPlan.for_workload(w, **plan_kw)
    out = np.zeros((w.M, w.N), dtype=W.storage_numpy_dtype(w.c_type))
    if not w.clear_accum and w.C0 is not None:
        out[...] = w.C0
    try:
        plan.run_host(np.ascontiguousarray(w.A), np.ascontiguousarray(w.B), out, w.scale_a, w.scale_b)
    finally:
        plan.close()
    return out


def reduce_desc(shape, dim: int, dtype: int, kind: str, clear: bool = True, device: int = -1) -> ReduceDesc:
    """``frisk.reduce`` of a row-major buffer of `shape` over dimension `dim` as the C ABI sees it:
    [outer, extent, inner] around the reduced dimension."""
    shape = [int(d) for d in shape]
    if not 0 <= dim < len(shape):
        raise ValueError(f"dimension {dim} is out of range for source of rank {len(shape)}")
    if kind not in REDUCE_KINDS:
        raise ValueError(f"unsupported reduce kind: {kind}. Supported: add, mul, min, max")
    outer = int(np.prod(shape[:dim], dtype=np.int64))
    inner = int(np.prod(shape[dim + 1:], dtype=np.int64))
    return ReduceDesc(outer, shape[dim], inner, dtype, REDUCE_KINDS[kind], int(bool(clear)), device)


def reduce_info(desc: ReduceDesc, src_aligned: bool = True) -> dict:
    info = ReduceInfo()
    _check(lib().frisk_b200_reduce_info(C.byref(desc), int(src_aligned), C.byref(info)), "reduce_info")
    return info.as_dict()


def reduce_workspace_bytes(desc: ReduceDesc) -> int:
    n = C.c_size_t()
    _check(lib().frisk_b200_reduce_workspace_bytes(C.byref(desc), C.byref(n)), "reduce_workspace_bytes")
    return int(n.value)


def reduce_run(desc: ReduceDesc, src, dst, workspace=None, stream: int = 0) -> None:
    """Asynchronous launch on device buffers (torch CUDA tensors or raw addresses)."""
    ws_bytes = 0
    if workspace is not None and hasattr(workspace, "numel"):
        ws_bytes = workspace.numel() * workspace.element_size()
    rc = lib().frisk_b200_reduce_run(C.byref(desc), _ptr(src), _ptr(dst), _ptr(workspace), ws_bytes,
                                     stream or None)
    _check(rc, "reduce_run")


def reduce_host(src: np.ndarray, dst: np.ndarray, dim: int, dtype: int, kind: str, clear: bool = True) -> None:
    """Synchronous ``frisk.reduce`` on host arrays of raw storage (copies in, runs, copies dst back)."""
    desc = reduce_desc(src.shape, dim, dtype, kind, clear)
    if not (src.flags.c_contiguous and dst.flags.c_contiguous):
        raise ValueError("reduce_host wants C-contiguous arrays")
    if dst.size != desc.outer * desc.inner or src.dtype != dst.dtype:
        raise ValueError("destination must have the source's shape without the reduced dimension and its type")
    _check(lib().frisk_b200_reduce_run_host(C.byref(desc), _ptr(src), _ptr(dst)), "reduce_run_host")


def shard_rows(M: int, nranks: int, rank: int) -> tuple[int, int]:
    """Rows [row0, row0 + rows) of A and C that `rank` owns when C = A*B is split by rows."""
    r0, n = C.c_int64(), C.c_int64()
    _check(lib().frisk_b200_shard_rows(M, nranks, rank, C.byref(r0), C.byref(n)), "shard_rows")
    return int(r0.value), int(n.value)


def layout_to_tma(rows: int, cols: int, elem_bits: int, k_inner: bool) -> dict:
    ld = LayoutDesc(rows, cols, elem_bits, int(k_inner))
    out = TmaParams()
    _check(lib().frisk_b200_layout_to_tma(C.byref(ld), C.byref(out)), "layout_to_tma")
    return out.as_dict()


def swizzled_offset(row: int, col: int, rows: int, cols: int, elem_bits: int, mode: int) -> int:
    return int(lib().frisk_b200_swizzled_offset(row, col, rows, cols, elem_bits, mode))


def bank_conflicts(rows: int, cols: int, elem_bits: int, mode: int, lane_vector: int,
                   distinct_words_only: bool = False) -> dict:
    st = BankStats()
    _check(lib().frisk_b200_bank_conflicts(rows, cols, elem_bits, mode, lane_vector,
                                           int(distinct_words_only), C.byref(st)), "bank_conflicts")
    return {"avg_max_conflict": st.avg_max_conflict, "max_conflict": st.max_conflict,
            "samples": st.samples}


def measure_mma_peak(ab_type: int, pair: bool = True, k_blocks: int = 1024, reps: int = 10) -> dict:
    """Rate of back-to-back tcgen05.mma from resident shared memory on the current device."""
    tf, ms = C.c_double(), C.c_double()
    _check(lib().frisk_b200_measure_mma_peak(ab_type, int(pair), k_blocks, reps, C.byref(tf), C.byref(ms)),
           "measure_mma_peak")
    return {"tflops": tf.value, "ms_per_launch": ms.value, "k_blocks": k_blocks, "pair": bool(pair)}


def bank_conflicts_access(rows: int, cols: int, elem_bits: int, mode: int, access: int) -> dict:
    st = AccessStats()
    _check(lib().frisk_b200_bank_conflicts_access(rows, cols, elem_bits, mode, access, C.byref(st)),
           "bank_conflicts_access")
    return {n: getattr(st, n) for n, _ in st._fields_}


def device_sm_count() -> int:
    return int(lib().frisk_b200_device_sm_count())


def version() -> str:
    return lib().frisk_b200_version().decode()


# Names the reference-facing ``frisk.runtime`` module is asked for: ``plan`` makes a plan for one
# GEMM, ``workspace_size`` tells what ``run`` needs beside the operands.
plan = GemmPlan


def workspace_size(p: "GemmPlan") -> int:
    return p.workspace_bytes
