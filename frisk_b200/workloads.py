"""Synthetic GEMM workloads and numpy storage codecs.

The five configurations are seeded synthetic inputs with the shapes, layouts and value
distributions of the benchmark configurations (no dataset is involved).  RNG rule:
``numpy.random.default_rng(seed)``; draw A, then B, then scale_a, then scale_b, each as float32 in
C order, then round to nearest even into the storage type.

Storage types are carried as numpy arrays of raw bits: float32 -> float32, fp16 -> float16,
bf16 -> uint16 (upper half of the float32), e4m3fn -> uint8.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np

F32, F16, BF16, E4M3, E5M2 = 0, 1, 2, 3, 4  # frisk_dtype of include/frisk_b200.h
DTYPE_NAMES = {F32: "fp32", F16: "fp16", BF16: "bf16", E4M3: "e4m3fn", E5M2: "e5m2"}
ELEM_SIZE = {F32: 4, F16: 2, BF16: 2, E4M3: 1, E5M2: 1}


# --------------------------------------------------------------------------- codecs
def bf16_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bits (uint16), round to nearest even; NaN stays NaN."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = ((u.astype(np.uint64) + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    return np.where(nan, ((u >> 16) | 0x40).astype(np.uint16), rounded)


def bf16_decode(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _e4m3_table() -> np.ndarray:
    v = np.arange(256, dtype=np.int64)
    sign = np.where(v >> 7, -1.0, 1.0)
    exp = (v >> 3) & 0xF
    man = v & 7
    mag = np.where(exp == 0, man / 8.0 * 2.0 ** -6, (1.0 + man / 8.0) * 2.0 ** (exp - 7.0))
    out = (sign * mag).astype(np.float32)
    out[(exp == 15) & (man == 7)] = np.nan
    return out


E4M3_TABLE = _e4m3_table()
E4M3_MAX = 448.0


def e4m3_decode(q: np.ndarray) -> np.ndarray:
    return E4M3_TABLE[np.ascontiguousarray(q, dtype=np.uint8)]


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> e4m3fn bits, round to nearest even, saturating to +-448 (never NaN/inf)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    a = np.minimum(np.abs(x.astype(np.float64)), E4M3_MAX)
    a = np.where(np.isnan(a), E4M3_MAX, a)
    # spacing of the grid around a: 2^(e-3) for normals (e >= -6), 2^-9 below
    e = np.floor(np.log2(np.maximum(a, 2.0 ** -6)))
    step = 2.0 ** (e - 3)
    r = np.rint(a / step) * step  # np.rint rounds half to even; a/step is exact in float64
    r = np.minimum(r, E4M3_MAX)
    # back to bits
    e2 = np.floor(np.log2(np.maximum(r, 2.0 ** -6)))
    normal = r >= 2.0 ** -6
    man = np.where(normal, np.rint((r / 2.0 ** e2 - 1.0) * 8.0), np.rint(r / 2.0 ** -9))
    expf = np.where(normal, e2 + 7, 0)
    bits = (expf.astype(np.int64) << 3) | man.astype(np.int64)
    bits |= np.signbit(x).astype(np.int64) << 7
    return bits.astype(np.uint8)


E5M2_MAX = 57344.0


def e5m2_decode(q: np.ndarray) -> np.ndarray:
    """e5m2 bits are the top byte of an IEEE half."""
    return (np.ascontiguousarray(q, dtype=np.uint8).astype(np.uint16) << 8).view(np.float16).astype(np.float32)


def e5m2_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> e5m2 bits, round to nearest even, saturating to +-57344 (never NaN/inf), the
    same convention as e4m3_encode."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    a = np.minimum(np.abs(x.astype(np.float64)), E5M2_MAX)
    a = np.where(np.isnan(a), E5M2_MAX, a)
    # spacing of the grid around a: 2^(e-2) for normals (e >= -14), 2^-16 below
    e = np.floor(np.log2(np.maximum(a, 2.0 ** -14)))
    step = 2.0 ** (e - 2)
    r = np.minimum(np.rint(a / step) * step, E5M2_MAX)   # exact in float64; rint rounds half to even
    bits = (r.astype(np.float16).view(np.uint16) >> 8).astype(np.uint8)   # r is exact in fp16
    return bits | (np.signbit(x).astype(np.uint8) << 7)


def encode(x: np.ndarray, dtype: int) -> np.ndarray:
    if dtype == F32:
        return np.ascontiguousarray(x, dtype=np.float32)
    if dtype == F16:
        return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16)
    if dtype == BF16:
        return bf16_encode(x)
    if dtype == E4M3:
        return e4m3_encode(x)
    if dtype == E5M2:
        return e5m2_encode(x)
    raise ValueError(f"unknown dtype {dtype}")


def decode(x: np.ndarray, dtype: int) -> np.ndarray:
    if dtype == F32:
        return np.asarray(x, dtype=np.float32)
    if dtype == F16:
        return np.asarray(x).view(np.float16).astype(np.float32)
    if dtype == BF16:
        return bf16_decode(x)
    if dtype == E4M3:
        return e4m3_decode(x)
    if dtype == E5M2:
        return e5m2_decode(x)
    raise ValueError(f"unknown dtype {dtype}")


def storage_numpy_dtype(dtype: int):
    return {F32: np.float32, F16: np.float16, BF16: np.uint16, E4M3: np.uint8, E5M2: np.uint8}[dtype]


# --------------------------------------------------------------------------- workloads
@dataclass
class GemmWorkload:
    """One GEMM problem: logical A [M,K], B [K,N], C [M,N]; buffers hold the stored order."""

    name: str
    M: int
    N: int
    K: int
    ab_type: int
    c_type: int
    transA: bool = False  # A stored [K, M]
    transB: bool = False  # B stored [N, K] ("column-major B")
    clear_accum: bool = True
    seed: int = 0
    A: Optional[np.ndarray] = None  # stored order, storage bits
    B: Optional[np.ndarray] = None
    scale_a: Optional[np.ndarray] = None
    scale_b: Optional[np.ndarray] = None
    C0: Optional[np.ndarray] = None  # initial C when clear_accum is False
    meta: dict = field(default_factory=dict)

    @property
    def flops(self) -> int:
        return 2 * self.M * self.N * self.K

    @property
    def algorithmic_bytes(self) -> int:
        es, cs = ELEM_SIZE[self.ab_type], ELEM_SIZE[self.c_type]
        n = self.M * self.K * es + self.K * self.N * es + self.M * self.N * cs
        if self.scale_a is not None:
            n += 4 * (self.M + self.N)
        return n

    def a_logical(self) -> np.ndarray:
        a = decode(self.A, self.ab_type)
        return a.T if self.transA else a

    def b_logical(self) -> np.ndarray:
        b = decode(self.B, self.ab_type)
        return b.T if self.transB else b


def _normal(rng, shape, scale=1.0):
    x = rng.standard_normal(shape, dtype=np.float32)
    if scale != 1.0:
        x *= np.float32(scale)
    return x


def make_workload(name: str, M: int | None = None, N: int | None = None, K: int | None = None,
                  seed: int | None = None) -> GemmWorkload:
    """Builds one of the named configurations; M/N/K override the full sizes for small tests."""
    if name == "cfg1":  # fp32 512^3, row-major, U(-1, 1), seed 0
        M, N, K = M or 512, N or 512, K or 512
        seed = 0 if seed is None else seed
        rng = np.random.default_rng(seed)
        a = rng.uniform(-1.0, 1.0, (M, K)).astype(np.float32)
        b = rng.uniform(-1.0, 1.0, (K, N)).astype(np.float32)
        return GemmWorkload(name, M, N, K, F32, F32, seed=seed, A=a, B=b)
    if name == "cfg2":  # fp16 4096^3, A row-major, B column-major, N(0,1)/sqrt(K), seed 1
        M, N, K = M or 4096, N or 4096, K or 4096
        seed = 1 if seed is None else seed
        rng = np.random.default_rng(seed)
        s = 1.0 / np.sqrt(K)
        a = _normal(rng, (M, K), s)
        b = _normal(rng, (K, N), s)  # drawn in logical [K, N] order, stored transposed
        return GemmWorkload(name, M, N, K, F16, F16, transB=True, seed=seed,
                            A=encode(a, F16), B=np.ascontiguousarray(encode(b, F16).T))
    if name == "cfg3":  # bf16 skinny 16 x 8192 x 8192, A N(0,1), B N(0,0.02), seed 2
        M, N, K = M or 16, N or 8192, K or 8192
        seed = 2 if seed is None else seed
        rng = np.random.default_rng(seed)
        a = _normal(rng, (M, K))
        b = _normal(rng, (K, N), 0.02)
        return GemmWorkload(name, M, N, K, BF16, BF16, seed=seed, A=encode(a, BF16),
                            B=encode(b, BF16))
    if name == "cfg4":  # e4m3 8192^3, per-row / per-column fp32 scales, bf16 C, seed 3
        M, N, K = M or 8192, N or 8192, K or 8192
        seed = 3 if seed is None else seed
        rng = np.random.default_rng(seed)
        xa = _normal(rng, (M, K))
        xb = _normal(rng, (K, N))
        sa = (rng.uniform(0.5, 2.0, M) / 448.0).astype(np.float32)
        sb = (rng.uniform(0.5, 2.0, N) / 448.0).astype(np.float32)
        qa = e4m3_encode(xa / sa[:, None])
        qb = e4m3_encode(xb / sb[None, :])
        return GemmWorkload(name, M, N, K, E4M3, BF16, transB=True, seed=seed, A=qa,
                            B=np.ascontiguousarray(qb.T), scale_a=sa, scale_b=sb)
    if name in ("cfg5", "bf16_8192"):  # bf16, A N(0,1), B N(0,0.02), row-major; seeds 4 / 5
        if name == "cfg5":
            M, N, K = M or 65536, N or 8192, K or 8192
            seed = 4 if seed is None else seed
        else:
            M, N, K = M or 8192, N or 8192, K or 8192
            seed = 5 if seed is None else seed
        rng = np.random.default_rng(seed)
        a = encode(_normal(rng, (M, K)), BF16)
        b = encode(_normal(rng, (K, N), 0.02), BF16)
        return GemmWorkload(name, M, N, K, BF16, BF16, seed=seed, A=a, B=b)
    raise ValueError(f"unknown workload {name!r}")


WORKLOADS = ("cfg1", "cfg2", "cfg3", "cfg4", "cfg5", "bf16_8192")


# --------------------------------------------------------------------------- error metrics
def rel_frobenius(c: np.ndarray, ref: np.ndarray) -> float:
    c = np.asarray(c, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.linalg.norm(c - ref) / max(np.linalg.norm(ref), 1e-300))


def max_rel_error(c: np.ndarray, ref: np.ndarray, absdot: np.ndarray | None = None) -> float:
    """max |c - r| / max(|r|, floor).

    An output of a dot product can cancel to (almost) zero while its fp32 accumulation error stays
    proportional to the data it summed, so a plain relative error is unbounded there.  With
    ``absdot`` = sum_k |a||b| the floor is 1e-3 * absdot (error relative to the data behind each
    output); without it the floor is 1e-3 * rms(r), which is tighter and fits short K only.
    """
    c = np.asarray(c, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    if absdot is not None:
        floor = np.maximum(1e-3 * np.asarray(absdot, dtype=np.float64), 1e-300)
    else:
        floor = max(1e-3 * float(np.sqrt(np.mean(ref * ref))), 1e-300)
    den = np.maximum(np.abs(ref), floor)
    return float(np.max(np.abs(c - ref) / den))


def parity_metrics(c: np.ndarray, ref: np.ndarray, absdot: np.ndarray | None = None,
                   bound: float | None = None) -> dict:
    """Every error figure the parity tests report for one result, side by side:

    * ``rel_frobenius``: ||c - r||_F / ||r||_F;
    * ``max_rel_rms_floor``: max |c - r| / max(|r|, 1e-3 rms(r)) -- the floor relative to the
      size of a typical output;
    * ``max_rel_data_floor``: the same with the floor 1e-3 sum_k |a||b| (needs ``absdot``) --
      relative to the data behind each output, the one that stays meaningful for long K;
    * ``below_rms_floor``: the share of outputs whose |r| lies under the rms floor (the outputs
      on which the two floors differ);
    * ``over_bound_rms_floor`` (with ``bound``): the share of outputs whose rms-floor error exceeds
      the bound, and ``over_bound_largest_ref``: the largest |r| / rms(r) among them (how close
      to a typical output the worst offender is; 1e-3 is the floor itself).
    """
    c = np.asarray(c, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    rms_floor = max(1e-3 * float(np.sqrt(np.mean(ref * ref))), 1e-300)
    out = {
        "rel_frobenius": rel_frobenius(c, ref),
        "max_rel_rms_floor": max_rel_error(c, ref),
        "max_rel_data_floor": None if absdot is None else max_rel_error(c, ref, absdot),
        "below_rms_floor": float(np.mean(np.abs(ref) < rms_floor)),
    }
    if bound is not None:
        over = np.abs(c - ref) / np.maximum(np.abs(ref), rms_floor) > bound
        out["over_bound_rms_floor"] = float(np.mean(over))
        out["over_bound_largest_ref"] = float(np.max(np.abs(ref)[over]) / (1e3 * rms_floor)) if over.any() else 0.0
    return out


TOLERANCE = {  # (metric, bound) per input type
    F32: ("rel_frobenius", 1e-4),
    F16: ("max_rel", 1e-2),
    BF16: ("max_rel", 1e-2),
    E4M3: ("max_rel", 2e-2),
    E5M2: ("max_rel", 2e-2),
}


def check(c: np.ndarray, ref: np.ndarray, ab_type: int,
          absdot: np.ndarray | None = None) -> tuple[bool, float, str]:
    """Applies the tolerance of the input type: fp32 -> relative Frobenius error <= 1e-4;
    fp16/bf16 -> max relative error <= 1e-2; e4m3 -> <= 2e-2 (see max_rel_error for the floor)."""
    metric, bound = TOLERANCE[ab_type]
    err = rel_frobenius(c, ref) if metric == "rel_frobenius" else max_rel_error(c, ref, absdot)
    return bool(err <= bound), err, metric
