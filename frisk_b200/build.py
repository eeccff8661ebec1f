"""Builds the native parts in-tree: libfrisk_b200.so (CUDA, sm_100a) and the frisk_ffi module.

Run as ``python -m frisk_b200.build``; ``__graft_entry__.build()`` calls :func:`build_all`.
nvcc cross-compiles for sm_100a, so no GPU is needed to build.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "libfrisk_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str]) -> None:
    print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def _csrc_files(exts: tuple[str, ...], sub: str = "") -> list[str]:
    d = os.path.join(CSRC, sub)
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(exts))


def build_runtime(force: bool = False, verbose_ptxas: bool = False) -> str:
    """nvcc -> frisk_b200/libfrisk_b200.so (kernels + C ABI)."""
    deps = _csrc_files((".cu", ".cuh", ".cpp")) + [os.path.join(ROOT, "include", "frisk_b200.h")]
    if not force and _newer(LIB, deps):
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    srcs = [os.path.join(CSRC, "frisk_b200.cu"), os.path.join(CSRC, "reduce.cu"),
            os.path.join(CSRC, "layout_map.cpp")]
    cmd = [nvcc, *NVCC_FLAGS, "-shared", "-o", LIB, *srcs, "-lcudart"]
    if verbose_ptxas:
        cmd[1:1] = ["-Xptxas", "-v"]
    _run(cmd)
    return LIB


def ffi_path() -> str:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(HERE, "frisk_ffi" + suffix)


def build_ffi(force: bool = False) -> str:
    """g++ -> frisk_b200/frisk_ffi.<abi>.so (the MLIR-free IR builder, pybind11)."""
    import pybind11

    out = ffi_path()
    ir_dir = os.path.join(CSRC, "ir")
    if not os.path.isdir(ir_dir):
        return out
    srcs = _csrc_files((".cpp",), "ir")
    deps = srcs + _csrc_files((".h",), "ir")
    if not force and _newer(out, deps):
        return out
    # the system compiler first: some toolchain wrappers link shared objects without libstdc++
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else os.environ.get("CXX", "g++")
    cmd = [
        cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
        "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], *srcs, "-o", out,
        "-lstdc++",
    ]
    _run(cmd)
    return out


def build_all(force: bool = False) -> None:
    build_runtime(force)
    build_ffi(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    if "--ptxas" in sys.argv:
        build_runtime(force=True, verbose_ptxas=True)
