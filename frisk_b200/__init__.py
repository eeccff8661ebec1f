"""frisk_b200: a B200-native execution back end for ``frisk.gemm`` behind Frisk's IR-builder API.

* ``frisk_b200.runtime``  -- ctypes binding of libfrisk_b200.so (plans, launches, layout mapping);
* ``frisk_b200.workloads`` -- synthetic benchmark inputs and numpy storage codecs;
* the IR-builder surface of the reference (``context``, ``builder``, ``MemorySpace``, ...) comes
  from the native ``frisk_ffi`` module, which is loaded on first use: a process that only needs
  the workload generators (the CPU baseline of the benchmark) maps no native code of this package.
"""
import importlib

from . import workloads  # noqa: F401

_HELPERS = {"FriskHelper": ".common.utils", "create_context": ".common.utils",
            "create_session": ".common.utils", "find_gemms": ".execute", "run": ".execute",
            "parse_module": ".execute", "FriskWarning": ".execute"}


def __getattr__(name):
    """Resolves the IR-builder names on first access (PEP 562)."""
    if name.startswith("__"):
        raise AttributeError(name)
    if name in _HELPERS:
        return getattr(importlib.import_module(_HELPERS[name], __name__), name)
    if name in ("runtime", "execute", "sharding", "build", "common"):
        return importlib.import_module("." + name, __name__)
    try:
        ffi = importlib.import_module(".frisk_ffi", __name__)
    except ImportError as e:  # before `python -m frisk_b200.build`
        raise AttributeError(f"frisk_b200.{name}: the frisk_ffi module is not built ({e})") from None
    if name == "ir":
        return ffi.ir
    try:
        return getattr(ffi.ir, name)
    except AttributeError:
        raise AttributeError(f"module 'frisk_b200' has no attribute {name!r}") from None
