"""frisk_b200: a B200-native execution back end for ``frisk.gemm`` behind Frisk's IR-builder API.

* ``frisk_b200.runtime``  -- ctypes binding of libfrisk_b200.so (plans, launches, layout mapping);
* ``frisk_b200.workloads`` -- synthetic benchmark inputs and numpy storage codecs;
* the IR-builder surface of the reference (``context``, ``builder``, ``MemorySpace``, ...) is
  re-exported from the native ``frisk_ffi`` module when it has been built.
"""
from . import workloads  # noqa: F401

try:  # the IR builder is a separate native module; the runtime works without it
    from .frisk_ffi import ir  # noqa: F401
    from .frisk_ffi.ir import *  # noqa: F401,F403
    from .common.utils import FriskHelper, create_context, create_session  # noqa: F401
    from .execute import find_gemms, run  # noqa: F401
except ImportError:  # pragma: no cover - before `python -m frisk_b200.build`
    ir = None
