"""``import frisk as F`` -- the package name of the reference (python/frisk/__init__.py:1-4).

Everything comes from frisk_b200: the IR-builder surface (``context``, ``builder``, ``frisk``,
``MemorySpace``, ``AffineMap`` ...), the session helpers, and ``runtime`` / ``run`` for execution.
"""
from frisk_b200.frisk_ffi.ir import *  # noqa: F401,F403
from frisk_b200.frisk_ffi import ir  # noqa: F401
from frisk_b200.common.utils import FriskHelper, create_context, create_session  # noqa: F401
from frisk_b200 import runtime  # noqa: F401
from frisk_b200.execute import FriskWarning, find_gemms, parse_module, run  # noqa: F401

__all__ = [name for name in globals().keys() if not name.startswith("_")]
