"""pytest configuration: the ``gpu`` marker and one-time native builds."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100); run with -m gpu")


def _has_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def native_builds():
    """Builds libfrisk_b200.so, the frisk_ffi module and the oracle when they are missing
    (nvcc cross-compiles for sm_100a without a GPU)."""
    from frisk_b200 import build as B

    if not os.path.exists(B.LIB) or not os.path.exists(B.ffi_path()):
        B.build_all()
    from oracle import ref

    ref.build()
    yield
