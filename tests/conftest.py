import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _has_gpu():
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


@pytest.fixture(scope="session")
def native_libs():
    """Build (if stale) and return the path of the CUDA library; building needs nvcc only."""
    from orinmllm_b200 import build
    so = build.LIB / "libkpx.so"
    if not so.exists() or os.environ.get("KPX_REBUILD"):
        build.build_all()
    if os.environ.get("KPX_DECODE_VARIANT"):
        import ctypes
        ctypes.CDLL(str(so)).kpx_internal_set_decode_variant(int(os.environ["KPX_DECODE_VARIANT"]))
    return so


@pytest.fixture(scope="session")
def oracle():
    from tests import kvtest
    return kvtest.load_oracle()
