import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def _cuda_ok():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _cuda_ok():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def built_lib():
    """Builds (if stale) and loads the shared library."""
    from pratchya_b200.csrc.build import build
    build()
    from pratchya_b200 import _lib
    return _lib.load()


@pytest.fixture(scope="session")
def diag_lib():
    """Builds (if stale) and loads the diagnostics build of the library (test hooks, fault injection)."""
    from pratchya_b200.csrc.build import build
    build(diagnostics=True)
    from pratchya_b200 import _lib
    return _lib.load_diagnostics()
