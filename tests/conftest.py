import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu")


def _has_gpu():
    try:
        import ctypes as C
        from ancora_cutile_b200 import _lib
        n = C.c_int()
        _lib.lib().anc_device_count(C.byref(n))
        return n.value > 0
    except Exception:
        return False


@pytest.fixture(scope="session")
def ctx():
    """Device context; GPU tests fail (not skip) when the library or the GPU is missing,
    so a silent fallback can never pass them."""
    import ancora_cutile_b200 as anc
    return anc.get_context()


def pytest_collection_modifyitems(config, items):
    # When GPU tests are selected without a GPU (a plain `pytest tests` on a CPU box),
    # skip them; `-m gpu` on a GPU box runs them for real.
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
