import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def built_library():
    """Build (if stale) and load the C-ABI library; CPU-only hosts can do this too (nvcc cross-compiles)."""
    from int4matmul_kernels_b200 import _build, capi
    if not os.path.exists(capi.library_path()):
        _build.build_capi()
    return capi.load()
