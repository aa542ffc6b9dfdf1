import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# compiled kernels are cached in-tree so that a cache filled on one machine travels with the checkout
os.environ.setdefault("ACCELERATE_B200_CACHE_DIR", os.path.join(ROOT, ".kernel_cache"))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def lib_built():
    """Build the C-ABI library in-tree (g++/nvcc only; no GPU needed)."""
    from accelerate_b200 import build
    return build.build()


@pytest.fixture(scope="session")
def gpu_ctx(lib_built):
    from accelerate_b200 import backend
    return backend.default_context()
