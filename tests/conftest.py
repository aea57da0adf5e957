import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_ROOT = os.path.join(ROOT, "minfer-python_b200")
for p in (ROOT, PKG_ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")
    # the suite needs the C-ABI library in-tree; compile it (nvcc, no GPU needed) if it is missing or stale
    import importlib.util
    spec = importlib.util.spec_from_file_location("minfer_b200_build", os.path.join(PKG_ROOT, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()


@pytest.fixture(scope="session")
def kerns():
    """The reference-shaped facade; importing it registers the ops (reference: test/conftest.py:2)."""
    from minfer.kernels import KernelBackend
    return KernelBackend("torch_ext")
