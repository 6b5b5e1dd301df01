import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    """The package, with its libraries built (nvcc cross-compiles without a GPU)."""
    p = entry.load_package()
    if not all(os.path.exists(p.lib_path(k)) for k in p.LIB_FILES):
        p.build()
    return p


@pytest.fixture(scope="session")
def rt(pkg):
    import importlib
    return importlib.import_module(entry.PKG_ALIAS + ".runtime")


@pytest.fixture(scope="session")
def qz(pkg):
    import importlib
    return importlib.import_module(entry.PKG_ALIAS + ".runtime.quantize")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_vectors.npz"))
