import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def ref():
    """The CPU oracle (oracle/tl_ref.py) -- test infrastructure only."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import tl_ref
    tl_ref.build()
    return tl_ref


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_py.npz"))


@pytest.fixture(scope="session")
def lib():
    """libtlcuda.so, built in-tree if needed."""
    from tensorlogic_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.load()


@pytest.fixture(scope="session")
def dev(lib):
    """A device context; only GPU-marked tests may ask for it."""
    from tensorlogic_b200.api import Device
    d = Device(0)
    yield d
    d.close()


def rel_l2(a, b):
    import numpy as np
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
