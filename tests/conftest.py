import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    """The C restatement (checker)."""
    from oracle import build as obuild
    from oracle.pyoracle import Oracle
    obuild.build_oracle()
    return Oracle()


@pytest.fixture(scope="session")
def ref():
    """The reference's own C++ behind the MLX shim, if it was built; otherwise skip."""
    from oracle.pyoracle import Ref, have_ref
    if not have_ref():
        pytest.skip("oracle/_ref/libtq_ref.so not built (reference source tree absent)")
    return Ref()


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "golden_v1.npz"))


@pytest.fixture(scope="session")
def tq():
    """The product package with its CUDA library loaded (fails if it is not built)."""
    import turboquant_mlx_core_b200 as pkg
    pkg.load()
    return pkg


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
