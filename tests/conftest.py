import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    path = os.path.join(ROOT, "tests", "golden", "reference_vectors.npz")
    return dict(np.load(path, allow_pickle=False))


@pytest.fixture(scope="session")
def refmod():
    """The compiled, unmodified reference operator; skipped when it is not built and the
    reference sources are not available to build it."""
    from oracle import ref_python as rp

    if not rp.have_reference():
        pytest.skip("compiled reference (oracle/_ref) not available")
    return rp
