import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselected on CPU-only hosts")


@pytest.fixture(scope="session")
def oracle():
    from oracle.oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own format class compiled from its checkout; None where it is unavailable."""
    from oracle.oracle import Reference
    return Reference.load()


@pytest.fixture(scope="session")
def golden_format():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "format_golden.npz"))


@pytest.fixture(scope="session")
def golden_prune():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "prune_golden.npz"))
