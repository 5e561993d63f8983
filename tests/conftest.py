import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def golden():
    """name -> lazily loaded npz archive of tests/golden/."""
    cache = {}

    def load(name):
        if name not in cache:
            cache[name] = np.load(GOLDEN / f"{name}.npz")
        return cache[name]

    return load
