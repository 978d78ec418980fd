import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(ROOT / "tests" / "golden" / "reference_golden.npz")


@pytest.fixture(scope="session")
def lib():
    from flashsampling_b200 import build

    build.build_library()
    from flashsampling_b200 import _lib

    return _lib.load()
