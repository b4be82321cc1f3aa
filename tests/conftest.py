import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def lib():
    """The CUDA library through its ctypes binding; GPU tests fail loudly when it is missing."""
    from mase_triton_b200 import _lib

    return _lib.load()
