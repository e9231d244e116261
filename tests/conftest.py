import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs at least one CUDA device")
    config.addinivalue_line("markers", "multigpu: needs two or more CUDA devices")


@pytest.fixture(scope="session")
def native():
    """Builds (if needed) and loads the native library."""
    from piccl_b200 import _native
    return _native.lib()
