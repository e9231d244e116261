"""In-switch all-reduce (algorithm NVLS, PICCL_NVLS=1) on one GPU: see nvls_worker.py.
The run is a child process because the switch is read from the environment once per process."""
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_nvls_allreduce_on_a_one_device_multicast_object():
    r = subprocess.run([sys.executable, str(ROOT / "tests" / "nvls_worker.py")], capture_output=True, text=True, timeout=300)
    if "NVLS_UNAVAILABLE" in r.stdout:
        pytest.skip("no NVLink multicast window on this device: " + r.stderr[-300:])
    assert r.returncode == 0 and "NVLS_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
