"""In-switch collectives (algorithm NVLS) on ONE GPU with the switch emulated: see nvls_worker.py.
The run is a child process because the window geometry is read from the environment once per process."""
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("depth", ["4", "3", "2"])
def test_in_switch_collectives_with_an_emulated_switch(depth):
    import os
    env = dict(os.environ, PICCL_NVLS_DEPTH=depth)
    r = subprocess.run([sys.executable, str(ROOT / "tests" / "nvls_worker.py")], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "NVLS_EMULATED_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
