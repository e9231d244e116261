"""Multi-GPU tests (2 ranks by default, PICCL_TEST_RANKS to widen): every collective and algorithm
against NCCL, data-parallel training, the LD_PRELOAD shim under torch.distributed, and a host-injected
fault with a bounded device wait.  One process per GPU, launched with torch.distributed.run."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _ranks():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    want = int(os.environ.get("PICCL_TEST_RANKS", "2"))
    return min(n, want)


def _run(case, extra_env=None, nproc=None, timeout=600):
    n = nproc or _ranks()
    have = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if n < 2 or have < n:
        pytest.skip("needs at least two GPUs")
    env = dict(os.environ)
    env.update({"NCCL_NVLS_ENABLE": "0", "MASTER_ADDR": "127.0.0.1"})
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nnodes=1", f"--nproc-per-node={n}",
           str(ROOT / "tests" / "mp_worker.py"), case]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    ok = r.stdout.count(f"WORKER_OK {case}")
    assert r.returncode == 0 and ok == n, f"{case}: rc {r.returncode}, {ok}/{n} ranks ok\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}"
    return r.stdout


def test_collectives_match_nccl():
    _run("collectives")


def test_data_parallel_training():
    _run("ddp")


def test_fused_tensor_parallel_kernels():
    _run("tp")


def test_in_switch_collectives():
    out = _run("nvls", {"PICCL_NVLS": "1", "PICCL_LOG": "1"})
    if "NVLS_UNAVAILABLE" in out:
        pytest.skip("no NVLink multicast window on this machine")


def test_preload_shim_under_torch_distributed():
    from piccl_b200 import build
    so = str(build.lib_path("piccl.so"))
    env = {"LD_PRELOAD": so, "PICCL_ALLREDUCE_ALGO": "RING", "PICCL_ALLGATHER_ALGO": "PRD", "PICCL_BROADCAST_ALGO": "K_RING", "PICCL_BROADCAST_K": "2",
           "PICCL_REDUCE_SCATTER_ALGO": "PRM", "PICCL_REDUCE_SCATTER_K": "2", "PICCL_LOG": "1"}
    _run("shim", env)
    # algorithms unset: everything is handed to NCCL, as in the reference
    _run("shim", {"LD_PRELOAD": so, "EXPECT_NATIVE": "0"})


def test_host_injected_fault_is_reported_not_hung():
    # no multicast window in this test: a rank may leave while the others still wait
    _run("fault", {"PICCL_FAULT": "1:3:skip_call", "PICCL_NVLS": "0"}, nproc=2)
