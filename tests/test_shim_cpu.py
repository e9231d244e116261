"""Load path and configuration of the preload library, no GPU needed: banner, environment echo, exported
NCCL symbols, lazy resolution (nothing is opened at load time), and the schedule command line tool."""
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _so():
    sys.path.insert(0, str(ROOT))
    from piccl_b200 import _native
    _native.lib()
    return ROOT / "piccl_b200" / "lib" / "piccl.so"


def test_preload_banner_and_environment_echo():
    so = _so()
    env = dict(os.environ, LD_PRELOAD=str(so), PICCL_LOG="1", PICCL_ALLREDUCE_ALGO="PRM", PICCL_ALLREDUCE_K="4", PICCL_BROADCAST_ALGO="nonsense")
    r = subprocess.run(["/bin/true"], env=env, capture_output=True, text=True)
    assert r.returncode == 0
    assert "[PICCL] loaded (PID" in r.stderr                      # same banner as the reference (src/piccl.c:202)
    assert "ALLREDUCE_ALGO=PRM K=4" in r.stderr
    assert "BROADCAST_ALGO=DEFAULT" in r.stderr                   # unknown value: NCCL passthrough, as in the reference


def test_exports_the_nccl_abi_and_links_no_nccl():
    so = _so()
    syms = subprocess.run(["nm", "-D", "--defined-only", str(so)], capture_output=True, text=True).stdout
    for name in ["ncclAllReduce", "ncclAllGather", "ncclReduceScatter", "ncclReduce", "ncclBroadcast", "ncclCommInitRank", "ncclCommDestroy",
                 "ncclCommAbort", "ncclCommGetAsyncError", "ncclGroupStart", "ncclGroupEnd", "ncclBcast"]:
        assert f" T {name}\n" in syms, name
    needed = subprocess.run(["readelf", "-d", str(so)], capture_output=True, text=True).stdout
    assert "libnccl" not in needed                                # real symbols are resolved lazily with dlsym, never by linking
    assert "libcudart" not in needed                              # the CUDA runtime is linked statically


def test_algorithm_names_are_the_reference_names():
    sys.path.insert(0, str(ROOT))
    from piccl_b200 import _native as N
    lib = N.lib()
    names = {"RING": 1, "K_RING": 2, "RD": 3, "RM": 4, "PRD": 5, "PRM": 6, "AUTO": 7}
    for k, v in names.items():
        assert lib.piccl_algo_from_string(k.encode()) == v
    for bad in [b"ring", b"", b"NCCL", b"DEFAULT"]:
        assert lib.piccl_algo_from_string(bad) == 0               # anything else: passthrough


def test_piccl_sched_cli():
    sys.path.insert(0, str(ROOT))
    from piccl_b200 import build
    tool = build.lib_path("piccl_sched")
    if not tool.exists():
        build.build(only=["piccl_sched"])
    r = subprocess.run([str(tool), "validate", "--collective", "allreduce", "--algorithm", "PRM", "--k", "4", "--nodes", "8", "--buffer-size", "65536", "--cta", "4", "--fifo", "2"],
                       capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.startswith("OK")
    r = subprocess.run([str(tool), "xml", "--collective", "bcast", "--algorithm", "PRD", "--nodes", "8", "--buffer-size", "1024"], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.count("<transfer") == 7
    r = subprocess.run([str(tool), "json", "--collective", "allgather", "--algorithm", "PRD", "--nodes", "4", "--buffer-size", "4096", "--rank", "1"], capture_output=True, text=True)
    assert '"algorithm":"PRD"' in r.stdout
