"""Host code under AddressSanitizer + UndefinedBehaviorSanitizer: the schedule compiler / validator / dumps
(src/coll, src/tools/piccl_sched.cc) and the descriptor hand-over between ranks (src/runtime/fdshare.cc).
Device code cannot be run under these tools here; its bounds are checked by the CPU validator and by PICCL_DEBUG=1."""
import itertools
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SAN = ["-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer", "-Wall", "-Wextra", "-Werror"]
ENV = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")


def _build(out: Path, sources, extra=()):
    cmd = ["g++", *SAN, f"-I{ROOT / 'src' / 'include'}", *map(str, sources), "-o", str(out), "-lpthread", *extra]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]
    return out


@pytest.fixture(scope="module")
def sched(tmp_path_factory):
    d = tmp_path_factory.mktemp("san")
    return _build(d / "piccl_sched_san", sorted((ROOT / "src" / "coll").glob("*.cc")) + [ROOT / "src" / "tools" / "piccl_sched.cc"])


def _run(tool, *args):
    r = subprocess.run([str(tool), *map(str, args)], capture_output=True, text=True, env=ENV, timeout=120)
    assert "runtime error" not in r.stderr and "AddressSanitizer" not in r.stderr and "LeakSanitizer" not in r.stderr, r.stderr[-3000:]
    return r


def test_schedule_layer_is_clean_under_asan_and_ubsan(sched):
    colls = ["allgather", "allreduce", "bcast", "reduce", "reduce_scatter"]
    algos = ["RING", "K_RING", "RD", "RM", "PRD", "PRM", "DIRECT", "NVLS"]
    for coll, algo in itertools.product(colls, algos):
        for n, k in [(1, -1), (3, 2), (8, 2), (8, 8), (12, 5), (16, 4)]:
            r = _run(sched, "validate", "--collective", coll, "--algorithm", algo, "--k", k, "--nodes", n, "--buffer-size", 4 * 257 * n, "--cta", 3, "--fifo", 2, "--seg", 32)
            assert r.returncode == 0 and r.stdout.startswith("OK"), (coll, algo, n, k, r.stdout, r.stderr[-500:])
        r = _run(sched, "validate", "--collective", coll, "--algorithm", algo, "--nodes", 8, "--buffer-size", 4096, "--in-place", "--int", "--op", "max")
        assert r.returncode == 0 and r.stdout.startswith("OK"), (coll, algo, r.stdout)
        assert _run(sched, "xml", "--collective", coll, "--algorithm", algo, "--k", 4, "--nodes", 8, "--buffer-size", 8192).returncode == 0
        assert _run(sched, "json", "--collective", coll, "--algorithm", algo, "--k", 3, "--nodes", 9, "--buffer-size", 9000, "--rank", 8).returncode == 0
    # sizes too large to materialise, tiny and zero sizes, invalid radices
    assert _run(sched, "validate", "--collective", "allreduce", "--algorithm", "PRM", "--k", 8, "--nodes", 8, "--buffer-size", 1 << 30, "--symbolic", "--cta", 64, "--fifo", 2).stdout.startswith("OK")
    for size in (0, 4, 8):
        assert _run(sched, "validate", "--collective", "allreduce", "--algorithm", "DIRECT", "--nodes", 8, "--buffer-size", size).returncode == 0
    assert _run(sched, "validate", "--collective", "allgather", "--algorithm", "K_RING", "--k", 0, "--nodes", 6, "--buffer-size", 4096).returncode == 0


def test_descriptor_hand_over_is_clean_under_asan_and_ubsan(tmp_path):
    tool = _build(tmp_path / "fdshare_san", [ROOT / "src" / "runtime" / "fdshare.cc", ROOT / "tests" / "native" / "fdshare_main.cc"])
    payload = tmp_path / "payload.txt"
    payload.write_text("hand-over")
    name = f"piccl-san-{os.getpid()}"
    procs = [subprocess.Popen([str(tool), str(r), "3", name, "5000", "1", str(payload)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=ENV) for r in range(3)]
    outs = [p.communicate(timeout=60) for p in procs]
    for out, err in outs:
        assert "runtime error" not in err and "AddressSanitizer" not in err and "LeakSanitizer" not in err, err[-3000:]
        assert out.startswith("0 1 hand-over|"), (out, err)
    # a rank that never shows up: everybody gives up within the limit, nothing leaks
    procs = [subprocess.Popen([str(tool), str(r), "3", name + "-b", "800", "1", str(payload)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=ENV) for r in range(2)]
    outs = [p.communicate(timeout=60) for p in procs]
    for out, err in outs:
        assert "runtime error" not in err and "AddressSanitizer" not in err and "LeakSanitizer" not in err, err[-3000:]
        assert not out.startswith("0 1")
