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
    names = {"RING": 1, "K_RING": 2, "RD": 3, "RM": 4, "PRD": 5, "PRM": 6, "AUTO": 7, "DIRECT": 8, "NVLS": 9}
    for k, v in names.items():
        assert lib.piccl_algo_from_string(k.encode()) == v
    for bad in [b"ring", b"", b"NCCL", b"DEFAULT"]:
        assert lib.piccl_algo_from_string(bad) == 0               # anything else: passthrough


def test_protocol_switch_and_effective_configuration():
    """PICCL_PROTO narrows the per-call choice of data path; piccl_env_describe reports what is in force."""
    code = ("import ctypes as C, sys; sys.path.insert(0, %r); from piccl_b200 import _native as N; l = N.lib(); "
            "b = C.create_string_buffer(1024); l.piccl_env_describe(b, 1024); print(b.value.decode())") % str(ROOT)

    def describe(**env):
        e = dict(os.environ); e.update(env)
        out = subprocess.run([sys.executable, "-c", code], env=e, capture_output=True, text=True, check=True).stdout.strip().splitlines()[-1]
        return dict(kv.split("=", 1) for kv in out.split())

    d = describe()
    assert d["proto"] == "auto" and d["ll_kb"] == "1024" and d["llf_kb"] == "64" and d["nvls"] == "1" and d["allreduce"] == "DEFAULT/-1"
    d = describe(PICCL_PROTO="simple")
    assert d["proto"] == "simple" and d["ll_kb"] == "0" and d["llf_kb"] == "0"
    d = describe(PICCL_PROTO="ll")
    assert d["proto"] == "ll" and d["llf_kb"] == "1024"
    d = describe(PICCL_PROTO="nvls", PICCL_ALLREDUCE_ALGO="DIRECT", PICCL_ALLGATHER_ALGO="PRM", PICCL_ALLGATHER_K="4", PICCL_NVLS_MIN_KB="32")
    assert d["proto"] == "nvls" and d["nvls"] == "1" and d["nvls_min_kb"] == "32" and d["allreduce"] == "DIRECT/-1" and d["allgather"] == "PRM/4"
    d = describe(PICCL_PROTO="bogus")
    assert d["proto"] == "auto"


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


# ---------------------------------------------------------------- descriptor hand-over between the ranks of one host
def _fdshare_rank(rank, nranks, name, path, ok, timeout_ms, q):
    import ctypes as C
    import os
    from piccl_b200 import _native as N
    l = N.lib()
    fd = os.open(path, os.O_RDONLY) if rank == 0 else -1
    out, all_ok, err = C.c_int(-1), C.c_int(-1), C.create_string_buffer(256)
    rc = l.piccl_fdshare_selftest(rank, nranks, name.encode(), fd, timeout_ms, int(ok), C.byref(out), C.byref(all_ok), err, 256)
    text = None
    if rc == 0 or out.value >= 0:
        try:
            text = os.pread(out.value, 64, 0).decode()
        except OSError:
            text = None
    q.put((rank, rc, all_ok.value, text, err.value.decode()))


def _run_fdshare(nranks, votes, tmp_path, timeout_ms=5000, absent=()):
    import multiprocessing as mp
    import os
    ctx = mp.get_context("spawn")
    path = tmp_path / "payload.txt"
    path.write_text("descriptor payload")
    name = f"piccl-test-{os.getpid()}-{nranks}-{len(absent)}-{sum(votes)}"
    q = ctx.Queue()
    procs = [ctx.Process(target=_fdshare_rank, args=(r, nranks, name, str(path), votes[r], timeout_ms, q)) for r in range(nranks) if r not in absent]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=60) for _ in procs)
    for p in procs:
        p.join(30)
    return res


def test_fdshare_hands_the_descriptor_to_every_rank(tmp_path):
    res = _run_fdshare(4, [True] * 4, tmp_path)
    assert [r[0] for r in res] == [0, 1, 2, 3]
    for rank, rc, all_ok, text, err in res:
        assert rc == 0 and all_ok == 1 and text == "descriptor payload", (rank, rc, err)


def test_fdshare_barrier_spreads_one_rank_failure(tmp_path):
    res = _run_fdshare(3, [True, False, True], tmp_path)
    for rank, rc, all_ok, text, err in res:
        assert rc == 0 and all_ok == 0, (rank, rc, err)


def test_fdshare_missing_rank_is_reported_within_the_limit(tmp_path):
    import time
    t0 = time.time()
    res = _run_fdshare(3, [True] * 3, tmp_path, timeout_ms=1500, absent=(2,))
    assert time.time() - t0 < 30
    by_rank = {r[0]: r for r in res}
    assert by_rank[0][1] == -1 and "timed out waiting for 1 peer" in by_rank[0][4]
    assert by_rank[1][1] != 0          # rank 1 connected but never got a descriptor


# ---------------------------------------------------------------- the interposer in front of a stand-in NCCL, no GPU
def _fake_nccl_world(tmp_path):
    native = ROOT / "tests" / "native"
    lib = tmp_path / "libnccl.so.2"
    app = tmp_path / "nccl_app"
    subprocess.run(["gcc", "-shared", "-fPIC", "-Wall", "-Wextra", "-Werror", "-Wl,-soname,libnccl.so.2", str(native / "fake_nccl.c"), "-o", str(lib)], check=True)
    subprocess.run(["gcc", "-Wall", "-Wextra", "-Werror", str(native / "nccl_app.c"), "-o", str(app), f"-L{tmp_path}", "-l:libnccl.so.2", f"-Wl,-rpath,{tmp_path}"], check=True)
    return app


def _run_app(app, **env):
    e = dict(os.environ, LD_PRELOAD=str(_so()), PICCL_LOG="1", PICCL_TIMEOUT_MS="2000")
    e.pop("CUDA_VISIBLE_DEVICES", None)
    e.update(env)
    return subprocess.run([str(app)], env=e, capture_output=True, text=True, timeout=120)


def test_unset_algorithms_pass_every_call_to_the_real_library(tmp_path):
    """Reference behaviour: no PICCL_<COLL>_ALGO -> real NCCL (src/piccl.c:53-57 and the like)."""
    app = _fake_nccl_world(tmp_path)
    r = _run_app(app)
    assert r.returncode == 0 and "init=0" in r.stdout and "collectives=0 async=0/0" in r.stdout and "destroy=0" in r.stdout, r.stdout + r.stderr
    assert "FAKE_NCCL allreduce=2 allgather=2 reduce_scatter=2 reduce=2 broadcast=2 init=1 destroy=1 group=1" in r.stdout
    assert "allreduce: 0 fused, 2 passed to NCCL" in r.stderr and "broadcast: 0 fused, 2 passed to NCCL" in r.stderr


def test_a_communicator_the_executor_cannot_serve_falls_back_without_breaking_the_application(tmp_path):
    """Algorithms set, but (a) a one-rank communicator, (b) several ranks on a machine where CUDA cannot be initialised:
    the set-up fails on the host, every call still reaches the real library and returns success."""
    app = _fake_nccl_world(tmp_path)
    algos = {f"PICCL_{c}_ALGO": "RING" for c in ("ALLREDUCE", "ALLGATHER", "REDUCE_SCATTER", "REDUCE", "BROADCAST")}
    r = _run_app(app, **algos)
    assert r.returncode == 0 and "collectives=0" in r.stdout, r.stdout + r.stderr
    assert "FAKE_NCCL allreduce=2 allgather=2 reduce_scatter=2 reduce=2 broadcast=2" in r.stdout
    assert "allreduce: 0 fused, 2 passed to NCCL" in r.stderr
    import torch
    if torch.cuda.is_available():
        assert "communicator with 1 ranks: NCCL is used" in r.stderr
    else:
        # no usable CUDA device: the set-up is not even attempted (the stream cannot be queried), with any rank count
        r = _run_app(app, FAKE_NCCL_RANKS="4", **algos)
        assert r.returncode == 0 and "collectives=0" in r.stdout, r.stdout + r.stderr
        assert "FAKE_NCCL allreduce=2 allgather=2 reduce_scatter=2 reduce=2 broadcast=2" in r.stdout
        assert "allreduce: 0 fused, 2 passed to NCCL" in r.stderr


def test_the_set_up_is_decided_by_the_first_intercepted_call_whatever_its_count(tmp_path):
    """The set-up of a communicator is a collective of its own, so every rank must start it at the same call: the first one
    intercepted, even when this rank passes zero elements (which then goes to NCCL as before)."""
    app = _fake_nccl_world(tmp_path)
    r = _run_app(app, PICCL_ALLREDUCE_ALGO="RING", FAKE_NCCL_RANKS="4", NCCL_APP_ZERO_FIRST="1")
    assert r.returncode == 0 and "collectives=0" in r.stdout, r.stdout + r.stderr
    import re
    assert re.search(r"first intercepted call:? \(?allgather, count 0", r.stderr), r.stderr
    assert "FAKE_NCCL allreduce=2 allgather=3" in r.stdout          # the empty call itself still reached the library


def test_a_handle_that_comes_back_from_a_split_gets_fresh_state(tmp_path):
    """ncclCommFinalize drops what the interposer holds for a communicator; when a later ncclCommSplit hands out the same
    address, the decision is made again for the new communicator instead of reusing the dead one's."""
    app = _fake_nccl_world(tmp_path)
    r = _run_app(app, PICCL_ALLREDUCE_ALGO="RING", FAKE_NCCL_RANKS="4", NCCL_APP_SPLIT="1")
    assert r.returncode == 0 and "collectives=0" in r.stdout, r.stdout + r.stderr
    assert r.stderr.count("first intercepted call") == 2, r.stderr
    assert "FAKE_NCCL allreduce=3" in r.stdout
