"""Fused executor on one GPU: n virtual ranks in one cooperative launch, compared
with a plain PyTorch fp32 reference of the same collective."""
import itertools

import pytest
import torch

pytestmark = pytest.mark.gpu

ALGOS = ["RING", "K_RING", "RD", "RM", "PRD", "PRM", "DIRECT"]


@pytest.fixture(scope="module")
def groups():
    from piccl_b200.parallel.comm import LoopbackGroup, make_config
    cache = {}

    def get(n):
        if n not in cache:
            # small slots so that multi-segment pipelining is exercised with little data
            cache[n] = LoopbackGroup(n, config=make_config(max_cta=8, nslot=2, slot_bytes=4096, scratch_bytes=1 << 20, timeout_ms=5000))
        return cache[n]

    yield get
    for g in cache.values():
        g.close()


def _inputs(n, count, dtype, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype in (torch.int32, torch.int64):
        return [torch.randint(-1000, 1001, (count,), generator=g, device="cuda", dtype=dtype) for _ in range(n)]
    return [(torch.rand(count, generator=g, device="cuda", dtype=torch.float32) * 2 - 1).to(dtype) for _ in range(n)]


def _ref_reduce(xs, op):
    st = torch.stack([x.double() if x.dtype in (torch.int32, torch.int64) else x.float() for x in xs])
    if op == "sum":
        return st.sum(0)
    if op == "prod":
        return st.prod(0)
    if op == "max":
        return st.max(0).values
    if op == "min":
        return st.min(0).values
    return st.mean(0)


def _tol(dtype, n):
    return {torch.float32: 1e-5 * n, torch.float64: 1e-5 * n, torch.bfloat16: 2e-2, torch.float16: 2e-3}.get(dtype, 0.0)


def _check_ok(g):
    torch.cuda.synchronize()
    st = g.status()
    assert st.aborted == 0, f"device wait gave up: code {st.code} rank {st.rank} cta {st.cta} action {st.action} peer {st.peer} seg {st.segment}"


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("algo", ALGOS)
def test_allreduce_fp32(groups, n, algo):
    g = groups(n)
    for count, k in itertools.product([1, 7, 1024, 40000], [2, 4]):
        xs = _inputs(n, count, torch.float32)
        outs = [torch.full_like(x, float("nan")) for x in xs]
        g.run("allreduce", xs, outs, count, op="sum", algo=algo, k=k)
        _check_ok(g)
        ref = _ref_reduce(xs, "sum")
        for r in range(n):
            assert torch.allclose(outs[r].float(), ref, atol=_tol(torch.float32, n), rtol=0), f"n={n} {algo} k={k} count={count} rank {r}"
        # all ranks hold bit-identical results
        for r in range(1, n):
            assert torch.equal(outs[r], outs[0])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.int32, torch.float64, torch.int64])
@pytest.mark.parametrize("op", ["sum", "max", "min", "prod"])
def test_allreduce_dtypes_ops_in_place(groups, dtype, op):
    n = 4
    g = groups(n)
    for algo in ["RING", "PRD", "PRM"]:
        count = 3001
        xs = _inputs(n, count, dtype, seed=1)
        if op == "prod":
            xs = [(x.float().abs() * 0.05 + 0.98).to(dtype) if dtype.is_floating_point else (x % 2 + 1) for x in xs]
        ref = _ref_reduce(xs, op)
        bufs = [x.clone() for x in xs]
        g.run("allreduce", bufs, bufs, count, op=op, algo=algo, k=4)
        _check_ok(g)
        for r in range(n):
            got = bufs[r].double() if not dtype.is_floating_point else bufs[r].float()
            tol = _tol(dtype, n) * (4 if op in ("sum", "prod") else 1)
            assert torch.allclose(got, ref.to(got.dtype), atol=tol, rtol=tol), f"{dtype} {op} {algo} rank {r}"


def test_allreduce_avg(groups):
    n = 4
    g = groups(n)
    xs = _inputs(n, 5000, torch.float32, seed=2)
    outs = [torch.empty_like(x) for x in xs]
    for algo in ["RING", "PRD", "PRM"]:
        g.run("allreduce", xs, outs, 5000, op="avg", algo=algo, k=2)
        _check_ok(g)
        assert torch.allclose(outs[1], _ref_reduce(xs, "avg"), atol=1e-5)


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("algo", ALGOS)
def test_allgather(groups, n, algo):
    g = groups(n)
    for count, k, dtype in [(1, 2, torch.float32), (1000, 4, torch.bfloat16), (5003, 2, torch.int32), (33333, 8, torch.uint8)]:
        if dtype == torch.uint8:
            xs = [torch.randint(0, 255, (count,), device="cuda", dtype=dtype) for _ in range(n)]
        else:
            xs = _inputs(n, count, dtype, seed=3)
        outs = [torch.zeros(n * count, device="cuda", dtype=dtype) for _ in range(n)]
        g.run("allgather", xs, outs, count, algo=algo, k=k)
        _check_ok(g)
        ref = torch.cat(xs)
        for r in range(n):
            assert torch.equal(outs[r], ref), f"n={n} {algo} k={k} count={count} rank {r}"
    # in place: the send buffer is the rank's own block of the receive buffer
    count = 2048
    outs = [torch.zeros(n * count, device="cuda") for _ in range(n)]
    xs = []
    for r in range(n):
        outs[r][r * count:(r + 1) * count] = torch.arange(count, device="cuda") + 10000 * r
        xs.append(outs[r][r * count:(r + 1) * count])
    ref = torch.cat([x.clone() for x in xs])
    g.run("allgather", xs, outs, count, algo=algo, k=2)
    _check_ok(g)
    for r in range(n):
        assert torch.equal(outs[r], ref)


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("algo", ALGOS)
def test_reduce_scatter(groups, n, algo):
    g = groups(n)
    for count, k in [(1, 2), (999, 4), (20000, 2)]:
        xs = _inputs(n, n * count, torch.float32, seed=4)
        outs = [torch.zeros(count, device="cuda") for _ in range(n)]
        g.run("reduce_scatter", xs, outs, count, op="sum", algo=algo, k=k)
        _check_ok(g)
        ref = _ref_reduce(xs, "sum")
        for r in range(n):
            assert torch.allclose(outs[r], ref[r * count:(r + 1) * count], atol=_tol(torch.float32, n)), f"n={n} {algo} k={k} count={count} rank {r}"


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("algo", ALGOS)
def test_broadcast_and_reduce(groups, n, algo):
    g = groups(n)
    for count, root, k in [(5, 0, 2), (4097, n - 1, 4), (30000, n // 2, 2)]:
        xs = _inputs(n, count, torch.float32, seed=5)
        outs = [torch.zeros(count, device="cuda") for _ in range(n)]
        g.run("broadcast", xs, outs, count, root=root, algo=algo, k=k)
        _check_ok(g)
        for r in range(n):
            assert torch.equal(outs[r], xs[root]), f"bcast n={n} {algo} root={root} rank {r}"
        outs = [torch.full((count,), -5.0, device="cuda") for _ in range(n)]
        g.run("reduce", xs, outs, count, op="sum", root=root, algo=algo, k=k)
        _check_ok(g)
        assert torch.allclose(outs[root], _ref_reduce(xs, "sum"), atol=_tol(torch.float32, n))
        for r in range(n):
            if r != root:
                assert torch.all(outs[r] == -5.0), "non-root receive buffer must stay untouched"


def test_unaligned_buffers(groups):
    n = 4
    g = groups(n)
    count = 1237
    base = [torch.zeros(count + 8, device="cuda") for _ in range(n)]
    xs = [b[1:1 + count] for b in base]           # 4-byte aligned only
    for i, x in enumerate(xs):
        x.copy_(torch.arange(count, device="cuda") * 0.001 + i)
    outs_base = [torch.zeros(count + 8, device="cuda") for _ in range(n)]
    outs = [b[3:3 + count] for b in outs_base]
    g.run("allreduce", xs, outs, count, op="sum", algo="RING")
    _check_ok(g)
    ref = _ref_reduce([x.clone() for x in xs], "sum")
    for r in range(n):
        assert torch.allclose(outs[r], ref, atol=1e-4)
        assert outs_base[r][:3].abs().sum() == 0 and outs_base[r][3 + count:].abs().sum() == 0


def test_program_cache_and_stats(groups):
    n = 2
    g = groups(n)
    xs = _inputs(n, 4096, torch.float32)
    outs = [torch.empty_like(x) for x in xs]
    before = g.stats(0)
    for _ in range(3):
        g.run("allreduce", xs, outs, 4096, algo="RING")      # FIFO path: compiled programs are cached
    _check_ok(g)
    after = g.stats(0)
    assert after.calls[1] - before.calls[1] == 3
    assert after.program_cache_hits - before.program_cache_hits >= 2
    assert after.launches - before.launches == 3


def test_low_latency_path_matches_fifo_path(groups):
    # small exchange-type all-reduces run the flag-in-data kernel, large ones the FIFO executor: same values
    n = 8
    g = groups(n)
    for algo, k in [("PRD", 2), ("PRM", 8), ("RM", 4), ("RD", 2)]:
        for dtype in (torch.float32, torch.bfloat16):
            small = _inputs(n, 2000, dtype, seed=9)                       # 4-8 KB: low-latency kernel
            outs = [torch.empty_like(x) for x in small]
            before = g.stats(0).program_cache_misses + g.stats(0).program_cache_hits
            g.run("allreduce", small, outs, 2000, algo=algo, k=k)
            _check_ok(g)
            assert g.stats(0).program_cache_misses + g.stats(0).program_cache_hits == before, "expected the low-latency kernel"
            ref = _ref_reduce(small, "sum")
            tol = _tol(dtype, n) * 4
            for r in range(n):
                assert torch.allclose(outs[r].float(), ref, atol=tol, rtol=tol), f"{algo} {dtype} rank {r}"
                assert torch.equal(outs[r], outs[0])


@pytest.mark.parametrize("n", [2, 3, 8])
def test_low_latency_exchange_kernels(groups, n):
    """Small all-gather / reduce-scatter with a one-exchange schedule (DIRECT, PRM with radix = rank count) run the flag-in-data
    kernels of ll_exchange.cu; mixed with low-latency all-reduces back to back, no synchronisation, they share slots and epochs."""
    g = groups(n)
    launches0 = g.stats().launches
    for rep in range(3):
        results = []
        for dtype, op, count in [(torch.float32, "sum", 777), (torch.bfloat16, "avg", 4099), (torch.int32, "max", 1), (torch.float16, "min", 3000), (torch.float64, "prod", 17)]:
            xs = _inputs(n, n * count, dtype, seed=50 + rep)
            if op == "prod":
                xs = [x * 0 + 1 + 0.01 * (r + 1) for r, x in enumerate(xs)]
            outs = [torch.zeros(count, device="cuda", dtype=dtype) for _ in range(n)]
            g.run("reduce_scatter", xs, outs, count, op=op, algo="DIRECT")
            results.append(("rs", dtype, op, count, xs, outs))
            ys = _inputs(n, count, dtype, seed=60 + rep)
            gath = [torch.zeros(n * count, device="cuda", dtype=dtype) for _ in range(n)]
            g.run("allgather", ys, gath, count, algo="PRM", k=8 if n == 8 else n)
            results.append(("ag", dtype, op, count, ys, gath))
            zs = _inputs(n, count, dtype, seed=70 + rep)
            red = [torch.zeros_like(z) for z in zs]
            g.run("allreduce", zs, red, count, op="sum", algo="PRD" if n != 3 else "RING")
            results.append(("ar", dtype, "sum", count, zs, red))
        _check_ok(g)
        for kind, dtype, op, count, xs, outs in results:
            if kind == "ag":
                for r in range(n):
                    assert torch.equal(outs[r], torch.cat(xs)), f"allgather {dtype} {count} rank {r}"
            elif kind == "rs":
                ref = _ref_reduce(xs, op)
                for r in range(n):
                    got = outs[r].double() if dtype in (torch.int32, torch.int64) else outs[r].float()
                    assert torch.allclose(got, ref[r * count:(r + 1) * count].to(got.dtype), atol=_tol(dtype, n), rtol=2e-2), f"reduce_scatter {dtype} {op} {count} rank {r}"
            else:
                ref = _ref_reduce(xs, "sum")
                got = outs[0].double() if dtype in (torch.int32, torch.int64) else outs[0].float()
                assert torch.allclose(got, ref.to(got.dtype), atol=_tol(dtype, n) * 4, rtol=2e-2), f"allreduce {dtype} {count}"
    # unaligned user buffers and an odd number of bytes per rank
    base = [torch.arange(1, 1 + n * 1001 + 1, device="cuda", dtype=torch.uint8) + r for r in range(n)]
    xs = [b[1:1002] for b in base]
    outs_base = [torch.zeros(n * 1001 + 3, device="cuda", dtype=torch.uint8) for _ in range(n)]
    outs = [o[3:] for o in outs_base]
    g.run("allgather", xs, outs, 1001, algo="DIRECT")
    _check_ok(g)
    for r in range(n):
        assert torch.equal(outs[r], torch.cat(xs))
    # every call above was one launch
    assert g.stats().launches - launches0 == 3 * 15 + 1


def test_persistent_launcher_serves_and_leaves():
    # separate process: the launch mode is read from the environment when the library is loaded
    import os
    import subprocess
    import sys
    from pathlib import Path
    env = dict(os.environ, PICCL_LAUNCH="persistent", PICCL_PERSIST_IDLE_US="300")
    r = subprocess.run([sys.executable, str(Path(__file__).parent / "persistent_worker.py")], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "PERSISTENT_OK 45" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_bounded_wait_reports_instead_of_hanging():
    # a wait for data nobody sends runs into its limit; the kernel returns, the status says where
    from piccl_b200.parallel.comm import LoopbackGroup, make_config
    import ctypes as C
    from piccl_b200 import _native as N
    g = LoopbackGroup(1, config=make_config(max_cta=2, nslot=2, slot_bytes=4096, scratch_bytes=1 << 16, timeout_ms=300))
    lib = N.lib()
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    N.check(lib.piccl_test_unmatched_wait(g._hs[0], 300, torch.cuda.current_stream().cuda_stream), "unmatched wait")
    t1.record()
    torch.cuda.synchronize()
    st = g.status()
    assert st.aborted == 1 and st.code == 2 and st.peer == 0 and st.want == 1 and st.have == 0
    assert 250 < t0.elapsed_time(t1) < 3000
    # the communicator refuses further work instead of running on inconsistent counters
    x = torch.ones(16, device="cuda")
    with pytest.raises(N.PicclError):
        g.run("allreduce", [x], [x], 16)
    # the context is still usable
    assert float((x + 1).sum()) == 32.0
    g.close()
