"""The per-rank action programs executed by real processes over gloo (world size 4 and 3), compared with
torch.distributed's own collectives."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
ALGOS = ["RING", "K_RING", "RD", "RM", "PRD", "PRM", "DIRECT"]


def _worker(rank, world, port, q):
    try:
        sys.path.insert(0, str(ROOT))
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from piccl_b200.parallel.host_exec import host_collective
        count = 37
        for algo in ALGOS:
            for k in (2, 3):
                g = torch.Generator().manual_seed(1000 + rank)
                x = torch.randint(-50, 50, (count,), generator=g, dtype=torch.int64)
                # allreduce
                want = x.clone(); dist.all_reduce(want)
                out = torch.zeros(count, dtype=torch.int64)
                host_collective("allreduce", algo, x, out, count, k=k)
                assert torch.equal(out, want), ("allreduce", algo, k)
                # allgather
                ref = [torch.zeros(count, dtype=torch.int64) for _ in range(world)]
                dist.all_gather(ref, x)
                out = torch.zeros(world * count, dtype=torch.int64)
                host_collective("allgather", algo, x, out, count, k=k)
                assert torch.equal(out, torch.cat(ref)), ("allgather", algo, k)
                # reduce_scatter (max)
                big = torch.randint(-50, 50, (world * count,), generator=g, dtype=torch.int64)
                full = big.clone(); dist.all_reduce(full, op=dist.ReduceOp.MAX)
                out = torch.zeros(count, dtype=torch.int64)
                host_collective("reduce_scatter", algo, big, out, count, k=k, op="max")
                assert torch.equal(out, full[rank * count:(rank + 1) * count]), ("reduce_scatter", algo, k)
                # broadcast / reduce, root = last rank
                root = world - 1
                b = x.clone(); dist.broadcast(b, src=root)
                out = torch.zeros(count, dtype=torch.int64)
                host_collective("broadcast", algo, x, out, count, k=k, root=root)
                assert torch.equal(out, b), ("broadcast", algo, k)
                r = x.clone(); dist.reduce(r, dst=root)
                out = torch.full((count,), -7, dtype=torch.int64)
                host_collective("reduce", algo, x, out, count, k=k, root=root)
                if rank == root:
                    assert torch.equal(out, r), ("reduce", algo, k)
                else:
                    assert torch.all(out == -7)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"{type(e).__name__}: {e}"))


@pytest.mark.parametrize("world,port", [(4, 29671), (3, 29672)])
def test_programs_over_gloo(world, port):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    for _ in range(world):
        results.append(q.get(timeout=240))
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()       # this exact child
    assert all(msg == "ok" for _, msg in results), results


def _fault_worker(rank, world, port, q):
    import datetime
    import time
    try:
        sys.path.insert(0, str(ROOT))
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
        from piccl_b200.parallel.host_exec import host_collective
        x = torch.ones(16)
        out = torch.zeros(16)
        host_collective("allreduce", "RING", x, out, 16)          # a healthy call first
        assert torch.all(out == world)
        if rank == 1:
            q.put((rank, "left"))                                  # this rank never joins the next collective
            time.sleep(8)
            return
        t0 = time.time()
        try:
            host_collective("allreduce", "RING", x, out, 16)
            q.put((rank, "no error"))
        except Exception as e:  # noqa: BLE001
            q.put((rank, f"error after {time.time() - t0:.1f}s: {type(e).__name__}"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"setup failed: {type(e).__name__}: {e}"))


def test_rank_that_never_joins_is_reported_within_the_time_limit():
    """Failure made on the host, no GPU involved: one of two ranks skips a collective; the other one's receive
    ends with an error when the process-group time limit runs out instead of waiting for ever."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_fault_worker, args=(r, 2, 29673, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.terminate()
    assert results[1] == "left"
    assert results[0].startswith("error after"), results
    assert float(results[0].split()[2].rstrip("s:")) < 30
