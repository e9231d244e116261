"""Worker of the multi-process tests (launched with torch.distributed.run by test_multigpu.py).
Each case prints 'WORKER_OK <case>' on success on every rank."""
import ctypes as C
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

ALGOS = ["RING", "K_RING", "RD", "RM", "PRD", "PRM", "DIRECT"]


def setup():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world


def rand(count, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype == torch.int32:
        return torch.randint(-1000, 1001, (count,), generator=g, device="cuda", dtype=dtype)
    return (torch.rand(count, generator=g, device="cuda") * 2 - 1).to(dtype)


def tol(dtype, n):
    return {torch.float32: 1e-5 * n, torch.bfloat16: 4e-2, torch.float16: 4e-3}.get(dtype, 0)


def healthy(comm):
    torch.cuda.synchronize()
    st = comm.status()
    assert st.aborted == 0, f"wait gave up: code {st.code} rank {st.rank} cta {st.cta} action {st.action} peer {st.peer} seg {st.segment}"


def case_collectives(rank, world):
    from piccl_b200.parallel.comm import Communicator, make_config
    comm = Communicator(config=make_config(timeout_ms=20000))
    for algo in ALGOS:
        for dtype, count, k in [(torch.float32, 1, 2), (torch.bfloat16, 4099, 4), (torch.float32, 1 << 20, 2), (torch.int32, 300001, 8)]:
            x = rand(count, dtype, 100 + rank)
            want = x.clone()
            dist.all_reduce(want)
            got = comm.all_reduce(x.clone(), algo=algo, k=k)
            healthy(comm)
            assert torch.allclose(got.float(), want.float(), atol=tol(dtype, world), rtol=1e-2 if dtype != torch.int32 else 0), f"allreduce {algo} {dtype} {count}"
            # allgather
            out = torch.empty(world * count, dtype=dtype, device="cuda")
            ref = torch.empty_like(out)
            dist.all_gather_into_tensor(ref, x)
            comm.all_gather(x, out, algo=algo, k=k)
            healthy(comm)
            assert torch.equal(out, ref), f"allgather {algo} {dtype} {count}"
            # reduce_scatter
            big = rand(world * count, dtype, 200 + rank)
            rs_ref = torch.empty(count, dtype=dtype, device="cuda")
            dist.reduce_scatter_tensor(rs_ref, big.clone())
            rs = torch.empty(count, dtype=dtype, device="cuda")
            comm.reduce_scatter(big, rs, algo=algo, k=k)
            healthy(comm)
            assert torch.allclose(rs.float(), rs_ref.float(), atol=tol(dtype, world), rtol=1e-2 if dtype != torch.int32 else 0), f"reduce_scatter {algo} {dtype} {count}"
            # broadcast / reduce with a non-zero root
            root = world - 1
            b = x.clone()
            bref = x.clone()
            dist.broadcast(bref, src=root)
            comm.broadcast(b, root=root, algo=algo, k=k)
            healthy(comm)
            assert torch.equal(b, bref), f"broadcast {algo}"
            r_ref = x.clone()
            dist.reduce(r_ref, dst=root)
            r_out = torch.zeros_like(x)
            comm.reduce(x, r_out, root=root, algo=algo, k=k)
            healthy(comm)
            if rank == root:
                assert torch.allclose(r_out.float(), r_ref.float(), atol=tol(dtype, world), rtol=1e-2 if dtype != torch.int32 else 0), f"reduce {algo}"
    # a large message through every FIFO slot several times, AUTO selection, avg
    x = rand(48 << 20, torch.bfloat16, 7 + rank)
    want = x.clone()
    dist.all_reduce(want, op=dist.ReduceOp.AVG)
    got = comm.all_reduce(x, op="avg", algo="AUTO")
    healthy(comm)
    assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    dist.barrier()
    comm.close()


def case_ddp(rank, world):
    from piccl_b200.models.gpt2 import GPT2Config
    from piccl_b200.parallel.comm import Communicator
    from piccl_b200.train import DataParallelTrainer
    comm = Communicator()
    cfg = GPT2Config.tiny()
    tr = DataParallelTrainer(cfg, comm, bucket_bytes=256 * 1024, algo="RING")
    g = torch.Generator().manual_seed(rank)
    tok = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len + 1), generator=g).cuda()
    a, b = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    # expected averaged gradient: local backward, then NCCL average
    tr.model.forward_backward(a, b)
    want = tr.model.flat_g.clone().float()
    dist.all_reduce(want, op=dist.ReduceOp.AVG)
    tr.averager.begin_step()
    tr.model.forward_backward(a, b, on_grads_ready=tr.averager.ready)
    tr.averager.finish()
    torch.cuda.synchronize()
    healthy(comm)
    assert tr.averager.launched >= 3
    got = tr.model.flat_g.float()
    rel = (got - want).norm() / want.norm()
    assert rel < 2e-2, float(rel)
    losses = [tr.step(a.cpu().pin_memory(), b.cpu().pin_memory()) for _ in range(6)]
    assert losses[-1] < losses[0]
    # parameters stay identical across ranks
    p = tr.model.flat_p.float()
    ref = p.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(p, ref)
    dist.barrier()
    comm.close()


def case_shim(rank, world):
    """Runs under LD_PRELOAD=piccl.so with PICCL_*_ALGO set: torch.distributed's own NCCL calls are intercepted."""
    lib = C.CDLL(os.environ["LD_PRELOAD"])
    x = rand(1 << 18, torch.float32, 5 + rank)
    exp = [rand(1 << 18, torch.float32, 5 + r) for r in range(world)]
    want = torch.stack(exp).sum(0)
    y = x.clone()
    dist.all_reduce(y)
    assert torch.allclose(y, want, atol=1e-4)
    z = x.to(torch.bfloat16)
    dist.all_reduce(z, op=dist.ReduceOp.AVG)
    assert torch.allclose(z.float(), torch.stack([e.to(torch.bfloat16).float() for e in exp]).mean(0), atol=2e-2)
    out = torch.empty(world * x.numel(), device="cuda")
    dist.all_gather_into_tensor(out, x)
    assert torch.equal(out, torch.cat(exp))
    b = x.clone()
    dist.broadcast(b, src=1)
    assert torch.equal(b, exp[1])
    rs = torch.empty(x.numel() // world, device="cuda")
    dist.reduce_scatter_tensor(rs, x.clone())
    n = x.numel() // world
    assert torch.allclose(rs, want[rank * n:(rank + 1) * n], atol=1e-4)
    torch.cuda.synchronize()
    native = (C.c_ulonglong * 5)()
    passed = (C.c_ulonglong * 5)()
    lib.piccl_shim_counters(native, passed)
    print(f"rank {rank} fused {list(native)} passed-through {list(passed)}", flush=True)
    expect_native = os.environ.get("EXPECT_NATIVE", "1") == "1"
    if expect_native:
        assert native[1] >= 2 and native[0] >= 1 and native[2] >= 1 and native[4] >= 1, list(native)
    else:
        assert sum(native) == 0
    dist.barrier()


def case_fault(rank, world):
    """Rank 1 omits one all-reduce on the host (PICCL_FAULT): rank 0's kernel gives up after the limit and
    reports which peer it waited for; nobody hangs, the CUDA context stays usable."""
    from piccl_b200 import _native as N
    from piccl_b200.parallel.comm import Communicator, make_config
    comm = Communicator(config=make_config(timeout_ms=500))
    x = torch.ones(4096, device="cuda")
    for _ in range(3):
        comm.all_reduce(x.clone(), algo="RING")
    healthy(comm)
    dist.barrier()
    comm.all_reduce(x.clone(), algo="RING")      # call index 3: skipped on rank 1
    torch.cuda.synchronize()
    st = comm.status()
    if rank == 0:
        assert st.aborted == 1 and st.peer == 1 and st.code == 2, (st.aborted, st.code, st.peer)
        try:
            comm.all_reduce(x.clone(), algo="RING")
            raise AssertionError("a broken communicator must refuse work")
        except N.PicclError:
            pass
    assert float((x * 2).sum()) == 8192.0
    dist.barrier()
    comm.close()


def case_tp(rank, world):
    """Fused GEMM->reduce-scatter and all-gather->GEMM across real GPUs against cuBLAS + NCCL."""
    from piccl_b200.parallel import tp
    from piccl_b200.parallel.comm import Communicator, make_config
    M, N, K = 256 * world * 2, 1024, 512
    M3, N3, K3 = 128 * world, 512, 256                          # a second, smaller GEMM -> reduce-scatter shape
    ws = max(tp.workspace_bytes("gemm_rs", world, M, N, K), tp.workspace_bytes("ag_gemm", world, M, N, K))
    comm = Communicator(config=make_config(tp_bytes=ws, timeout_ms=20000))
    g = torch.Generator(device="cuda").manual_seed(50 + rank)
    A = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    B = (torch.randn(N, K, generator=g, device="cuda") * 0.1).to(torch.bfloat16)
    out = torch.empty(M // world, N, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        tp.gemm_rs(comm, A, B, out)
    torch.cuda.synchronize()
    assert tp.tp_status(comm) == 0
    part = (A @ B.t())
    ref = torch.empty_like(out)
    dist.reduce_scatter_tensor(ref, part)
    tol = 0.03 * ref.float().abs().max().item() + 0.05
    assert torch.allclose(out.float(), ref.float(), atol=tol, rtol=3e-2), (out.float() - ref.float()).abs().max().item()
    # all-gather -> GEMM
    As = torch.randn(M // world, K, generator=g, device="cuda").to(torch.bfloat16)
    out2 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        tp.ag_gemm(comm, As, B, out2)
    torch.cuda.synchronize()
    assert tp.tp_status(comm) == 0
    full = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
    dist.all_gather_into_tensor(full, As)
    ref2 = full @ B.t()
    tol = 0.03 * ref2.float().abs().max().item() + 0.05
    assert torch.allclose(out2.float(), ref2.float(), atol=tol, rtol=3e-2), (out2.float() - ref2.float()).abs().max().item()
    # the two kernels and two shapes alternating on one stream with no host synchronisation in between
    A3 = torch.randn(M3, K3, generator=g, device="cuda").to(torch.bfloat16)
    B3 = (torch.randn(N3, K3, generator=g, device="cuda") * 0.1).to(torch.bfloat16)
    out3 = torch.empty(M3 // world, N3, device="cuda", dtype=torch.bfloat16)
    out.fill_(float("nan")); out2.fill_(float("nan"))
    for _ in range(5):
        tp.ag_gemm(comm, As, B, out2)
        tp.gemm_rs(comm, A, B, out)
        tp.gemm_rs(comm, A3, B3, out3)
    torch.cuda.synchronize()
    assert tp.tp_status(comm) == 0
    ref3 = torch.empty_like(out3)
    dist.reduce_scatter_tensor(ref3, A3 @ B3.t())
    assert torch.allclose(out.float(), ref.float(), atol=0.03 * ref.float().abs().max().item() + 0.05, rtol=3e-2)
    assert torch.allclose(out2.float(), ref2.float(), atol=0.03 * ref2.float().abs().max().item() + 0.05, rtol=3e-2)
    assert torch.allclose(out3.float(), ref3.float(), atol=0.03 * ref3.float().abs().max().item() + 0.05, rtol=3e-2)
    dist.barrier()
    comm.close()


def case_nvls(rank, world):
    """Every collective through the NVSwitch (algorithm NVLS: multimem load-reduce, multicast stores) against NCCL."""
    from piccl_b200.parallel.comm import Communicator, make_config
    comm = Communicator(config=make_config(timeout_ms=20000))
    probe = torch.ones(1024, device="cuda")
    comm.all_reduce(probe, algo="NVLS")
    torch.cuda.synchronize()
    if comm.stats().nvls_calls == 0:
        assert torch.equal(probe, torch.full_like(probe, float(world)))      # a peer-to-peer schedule ran instead
        print("NVLS_UNAVAILABLE", flush=True)
    else:
        calls = 1
        for dtype, count in [(torch.float32, 1), (torch.float32, 1000), (torch.bfloat16, (1 << 20) + 3), (torch.float16, 300001), (torch.float32, 48 << 20)]:
            for op in ("sum", "avg") if dtype == torch.float32 else ("sum", "avg", "max"):
                x = rand(count, dtype, 300 + rank)
                want = x.clone()
                dist.all_reduce(want, op={"sum": dist.ReduceOp.SUM, "avg": dist.ReduceOp.AVG, "max": dist.ReduceOp.MAX}[op])
                got = comm.all_reduce(x.clone(), op=op, algo="NVLS")
                calls += 1
                healthy(comm)
                assert torch.allclose(got.float(), want.float(), atol=tol(dtype, world), rtol=1e-2), f"nvls {op} {dtype} {count}: {(got.float() - want.float()).abs().max().item()}"
        # every rank ends with the same bits
        x = rand(1 << 20, torch.bfloat16, 400 + rank)
        got = comm.all_reduce(x, algo="NVLS")
        calls += 1
        ref = got.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(got, ref)
        # the other collectives, interleaved; blocks of 16 bytes, of 1 MiB + 16 bytes and of 24 MiB
        for dtype, count in [(torch.float32, 4), (torch.bfloat16, (1 << 19) + 8), (torch.float32, 6 << 20)]:
            x = rand(count, dtype, 500 + rank)
            out = torch.empty(world * count, dtype=dtype, device="cuda")
            ref = torch.empty_like(out)
            dist.all_gather_into_tensor(ref, x)
            comm.all_gather(x, out, algo="NVLS")
            healthy(comm)
            assert torch.equal(out, ref), f"nvls allgather {dtype} {count}"
            big = rand(world * count, dtype, 600 + rank)
            rs_ref = torch.empty(count, dtype=dtype, device="cuda")
            dist.reduce_scatter_tensor(rs_ref, big.clone())
            rs = torch.empty(count, dtype=dtype, device="cuda")
            comm.reduce_scatter(big, rs, algo="NVLS")
            healthy(comm)
            assert torch.allclose(rs.float(), rs_ref.float(), atol=tol(dtype, world), rtol=1e-2), f"nvls reduce_scatter {dtype} {count}"
            root = world - 1
            b = x.clone()
            bref = x.clone()
            dist.broadcast(bref, src=root)
            comm.broadcast(b, root=root, algo="NVLS")
            healthy(comm)
            assert torch.equal(b, bref), f"nvls broadcast {dtype} {count}"
            r_ref = x.clone()
            dist.reduce(r_ref, dst=root)
            r_out = torch.zeros_like(x)
            comm.reduce(x, r_out, root=root, algo="NVLS")
            healthy(comm)
            if rank == root:
                assert torch.allclose(r_out.float(), r_ref.float(), atol=tol(dtype, world), rtol=1e-2), f"nvls reduce {dtype} {count}"
            calls += 4
        assert comm.stats().nvls_calls == calls, (comm.stats().nvls_calls, calls)
        # AUTO takes the switch for large messages from four ranks on
        x = rand(8 << 20, torch.bfloat16, 700 + rank)
        want = x.clone()
        dist.all_reduce(want, op=dist.ReduceOp.AVG)
        got = comm.all_reduce(x, op="avg", algo="AUTO")
        healthy(comm)
        assert comm.stats().nvls_calls == calls + (1 if world >= 4 else 0)
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        # replay from a CUDA graph: the use counters live in device memory
        x = torch.randn(1 << 20, device="cuda")
        out = torch.empty_like(x)
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            comm.all_reduce(x, out, algo="NVLS", stream=s)
            s.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=s):
                comm.all_reduce(x, out, algo="NVLS", stream=s)
            for i in range(3):
                x.fill_(float(i + rank))
                graph.replay()
                s.synchronize()
                assert torch.equal(out, torch.full_like(out, float(world * i + world * (world - 1) // 2)))
        healthy(comm)
    dist.barrier()
    comm.close()


if __name__ == "__main__":
    case = sys.argv[1]
    rank, world = setup()
    {"collectives": case_collectives, "ddp": case_ddp, "shim": case_shim, "fault": case_fault, "tp": case_tp, "nvls": case_nvls}[case](rank, world)
    print(f"WORKER_OK {case} rank {rank}", flush=True)
    dist.destroy_process_group()
