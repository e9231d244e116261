"""Fused tensor-parallel kernels against the unfused cuBLAS + NCCL path (run under torch.distributed.run).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/tp_bench.py

Shapes of the baseline configuration: GEMM->reduce-scatter [M=8192, K=28672/n] x [K/n, N=8192]; all-gather->GEMM
gathers [8192/n, 8192] shards and multiplies by [8192, 28672/n].  bf16, weights ~N(0, 0.02), activations ~N(0, 1).
Times are CUDA-event medians of 20 iterations after 5 warm-ups, maximum over ranks; inputs (>= 100 MB per operand)
exceed the L2.  Roofline = max(FLOPs / measured bf16 peak, bytes over NVLink per rank / 770 GB/s measured copy rate).
"""
from __future__ import annotations

import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from piccl_b200.parallel import tp  # noqa: E402
from piccl_b200.parallel.comm import Communicator, make_config  # noqa: E402


def timed(fn, iters=20, warmup=5):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record(); torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    M, N, Kfull = 8192, 8192, 28672
    Kl = Kfull // world // 64 * 64
    peak = 1590.0
    p = ROOT / "MEASURED_PEAKS.json"
    src = "fallback"
    if p.exists():
        peak = float(json.loads(p.read_text())["bf16_tflops"]); src = "measured"
    ws = max(tp.workspace_bytes("gemm_rs", world, M, N, Kl), tp.workspace_bytes("ag_gemm", world, M, Kl, N))
    comm = Communicator(config=make_config(tp_bytes=ws))
    g = torch.Generator(device="cuda").manual_seed(rank)
    res = {}
    # ---- GEMM -> reduce-scatter
    A = torch.randn(M, Kl, generator=g, device="cuda").to(torch.bfloat16)
    B = (torch.randn(N, Kl, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.empty(M // world, N, device="cuda", dtype=torch.bfloat16)
    part = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ref = torch.empty_like(out)

    def unfused_rs():
        torch.mm(A, B.t(), out=part)
        dist.reduce_scatter_tensor(ref, part)

    t_f = timed(lambda: tp.gemm_rs(comm, A, B, out))
    t_u = timed(unfused_rs)
    ok = tp.tp_status(comm) == 0 and torch.allclose(out.float(), ref.float(), atol=0.03 * ref.float().abs().max().item() + 0.05, rtol=3e-2)
    flops = 2.0 * M * N * Kl
    nv_bytes = (world - 1) / world * M * N * 2
    roof = max(flops / (peak * 1e12), nv_bytes / 770e9) * 1e3
    res["gemm_rs"] = {"fused_ms": round(t_f, 4), "unfused_ms": round(t_u, 4), "speedup": round(t_u / t_f, 3), "tflops_per_gpu": round(flops / t_f / 1e9, 1),
                      "roofline_ms": round(roof, 4), f"fraction_of_{src}_roofline": round(roof / t_f, 3), "correct": bool(ok)}
    # ---- all-gather -> GEMM
    As = torch.randn(M // world, N, generator=g, device="cuda").to(torch.bfloat16)          # [M/n, K=8192]
    B2 = (torch.randn(Kl, N, generator=g, device="cuda") * 0.02).to(torch.bfloat16)          # [N_local, K]
    out2 = torch.empty(M, Kl, device="cuda", dtype=torch.bfloat16)
    full = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ref2 = torch.empty_like(out2)

    def unfused_ag():
        dist.all_gather_into_tensor(full, As)
        torch.mm(full, B2.t(), out=ref2)

    t_f = timed(lambda: tp.ag_gemm(comm, As, B2, out2))
    t_u = timed(unfused_ag)
    ok = tp.tp_status(comm) == 0 and torch.allclose(out2.float(), ref2.float(), atol=0.03 * ref2.float().abs().max().item() + 0.05, rtol=3e-2)
    roof = max(flops / (peak * 1e12), (world - 1) / world * M * N * 2 / 770e9) * 1e3
    res["ag_gemm"] = {"fused_ms": round(t_f, 4), "unfused_ms": round(t_u, 4), "speedup": round(t_u / t_f, 3), "tflops_per_gpu": round(flops / t_f / 1e9, 1),
                      "roofline_ms": round(roof, 4), f"fraction_of_{src}_roofline": round(roof / t_f, 3), "correct": bool(ok)}
    if rank == 0:
        print(json.dumps({"n_gpus": world, "M": M, "N": N, "K_local": Kl, **res}), flush=True)
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
