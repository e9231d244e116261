"""Small, self-terminating workloads for ncu captures (one kernel, a few launches, well under a few GB):

    python benchmarks/profile_cases.py exec      # fused collective executor: 2 virtual ranks, ring all-reduce of 256 MiB fp32
    python benchmarks/profile_cases.py exec_ll   # low-latency all-reduce, 8 virtual ranks, 16 KiB
    python benchmarks/profile_cases.py gemm      # tcgen05 GEMM 8192 x 8192 x 3584 bf16
    python benchmarks/profile_cases.py gemm_pair # the same product on CTA pairs (tcgen05.mma.cta_group::2); checks the result first
    python benchmarks/profile_cases.py direct    # DIRECT all-reduce, 8 virtual ranks, 16 MiB fp32
    python benchmarks/profile_cases.py tp        # fused GEMM -> reduce-scatter, 2 virtual ranks, 4096 x 4096 x 2048
    python benchmarks/profile_cases.py ln        # residual-add + LayerNorm forward/backward, 8192 x 1024
    python benchmarks/profile_cases.py ce        # cross entropy forward+backward, 8192 x 50304
    python benchmarks/profile_cases.py nvls      # in-switch all-reduce kernel with the switch emulated: 4 virtual ranks, 64 MiB bf16 each
    python benchmarks/profile_cases.py llf       # low-latency executor: all-gather of 16 KiB per rank, 8 virtual ranks
    python benchmarks/profile_cases.py ag_gemm   # fused all-gather -> GEMM, 2 virtual ranks, 4096 x 2048 x 4096
    python benchmarks/profile_cases.py elementwise  # AdamW on 128 Mi parameters, bias + GELU forward / backward on 8192 x 4096, embedding 8192 x 1024, column sum

Typical capture (after the same command has exited 0 without ncu):
    ncu --set full --clock-control none -k regex:<kernel> -s 2 -c 2 -o <name> python benchmarks/profile_cases.py <case>
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def case_exec(ll: bool = False):
    from piccl_b200.parallel.comm import LoopbackGroup
    n = 8 if ll else 2
    count = 4096 if ll else 64 << 20
    g = LoopbackGroup(n)
    xs = [torch.ones(count, device="cuda") for _ in range(n)]
    outs = [torch.empty_like(x) for x in xs]
    for _ in range(4):
        g.run("allreduce", xs, outs, count, algo="PRD" if ll else "RING")
    torch.cuda.synchronize()
    assert g.status().aborted == 0
    g.close()


def case_gemm():
    from piccl_b200.ops import gemm_sm100
    a = torch.randn(8192, 3584, device="cuda").to(torch.bfloat16)
    b = torch.randn(8192, 3584, device="cuda").to(torch.bfloat16)
    o = torch.empty(8192, 8192, device="cuda", dtype=torch.bfloat16)
    for _ in range(4):
        gemm_sm100.gemm_nt(a, b, o)
    torch.cuda.synchronize()


def case_gemm_pair():
    from piccl_b200.ops import gemm_sm100
    a = torch.randn(8192, 3584, device="cuda").to(torch.bfloat16)
    b = (torch.randn(8192, 3584, device="cuda") * 0.05).to(torch.bfloat16)
    o = torch.empty(8192, 8192, device="cuda", dtype=torch.bfloat16)
    gemm_sm100.gemm_nt_pair(a, b, o)
    st = gemm_sm100.pair_status()
    assert st == 0, f"a bounded wait ran out (role {st})"
    ref = torch.mm(a, b.t())
    err = (o.float() - ref.float()).abs().max().item()
    assert err < 0.05 * ref.float().abs().max().item(), err
    for _ in range(3):
        gemm_sm100.gemm_nt_pair(a, b, o)
    torch.cuda.synchronize()


def case_direct():
    from piccl_b200.parallel.comm import LoopbackGroup
    n, count = 8, 4 << 20
    g = LoopbackGroup(n)
    xs = [torch.full((count,), float(r + 1), device="cuda") for r in range(n)]
    outs = [torch.empty_like(x) for x in xs]
    for _ in range(4):
        g.run("allreduce", xs, outs, count, algo="DIRECT")
    torch.cuda.synchronize()
    assert g.status().aborted == 0 and float(outs[3][12345]) == n * (n + 1) / 2
    g.close()


def case_tp():
    from piccl_b200.parallel import tp
    from piccl_b200.parallel.comm import LoopbackGroup, make_config
    n, M, N, K = 2, 4096, 4096, 2048
    g = LoopbackGroup(n, config=make_config(tp_bytes=tp.workspace_bytes("gemm_rs", n, M, N, K)))
    As = [torch.randn(M, K, device="cuda").to(torch.bfloat16) for _ in range(n)]
    Bs = [torch.randn(N, K, device="cuda").to(torch.bfloat16) for _ in range(n)]
    outs = [torch.empty(M // n, N, device="cuda", dtype=torch.bfloat16) for _ in range(n)]
    for _ in range(4):
        tp.gemm_rs_group(g, As, Bs, outs)
    torch.cuda.synchronize()
    g.close()


def case_nvls():
    """The kernel of the in-switch collectives on one GPU: the multimem instructions are replaced by loops over the virtual
    ranks' windows, everything else (bulk copies, warp groups, counters) is what runs on NVLink multicast windows."""
    from piccl_b200.parallel.comm import LoopbackGroup
    n, count = 4, 32 << 20
    g = LoopbackGroup(n)
    xs = [torch.ones(count, device="cuda", dtype=torch.bfloat16) for _ in range(n)]
    outs = [torch.empty_like(x) for x in xs]
    for _ in range(3):
        g.run("allreduce", xs, outs, count, algo="NVLS")
    torch.cuda.synchronize()
    assert g.status().aborted == 0 and g.stats().nvls_calls == 3 and float(outs[1][777]) == float(n)
    g.close()


def case_llf():
    from piccl_b200.parallel.comm import LoopbackGroup
    n, count = 8, 4096
    g = LoopbackGroup(n)
    xs = [torch.full((count,), float(r), device="cuda") for r in range(n)]
    outs = [torch.empty(n * count, device="cuda") for _ in range(n)]
    for _ in range(4):
        g.run("allgather", xs, outs, count, algo="RING")
    torch.cuda.synchronize()
    assert g.status().aborted == 0 and float(outs[2][5 * count + 1]) == 5.0
    g.close()


def case_ag_gemm():
    from piccl_b200.parallel import tp
    from piccl_b200.parallel.comm import LoopbackGroup, make_config
    n, M, N, K = 2, 4096, 2048, 4096
    g = LoopbackGroup(n, config=make_config(tp_bytes=tp.workspace_bytes("ag_gemm", n, M, N, K)))
    As = [torch.randn(M // n, K, device="cuda").to(torch.bfloat16) for _ in range(n)]
    Bs = [torch.randn(N, K, device="cuda").to(torch.bfloat16) for _ in range(n)]
    outs = [torch.empty(M, N, device="cuda", dtype=torch.bfloat16) for _ in range(n)]
    for _ in range(4):
        tp.ag_gemm_group(g, As, Bs, outs)
    torch.cuda.synchronize()
    assert all(tp.tp_status(h) == 0 for h in g._hs)
    g.close()


def case_elementwise():
    """The memory-bound model kernels of src/ops/elementwise.cu on GPT-2-medium shapes (operands far larger than L2)."""
    from piccl_b200 import ops
    n = 128 << 20
    p = torch.zeros(n, device="cuda", dtype=torch.bfloat16); master = torch.zeros(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    g = torch.full((n,), 0.01, device="cuda", dtype=torch.bfloat16)
    T, H, C_ = 8192, 4096, 1024
    h = torch.randn(T, H, device="cuda").bfloat16(); bias = torch.randn(H, device="cuda").bfloat16()
    h_out, act, dh = torch.empty_like(h), torch.empty_like(h), torch.empty_like(h)
    idx = torch.randint(0, 50257, (T,), device="cuda")
    wte = torch.randn(50304, C_, device="cuda").bfloat16(); wpe = torch.randn(1024, C_, device="cuda").bfloat16()
    emb = torch.empty(T, C_, device="cuda", dtype=torch.bfloat16)
    cs = torch.empty(H, device="cuda", dtype=torch.bfloat16)
    for step in range(1, 3):
        ops.adamw(p, master, m, v, g, 3e-4, 0.9, 0.95, 1e-8, 0.1, step)
        ops.bias_gelu_fwd(h, bias, h_out, act)
        ops.gelu_bwd(act, h_out, dh)
        ops.embed_fwd(idx, wte, wpe, emb, 1024)
        ops.colsum(dh, cs)
    torch.cuda.synchronize()
    assert torch.isfinite(cs.float()).all() and float(master.abs().max()) > 0


def case_ln():
    from piccl_b200 import ops
    T, C = 8192 * 4, 1024
    x, r = torch.randn(T, C, device="cuda").bfloat16(), torch.randn(T, C, device="cuda").bfloat16()
    g_, b_ = torch.ones(C, device="cuda").bfloat16(), torch.zeros(C, device="cuda").bfloat16()
    s, y = torch.empty_like(x), torch.empty_like(x)
    mean, rstd = torch.empty(T, device="cuda"), torch.empty(T, device="cuda")
    dx, dg, db = torch.empty_like(x), torch.empty_like(g_), torch.empty_like(b_)
    for _ in range(4):
        ops.layernorm_fwd(x, r, g_, b_, s, y, mean, rstd)
        ops.layernorm_bwd(y, s, g_, mean, rstd, r, dx, dg, db)
    torch.cuda.synchronize()


def case_ce():
    from piccl_b200 import ops
    T, V, Vp = 8192, 50257, 50304
    logits = torch.randn(T, Vp, device="cuda").bfloat16()
    tgt = torch.randint(0, V, (T,), device="cuda")
    loss = torch.empty(T, device="cuda")
    for _ in range(4):
        ops.cross_entropy_fwd_bwd(logits, tgt, loss, V, 1.0 / T)
    torch.cuda.synchronize()


if __name__ == "__main__":
    which = sys.argv[1] if len(sys.argv) > 1 else "exec"
    {"exec": case_exec, "exec_ll": lambda: case_exec(True), "gemm": case_gemm, "gemm_pair": case_gemm_pair, "direct": case_direct, "tp": case_tp, "ln": case_ln, "ce": case_ce, "nvls": case_nvls, "llf": case_llf, "ag_gemm": case_ag_gemm, "elementwise": case_elementwise}[which]()
    print(f"profile case {which} done")
