"""Fused GEMM -> reduce-scatter and all-gather -> GEMM on one GPU (virtual ranks in one cooperative
launch) against a plain PyTorch fp32 reference of the same operation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bf(*shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def _group(n, which, M, N, K):
    from piccl_b200.parallel import tp
    from piccl_b200.parallel.comm import LoopbackGroup, make_config
    ws = tp.workspace_bytes(which, n, M, N, K)
    return LoopbackGroup(n, config=make_config(max_cta=4, nslot=2, slot_bytes=4096, scratch_bytes=1 << 16, timeout_ms=5000, tp_bytes=ws))


@pytest.mark.parametrize("n,M,N,K", [(1, 256, 256, 128), (2, 512, 512, 256), (4, 1024, 768, 192), (2, 2048, 1024, 512)])
def test_gemm_reduce_scatter(n, M, N, K):
    from piccl_b200.parallel import tp
    g = _group(n, "gemm_rs", M, N, K)
    As = [_bf(M, K, seed=10 + r) for r in range(n)]
    Bs = [_bf(N, K, seed=20 + r, scale=0.1) for r in range(n)]
    outs = [torch.full((M // n, N), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(n)]
    for rep in range(3):          # epochs / parity of the double-buffered inbox
        tp.gemm_rs_group(g, As, Bs, outs)
    torch.cuda.synchronize()
    assert all(tp.tp_status(h) == 0 for h in g._hs)
    # partial products are exchanged in bf16, as a bf16 reduce-scatter after a bf16 GEMM would
    ref = sum((As[r].float() @ Bs[r].float().t()).to(torch.bfloat16).float() for r in range(n))
    for r in range(n):
        want = ref[r * (M // n):(r + 1) * (M // n)]
        tol = 0.02 * want.abs().max().item() + 0.05
        assert torch.allclose(outs[r].float(), want, atol=tol, rtol=2e-2), f"rank {r}: max err {(outs[r].float() - want).abs().max().item()}"
    g.close()


@pytest.mark.parametrize("n,M,N,K", [(1, 256, 256, 128), (2, 512, 256, 256), (4, 1024, 512, 192), (2, 2048, 768, 512)])
def test_allgather_gemm(n, M, N, K):
    from piccl_b200.parallel import tp
    g = _group(n, "ag_gemm", M, N, K)
    As = [_bf(M // n, K, seed=30 + r) for r in range(n)]
    Bs = [_bf(N, K, seed=40 + r, scale=0.1) for r in range(n)]
    outs = [torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(n)]
    for rep in range(3):
        tp.ag_gemm_group(g, As, Bs, outs)
    torch.cuda.synchronize()
    assert all(tp.tp_status(h) == 0 for h in g._hs)
    full = torch.cat(As).float()
    for r in range(n):
        want = full @ Bs[r].float().t()
        tol = 0.02 * want.abs().max().item() + 0.05
        assert torch.allclose(outs[r].float(), want, atol=tol, rtol=2e-2), f"rank {r}: max err {(outs[r].float() - want).abs().max().item()}"
    g.close()


def test_kernels_and_shapes_interleaved_without_host_synchronisation():
    """all-gather -> GEMM, GEMM -> reduce-scatter and a second GEMM -> reduce-scatter shape back to back on one stream, several
    rounds, no synchronisation in between: each kernel owns its part of the workspace and the halves used by consecutive
    calls do not depend on the shape, so a rank that is a call ahead never writes where a peer still reads."""
    from piccl_b200.parallel import tp
    n = 2
    shapes = {"ag": (1024, 512, 256), "rs1": (1024, 768, 256), "rs2": (512, 256, 128)}
    ws = max(tp.workspace_bytes("ag_gemm", n, *shapes["ag"]), tp.workspace_bytes("gemm_rs", n, *shapes["rs1"]), tp.workspace_bytes("gemm_rs", n, *shapes["rs2"]))
    from piccl_b200.parallel.comm import LoopbackGroup, make_config
    g = LoopbackGroup(n, config=make_config(max_cta=4, nslot=2, slot_bytes=4096, scratch_bytes=1 << 16, timeout_ms=5000, tp_bytes=ws))
    M, N, K = shapes["ag"]
    ag_A = [_bf(M // n, K, seed=50 + r) for r in range(n)]; ag_B = [_bf(N, K, seed=60 + r, scale=0.1) for r in range(n)]
    ag_out = [torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(n)]
    rs = {}
    for key in ("rs1", "rs2"):
        M2, N2, K2 = shapes[key]
        rs[key] = ([_bf(M2, K2, seed=70 + r) for r in range(n)], [_bf(N2, K2, seed=80 + r, scale=0.1) for r in range(n)],
                   [torch.full((M2 // n, N2), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(n)])
    for rep in range(4):
        tp.ag_gemm_group(g, ag_A, ag_B, ag_out)
        tp.gemm_rs_group(g, *rs["rs1"])
        tp.gemm_rs_group(g, *rs["rs2"])
    torch.cuda.synchronize()
    assert all(tp.tp_status(h) == 0 for h in g._hs)
    full = torch.cat(ag_A).float()
    for r in range(n):
        want = full @ ag_B[r].float().t()
        assert torch.allclose(ag_out[r].float(), want, atol=0.02 * want.abs().max().item() + 0.05, rtol=2e-2)
    for key in ("rs1", "rs2"):
        As, Bs, outs = rs[key]
        M2 = shapes[key][0]
        ref = sum((As[r].float() @ Bs[r].float().t()).to(torch.bfloat16).float() for r in range(n))
        for r in range(n):
            want = ref[r * (M2 // n):(r + 1) * (M2 // n)]
            assert torch.allclose(outs[r].float(), want, atol=0.02 * want.abs().max().item() + 0.05, rtol=2e-2), key
    g.close()


def test_workspace_is_checked():
    from piccl_b200 import _native as N
    from piccl_b200.parallel import tp
    from piccl_b200.parallel.comm import LoopbackGroup, make_config
    g = LoopbackGroup(2, config=make_config(max_cta=2, nslot=2, slot_bytes=4096, scratch_bytes=1 << 16, tp_bytes=4096))
    a = [_bf(512, 128, seed=1) for _ in range(2)]
    b = [_bf(256, 128, seed=2) for _ in range(2)]
    o = [torch.empty(256, 256, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    with pytest.raises(N.PicclError):
        tp.gemm_rs_group(g, a, b, o)
    g.close()
