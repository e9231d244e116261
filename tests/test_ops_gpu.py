"""Model kernels against plain PyTorch fp32 references of the same operation."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("C", [256, 768, 1024])
@pytest.mark.parametrize("with_res", [False, True])
def test_layernorm_forward_backward(C, with_res):
    from piccl_b200 import ops
    T = 300
    x, res = _bf(T, C, seed=1), (_bf(T, C, seed=2) if with_res else None)
    gamma, beta = _bf(C, seed=3) * 0.1 + 1, _bf(C, seed=4) * 0.1
    y, s = torch.empty_like(x), torch.empty_like(x)
    mean, rstd = torch.empty(T, device="cuda"), torch.empty(T, device="cuda")
    ops.layernorm_fwd(x, res, gamma, beta, s if with_res else None, y, mean, rstd)
    xin = (x.float() + res.float()).to(torch.bfloat16).float() if with_res else x.float()
    xr = xin.clone().requires_grad_()
    gr, br = gamma.float().requires_grad_(), beta.float().requires_grad_()
    yr = F.layer_norm(xr, (C,), gr, br, 1e-5)
    assert torch.allclose(y.float(), yr, atol=3e-2, rtol=2e-2)
    if with_res:
        assert torch.equal(s.float(), xin)
    assert torch.allclose(mean, xin.mean(1), atol=1e-4)
    dy, dres = _bf(T, C, seed=5), _bf(T, C, seed=6)
    dx, dg, db = torch.empty_like(x), torch.empty_like(gamma), torch.empty_like(beta)
    ops.layernorm_bwd(dy, xin.to(torch.bfloat16), gamma, mean, rstd, dres, dx, dg, db)
    yr.backward(dy.float())
    assert torch.allclose(dx.float(), xr.grad + dres.float(), atol=5e-2, rtol=3e-2)
    assert torch.allclose(dg.float(), gr.grad, atol=0.3, rtol=3e-2)
    assert torch.allclose(db.float(), br.grad, atol=0.3, rtol=3e-2)


def test_bias_gelu_and_colsum():
    from piccl_b200 import ops
    T, C = 500, 1024
    h, b = _bf(T, C, seed=1), _bf(C, seed=2)
    hp, g = torch.empty_like(h), torch.empty_like(h)
    ops.bias_gelu_fwd(h, b, hp, g)
    hr = (h.float() + b.float())
    assert torch.allclose(hp.float(), hr, atol=2e-2, rtol=1e-2)
    hq = hp.float().requires_grad_()
    gr = F.gelu(hq, approximate="tanh")
    assert torch.allclose(g.float(), gr, atol=2e-2, rtol=1e-2)
    dg = _bf(T, C, seed=3)
    dh = torch.empty_like(dg)
    ops.gelu_bwd(dg, hp, dh)
    gr.backward(dg.float())
    assert torch.allclose(dh.float(), hq.grad, atol=2e-2, rtol=2e-2)
    out = torch.empty(C, device="cuda", dtype=torch.bfloat16)
    ops.colsum(dg, out)
    assert torch.allclose(out.float(), dg.float().sum(0), atol=0.3, rtol=2e-2)


def test_cross_entropy_with_padded_vocab():
    from piccl_b200 import ops
    T, V, Vp = 64, 1000, 1024
    logits = _bf(T, Vp, scale=2.0, seed=1)
    ref_in = logits[:, :V].float().clone().requires_grad_()
    tgt = torch.randint(0, V, (T,), device="cuda")
    loss_rows = torch.empty(T, device="cuda")
    ops.cross_entropy_fwd_bwd(logits, tgt, loss_rows, V, 1.0 / T)
    ref = F.cross_entropy(ref_in, tgt, reduction="none")
    assert torch.allclose(loss_rows, ref, atol=1e-3, rtol=1e-3)
    ref.mean().backward()
    assert torch.allclose(logits[:, :V].float(), ref_in.grad, atol=2e-4, rtol=2e-2)
    assert logits[:, V:].abs().sum() == 0


def test_adamw_matches_torch():
    from piccl_b200 import ops
    n = 4096
    p0 = _bf(n, seed=1)
    master = p0.float().clone()
    p = p0.clone()
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    ref = torch.nn.Parameter(p0.float().clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        g = _bf(n, seed=10 + step)
        ops.adamw(p, master, m, v, g, 1e-2, 0.9, 0.95, 1e-8, 0.1, step)
        ref.grad = g.float()
        opt.step()
    assert torch.allclose(master, ref.data, atol=1e-5, rtol=1e-4)
    assert torch.allclose(p.float(), ref.data, atol=1e-2, rtol=1e-2)


def test_embedding_forward_backward():
    from piccl_b200 import ops
    B, S, C, V = 3, 16, 256, 100
    idx = torch.randint(0, V, (B * S,), device="cuda")
    wte, wpe = _bf(V, C, seed=1), _bf(S, C, seed=2)
    out = torch.empty(B * S, C, device="cuda", dtype=torch.bfloat16)
    ops.embed_fwd(idx, wte, wpe, out, S)
    ref = wte.float()[idx] + wpe.float().repeat(B, 1)
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=1e-2)
    dx = _bf(B * S, C, seed=3)
    dwpe = torch.zeros_like(wpe)
    ops.wpe_bwd(dx, dwpe, B, S)
    assert torch.allclose(dwpe.float(), dx.float().view(B, S, C).sum(0), atol=5e-2, rtol=2e-2)
    dwte = torch.zeros_like(wte)
    stage = torch.zeros(V, C, device="cuda")
    ops.wte_bwd(idx, dx, stage, dwte)
    ref_g = torch.zeros(V, C, device="cuda").index_add_(0, idx, dx.float())
    assert torch.allclose(dwte.float(), ref_g, atol=5e-2, rtol=2e-2)
