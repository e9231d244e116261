"""The framework's GPT-2 (own kernels, hand-scheduled backward) against a conventional
PyTorch module with the same weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _pair():
    from benchmarks.torch_gpt2 import TorchGPT2
    from piccl_b200.models.gpt2 import GPT2, GPT2Config
    cfg = GPT2Config.tiny()
    mine = GPT2(cfg, seed=3)
    ref = TorchGPT2(cfg.vocab_size, cfg.seq_len, cfg.n_layer, cfg.n_head, cfg.d_model).cuda().float()
    sd = {k: v.float() for k, v in mine.state_dict().items()}
    missing = ref.load_state_dict(sd, strict=True)
    assert not missing.missing_keys
    return cfg, mine, ref


def test_loss_and_gradients_match_pytorch():
    cfg, mine, ref = _pair()
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len + 1), generator=g).cuda()
    a, b = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    loss = mine.forward_backward(a, b)
    rl = ref(a, b)
    rl.backward()
    assert abs(float(loss) - float(rl)) < 3e-2, (float(loss), float(rl))
    checks = {"lnf_g": ref.ln_f.weight.grad, "h1.w_fc": ref.h[1].mlp["c_fc"].weight.grad, "h0.w_qkv": ref.h[0].attn["c_attn"].weight.grad,
              "h0.b_qkv": ref.h[0].attn["c_attn"].bias.grad, "h1.ln2_b": ref.h[1].ln_2.bias.grad, "wpe": ref.wpe.weight.grad,
              "h0.w_proj": ref.h[0].mlp["c_proj"].weight.grad, "h1.w_o": ref.h[1].attn["c_proj"].weight.grad}
    for name, rg in checks.items():
        mg = mine.g[name].float()
        rel = (mg - rg).norm() / (rg.norm() + 1e-12)
        assert rel < 5e-2, f"{name}: relative gradient error {float(rel):.4f}"
    mg = mine.g["wte"][:cfg.vocab_size].float()
    rel = (mg - ref.wte.weight.grad).norm() / ref.wte.weight.grad.norm()
    assert rel < 5e-2, f"wte: {float(rel):.4f}"


def test_training_reduces_loss_and_ready_ranges_are_monotonic():
    from piccl_b200.models.gpt2 import GPT2, GPT2Config
    cfg = GPT2Config.tiny()
    m = GPT2(cfg, seed=1)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len + 1), generator=g).cuda()
    a, b = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    ends = []
    losses = []
    for _ in range(8):
        ends.clear()
        losses.append(float(m.forward_backward(a, b, on_grads_ready=ends.append)))
        m.optimizer_step(lr=1e-3)
    assert ends == sorted(ends) and ends[-1] == m.n_params
    assert losses[-1] < losses[0] - 0.5, losses
