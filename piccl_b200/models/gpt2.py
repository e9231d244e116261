"""GPT-2 written against the framework's own kernels, with a hand-scheduled
backward pass.

Why not autograd: the backward pass is where data-parallel communication
overlaps with compute, so the model itself decides when a contiguous range of
the flat gradient buffer is final and hands it to the bucketed all-reduce
(`on_grads_ready`).  Parameters and gradients live in two flat bf16 buffers laid
out in the order in which the backward pass finishes them; buckets are therefore
plain slices and never copied.  fp32 master weights and AdamW moments live in
flat fp32 buffers and are updated by one fused kernel per parameter group.

Kernels: residual-add + LayerNorm (forward / backward), bias + GELU, bias
gradients, embedding, softmax cross entropy with in-place gradient and AdamW are
this framework's CUDA kernels (src/ops); matrix products go through
`piccl_b200.ops.gemm` (tcgen05 kernel where enabled, cuBLAS otherwise) and
attention through PyTorch's fused SDPA.

The reference has no model code at all; this module exists for the end-to-end
data-parallel benchmark (GPT-2 medium under bucketed gradient all-reduce).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from .. import ops
from ..ops import gemm


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    seq_len: int = 1024
    n_layer: int = 24
    n_head: int = 16
    d_model: int = 1024
    ln_eps: float = 1e-5

    @property
    def padded_vocab(self) -> int:
        return (self.vocab_size + 127) // 128 * 128

    @staticmethod
    def medium() -> "GPT2Config":
        return GPT2Config()

    @staticmethod
    def tiny() -> "GPT2Config":
        return GPT2Config(vocab_size=1000, seq_len=128, n_layer=2, n_head=4, d_model=256)


_DECAY = ("w_qkv", "w_o", "w_fc", "w_proj")
_NODECAY = ("ln1_g", "ln1_b", "b_qkv", "b_o", "ln2_g", "ln2_b", "b_fc", "b_proj")


class GPT2:
    def __init__(self, cfg: GPT2Config, device="cuda", seed: int = 0):
        self.cfg = cfg
        self.device = torch.device(device)
        C, L, Vp, S = cfg.d_model, cfg.n_layer, cfg.padded_vocab, cfg.seq_len
        shapes = {"w_qkv": (3 * C, C), "w_o": (C, C), "w_fc": (4 * C, C), "w_proj": (C, 4 * C), "ln1_g": (C,), "ln1_b": (C,),
                  "b_qkv": (3 * C,), "b_o": (C,), "ln2_g": (C,), "ln2_b": (C,), "b_fc": (4 * C,), "b_proj": (C,)}
        # flat order = order in which the backward pass completes gradients
        layout = [("lnf_g", (C,), False), ("lnf_b", (C,), False)]
        for l in reversed(range(L)):
            layout += [(f"h{l}.{n}", shapes[n], True) for n in _DECAY]
            layout += [(f"h{l}.{n}", shapes[n], False) for n in _NODECAY]
        layout += [("wpe", (S, C), True), ("wte", (Vp, C), True)]
        total = sum(math.prod(s) for _, s, _ in layout)
        self.flat_p = torch.zeros(total, dtype=torch.bfloat16, device=self.device)
        self.flat_g = torch.zeros(total, dtype=torch.bfloat16, device=self.device)
        self.p: dict[str, torch.Tensor] = {}
        self.g: dict[str, torch.Tensor] = {}
        self.offset: dict[str, tuple[int, int]] = {}
        self.groups: list[tuple[int, int, bool]] = []     # (begin, end, decay) runs for the optimizer
        off = 0
        for name, shape, decay in layout:
            n = math.prod(shape)
            self.p[name] = self.flat_p[off:off + n].view(shape)
            self.g[name] = self.flat_g[off:off + n].view(shape)
            self.offset[name] = (off, off + n)
            if self.groups and self.groups[-1][2] == decay and self.groups[-1][1] == off:
                self.groups[-1] = (self.groups[-1][0], off + n, decay)
            else:
                self.groups.append((off, off + n, decay))
            off += n
        self.n_params = total
        self._init_weights(seed)
        self.master = self.flat_p.float()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.step_count = 0
        self.step_dev = torch.zeros(1, dtype=torch.int32, device=self.device)     # the same counter on the device (graph replay)
        self._bufs: dict = {}
        self._wte_stage: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ setup
    def _init_weights(self, seed: int) -> None:
        cfg = self.cfg
        gen = torch.Generator(device=self.device).manual_seed(seed)
        for name, t in self.p.items():
            base = name.split(".")[-1]
            if base in ("ln1_g", "ln2_g", "lnf_g"):
                t.fill_(1.0)
            elif base.startswith("b_") or base.endswith("_b"):
                t.zero_()
            else:
                std = 0.02 / math.sqrt(2 * cfg.n_layer) if base in ("w_o", "w_proj") else 0.02
                t.copy_((torch.randn(t.shape, generator=gen, device=self.device, dtype=torch.float32) * std).to(torch.bfloat16))
        self.p["wte"][cfg.vocab_size:].zero_()

    def _buf(self, key, shape, dtype=torch.bfloat16):
        t = self._bufs.get(key)
        if t is None or tuple(t.shape) != tuple(shape) or t.dtype != dtype:
            t = torch.empty(shape, dtype=dtype, device=self.device)
            self._bufs[key] = t
        return t

    # ------------------------------------------------------------------ forward + backward
    def forward_backward(self, idx: torch.Tensor, targets: torch.Tensor,
                         on_grads_ready: Optional[Callable[[int], None]] = None, loss_only: bool = False) -> torch.Tensor:
        """One training micro-step: returns the mean loss (fp32, on device) and leaves the
        gradients in `flat_g`.  `on_grads_ready(end)` is called whenever flat_g[:end] is final."""
        cfg = self.cfg
        B, S = idx.shape
        T, C, L, H = B * S, cfg.d_model, cfg.n_layer, cfg.n_head
        D = C // H
        p, g, buf = self.p, self.g, self._buf
        idx = idx.reshape(-1).contiguous()
        targets = targets.reshape(-1).contiguous()
        f32 = torch.float32

        x = buf("x0", (T, C))
        ops.embed_fwd(idx, p["wte"], p["wpe"], x, S)
        saved = []
        ln_in = buf(("ln1", 0), (T, C))
        mean1, rstd1 = buf(("mean1", 0), (T,), f32), buf(("rstd1", 0), (T,), f32)
        ops.layernorm_fwd(x, None, p["h0.ln1_g"], p["h0.ln1_b"], None, ln_in, mean1, rstd1, cfg.ln_eps)
        xin = x
        for l in range(L):
            P = lambda n: p[f"h{l}.{n}"]
            qkv = buf(("qkv", l), (T, 3 * C))
            gemm.linear(ln_in, P("w_qkv"), P("b_qkv"), out=qkv)
            qkv_leaf = qkv.detach().requires_grad_(not loss_only)
            with torch.enable_grad():
                q, k, v = qkv_leaf.view(B, S, 3, H, D).permute(2, 0, 3, 1, 4).unbind(0)
                att = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(T, C)
            a = buf("a", (T, C))
            gemm.linear(att.detach(), P("w_o"), P("b_o"), out=a)
            x2, ln2 = buf(("x2", l), (T, C)), buf(("ln2", l), (T, C))
            mean2, rstd2 = buf(("mean2", l), (T,), f32), buf(("rstd2", l), (T,), f32)
            ops.layernorm_fwd(a, xin, P("ln2_g"), P("ln2_b"), x2, ln2, mean2, rstd2, cfg.ln_eps)
            h, gl = buf(("h", l), (T, 4 * C)), buf(("g", l), (T, 4 * C))
            gemm.linear_gelu(ln2, P("w_fc"), P("b_fc"), h, gl)
            pr = buf("pr", (T, C))
            gemm.linear(gl, P("w_proj"), P("b_proj"), out=pr)
            x3 = buf(("x3", l), (T, C))
            nxt = buf(("ln1", l + 1), (T, C))
            nmean, nrstd = buf(("mean1", l + 1), (T,), f32), buf(("rstd1", l + 1), (T,), f32)
            if l + 1 < L:
                ops.layernorm_fwd(pr, x2, p[f"h{l + 1}.ln1_g"], p[f"h{l + 1}.ln1_b"], x3, nxt, nmean, nrstd, cfg.ln_eps)
            else:
                ops.layernorm_fwd(pr, x2, p["lnf_g"], p["lnf_b"], x3, nxt, nmean, nrstd, cfg.ln_eps)
            saved.append((xin, ln_in, mean1, rstd1, qkv_leaf, att, x2, ln2, mean2, rstd2, h, gl))
            xin, ln_in, mean1, rstd1 = x3, nxt, nmean, nrstd

        logits = buf("logits", (T, cfg.padded_vocab))
        gemm.linear(ln_in, p["wte"], None, out=logits)
        loss_rows = buf("loss_rows", (T,), f32)
        ops.cross_entropy_fwd_bwd(logits, targets, loss_rows, cfg.vocab_size, 1.0 / T)
        loss = loss_rows.mean()
        if loss_only:
            return loss

        # ---------------- backward (logits now hold d loss / d logits)
        ready = on_grads_ready or (lambda end: None)
        gemm.grad_weight(logits, ln_in, out=g["wte"])
        dln = buf("dlnf", (T, C))
        gemm.grad_input(logits, p["wte"], out=dln)
        dx = buf("dx_a", (T, C))
        ops.layernorm_bwd(dln, xin, p["lnf_g"], mean1, rstd1, None, dx, g["lnf_g"], g["lnf_b"])
        ready(self.offset["lnf_b"][1])
        for l in reversed(range(L)):
            P = lambda n: p[f"h{l}.{n}"]
            G = lambda n: g[f"h{l}.{n}"]
            xin_l, ln1_l, m1, r1, qkv_leaf, att, x2, ln2, m2, r2, h, gl = saved[l]
            # x3 = x2 + gelu(ln2 @ Wfc + bfc) @ Wproj + bproj
            ops.colsum(dx, G("b_proj"))
            gemm.grad_weight(dx, gl, out=G("w_proj"))
            dg = buf("dg", (T, 4 * C))
            gemm.grad_input(dx, P("w_proj"), out=dg)
            ops.gelu_bwd(dg, h, dg)
            ops.colsum(dg, G("b_fc"))
            gemm.grad_weight(dg, ln2, out=G("w_fc"))
            dln2 = buf("dln2", (T, C))
            gemm.grad_input(dg, P("w_fc"), out=dln2)
            dx2 = buf("dx_b", (T, C))
            ops.layernorm_bwd(dln2, x2, P("ln2_g"), m2, r2, dx, dx2, G("ln2_g"), G("ln2_b"))
            # x2 = xin + att @ Wo + bo
            ops.colsum(dx2, G("b_o"))
            gemm.grad_weight(dx2, att.detach(), out=G("w_o"))
            datt = buf("datt", (T, C))
            gemm.grad_input(dx2, P("w_o"), out=datt)
            (dqkv,) = torch.autograd.grad(att, qkv_leaf, datt)
            dqkv = dqkv.reshape(T, 3 * C)
            ops.colsum(dqkv, G("b_qkv"))
            gemm.grad_weight(dqkv, ln1_l, out=G("w_qkv"))
            dln1 = buf("dln1", (T, C))
            gemm.grad_input(dqkv, P("w_qkv"), out=dln1)
            ops.layernorm_bwd(dln1, xin_l, P("ln1_g"), m1, r1, dx2, dx, G("ln1_g"), G("ln1_b"))
            ready(self.offset[f"h{l}.b_proj"][1])
        ops.wpe_bwd(dx, g["wpe"], B, S)
        ready(self.offset["wpe"][1])
        if self._wte_stage is None:
            self._wte_stage = torch.empty(cfg.padded_vocab, C, dtype=f32, device=self.device)
        self._wte_stage.zero_()
        ops.wte_bwd(idx, dx, self._wte_stage, g["wte"])
        ready(self.n_params)
        return loss

    # ------------------------------------------------------------------ optimizer
    def optimizer_step(self, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1) -> None:
        """Fused AdamW over the flat buffers; the step number lives on the device so that the launches can be replayed."""
        self.step_count += 1
        self.step_dev.add_(1)
        for b, e, decay in self.groups:
            ops.adamw_devstep(self.flat_p[b:e], self.master[b:e], self.m[b:e], self.v[b:e], self.flat_g[b:e], lr, betas[0], betas[1], eps,
                              weight_decay if decay else 0.0, self.step_dev)

    @torch.no_grad()
    def loss(self, idx: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        return self.forward_backward(idx, targets, loss_only=True)

    # ------------------------------------------------------------------ interchange with a plain PyTorch module
    def state_dict(self) -> dict:
        """Parameters under the names of a conventional GPT-2 module (unpadded vocabulary)."""
        cfg = self.cfg
        sd = {"wte.weight": self.p["wte"][:cfg.vocab_size].clone(), "wpe.weight": self.p["wpe"].clone(),
              "ln_f.weight": self.p["lnf_g"].clone(), "ln_f.bias": self.p["lnf_b"].clone()}
        names = {"ln1_g": "ln_1.weight", "ln1_b": "ln_1.bias", "w_qkv": "attn.c_attn.weight", "b_qkv": "attn.c_attn.bias", "w_o": "attn.c_proj.weight",
                 "b_o": "attn.c_proj.bias", "ln2_g": "ln_2.weight", "ln2_b": "ln_2.bias", "w_fc": "mlp.c_fc.weight", "b_fc": "mlp.c_fc.bias",
                 "w_proj": "mlp.c_proj.weight", "b_proj": "mlp.c_proj.bias"}
        for l in range(cfg.n_layer):
            for k, v in names.items():
                sd[f"h.{l}.{v}"] = self.p[f"h{l}.{k}"].clone()
        return sd
