"""A conventional PyTorch GPT-2 (nn.Module, autograd, fused SDPA) used as the
workload of the reference arm and as the numerical oracle of the framework's own
model.  Nothing here uses the framework's kernels."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class Block(nn.Module):
    def __init__(self, C, H):
        super().__init__()
        self.H = H
        self.ln_1 = nn.LayerNorm(C)
        self.attn = nn.ModuleDict({"c_attn": nn.Linear(C, 3 * C), "c_proj": nn.Linear(C, C)})
        self.ln_2 = nn.LayerNorm(C)
        self.mlp = nn.ModuleDict({"c_fc": nn.Linear(C, 4 * C), "c_proj": nn.Linear(4 * C, C)})

    def forward(self, x):
        B, S, C = x.shape
        q, k, v = self.attn["c_attn"](self.ln_1(x)).view(B, S, 3, self.H, C // self.H).permute(2, 0, 3, 1, 4).unbind(0)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, C)
        x = x + self.attn["c_proj"](y)
        return x + self.mlp["c_proj"](F.gelu(self.mlp["c_fc"](self.ln_2(x)), approximate="tanh"))


class TorchGPT2(nn.Module):
    def __init__(self, vocab_size=50257, seq_len=1024, n_layer=24, n_head=16, d_model=1024):
        super().__init__()
        self.wte = nn.Embedding(vocab_size, d_model)
        self.wpe = nn.Embedding(seq_len, d_model)
        self.h = nn.ModuleList([Block(d_model, n_head) for _ in range(n_layer)])
        self.ln_f = nn.LayerNorm(d_model)
        self.n_layer = n_layer
        self.apply(self._init)
        for name, p in self.named_parameters():
            if name.endswith("c_proj.weight"):
                nn.init.normal_(p, mean=0.0, std=0.02 / math.sqrt(2 * n_layer))

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)
            if isinstance(m, nn.Linear) and m.bias is not None:
                nn.init.zeros_(m.bias)

    def forward(self, idx, targets):
        B, S = idx.shape
        x = self.wte(idx) + self.wpe(torch.arange(S, device=idx.device))
        for blk in self.h:
            x = blk(x)
        logits = F.linear(self.ln_f(x), self.wte.weight)      # tied output projection
        return F.cross_entropy(logits.view(-1, logits.size(-1)).float(), targets.view(-1))
