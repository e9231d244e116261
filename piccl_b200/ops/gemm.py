"""Matrix products of the model: y = x W^T (+ bias), dx = dy W, dW = dy^T x.

Two back ends, chosen once per process (`set_backend`):
  "tcgen05"  this framework's sm_100a kernel (src/ops/gemm_sm100.cu: TMA -> shared memory ->
             tcgen05.mma with TMEM accumulators) for the forward products whose shapes it
             supports; everything else through cuBLAS
  "cublas"   cuBLAS through torch.mm / torch.addmm for all three
"""
from __future__ import annotations

import os

import torch

_backend = os.environ.get("PICCL_GEMM", "auto")
_counts = {"tcgen05": 0, "cublas": 0}


def set_backend(name: str) -> None:
    global _backend
    assert name in ("auto", "tcgen05", "cublas")
    _backend = name


def backend() -> str:
    return _backend


def counts() -> dict:
    return dict(_counts)


def _own_kernel_ok(x, w, out, fused_epilogue: bool = False) -> bool:
    """"auto": the tcgen05 kernel where its fused epilogue saves a pass over the activations (bias + GELU);
    plain products stay on cuBLAS, which is still a little faster on those shapes.  "tcgen05": wherever supported."""
    if _backend == "cublas" or (_backend == "auto" and not fused_epilogue):
        return False
    from . import gemm_sm100
    return gemm_sm100.available() and gemm_sm100.supports(x, w, out)


def linear(x: torch.Tensor, w: torch.Tensor, bias, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T + bias[N]"""
    if _own_kernel_ok(x, w, out):
        from . import gemm_sm100
        gemm_sm100.gemm_nt(x, w, out, bias=bias)
        _counts["tcgen05"] += 1
        return out
    _counts["cublas"] += 1
    if bias is None:
        return torch.mm(x, w.t(), out=out)
    return torch.addmm(bias, x, w.t(), out=out)


def linear_gelu(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor, h_out: torch.Tensor, g_out: torch.Tensor) -> None:
    """h_out = x @ w^T + bias;  g_out = gelu_tanh(h_out)   — one kernel where the tcgen05 GEMM is usable."""
    if _own_kernel_ok(x, w, g_out, fused_epilogue=True):
        from . import gemm_sm100
        gemm_sm100.gemm_nt(x, w, g_out, bias=bias, gelu=True, pre=h_out)
        _counts["tcgen05"] += 1
        return
    from . import bias_gelu_fwd
    _counts["cublas"] += 1
    torch.mm(x, w.t(), out=h_out)
    bias_gelu_fwd(h_out, bias, h_out, g_out)


def grad_input(dy: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, K] = dy[M, N] @ w[N, K]"""
    _counts["cublas"] += 1
    return torch.mm(dy, w, out=out)


def grad_weight(dy: torch.Tensor, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[N, K] = dy[M, N]^T @ x[M, K]"""
    _counts["cublas"] += 1
    return torch.mm(dy.t(), x, out=out)
