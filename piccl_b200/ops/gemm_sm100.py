"""Front end of the tcgen05 GEMM (src/ops/gemm_sm100.cu)."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N
from . import _bump

_checked = None


def available() -> bool:
    global _checked
    if _checked is None:
        try:
            lib = N.ops_lib()
            _checked = hasattr(lib, "piccl_ops_gemm_bf16_nt_ex") and torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10
        except Exception:
            _checked = False
    return _checked


def supports(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    M, K = x.shape
    Nn = w.shape[0]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
            and out.is_contiguous() and K % 64 == 0 and Nn % 128 == 0 and M % 128 == 0 and K >= 64)


def gemm_nt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias=None, gelu: bool = False, pre=None) -> torch.Tensor:
    """out[M, N] = act(x[M, K] @ w[N, K]^T + bias); `pre` (optional) receives the value before the activation"""
    M, K = x.shape
    Nn = w.shape[0]
    rc = N.ops_lib().piccl_ops_gemm_bf16_nt_ex(C.c_void_p(x.data_ptr()), C.c_void_p(w.data_ptr()), C.c_void_p(out.data_ptr()),
                                               C.c_void_p(pre.data_ptr() if pre is not None else 0),
                                               C.c_void_p(bias.data_ptr() if bias is not None else 0), M, Nn, K, int(gelu),
                                               C.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc != 0:
        raise RuntimeError(f"piccl_ops_gemm_bf16_nt failed (code {rc}) for M={M} N={Nn} K={K}")
    _bump()
    return out


def gemm_nt_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias=None) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T + bias on CTA pairs (`tcgen05.mma.cta_group::2`, src/ops2/gemm_sm100_2cta.cu).
    M and N multiples of 256, K a multiple of 64.  Opt-in: nothing in the package calls it by default."""
    M, K = x.shape
    Nn = w.shape[0]
    rc = N.gemm2_lib().piccl_ops2_gemm_bf16_nt(C.c_void_p(x.data_ptr()), C.c_void_p(w.data_ptr()), C.c_void_p(out.data_ptr()),
                                               C.c_void_p(bias.data_ptr() if bias is not None else 0), M, Nn, K,
                                               C.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc != 0:
        raise RuntimeError(f"piccl_ops2_gemm_bf16_nt failed (code {rc}) for M={M} N={Nn} K={K}")
    _bump()
    return out


def pair_status() -> int:
    """0, or the role whose bounded wait ran out in the CTA-pair GEMM since the last call (synchronises the device)."""
    return int(N.gemm2_lib().piccl_ops2_gemm_status())
