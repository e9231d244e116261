"""Python front ends of the model kernels in libpiccl_ops.so.

Every function launches hand-written CUDA on the current stream and fails
loudly if the native library is missing; there is no PyTorch fallback.  A
process-wide launch counter (`launch_count()`) records how many of these
kernels were started, which the benchmark reports.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _native as N

_launches = 0


def launch_count() -> int:
    return _launches


def _bump(n: int = 1) -> None:
    global _launches
    _launches += n


def _s() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(t.data_ptr() if t is not None else 0)


def _chk(rc: int, name: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{name} failed (code {rc})")


_ws: dict = {}


def _workspace(n_floats: int, device) -> torch.Tensor:
    key = (device, "f32")
    w = _ws.get(key)
    if w is None or w.numel() < n_floats:
        w = torch.empty(max(n_floats, 1 << 20), dtype=torch.float32, device=device)
        _ws[key] = w
    return w


def layernorm_fwd(x, res, gamma, beta, sum_out, y, mean, rstd, eps: float = 1e-5):
    """y = LN(x + res) * gamma + beta; sum_out = x + res (either may be None)."""
    rows, Cc = x.shape
    _chk(N.ops_lib().piccl_ops_ln_fwd(_p(x), _p(res), _p(gamma), _p(beta), _p(sum_out), _p(y), _p(mean), _p(rstd), rows, Cc, C.c_float(eps), C.c_void_p(_s())), "ln_fwd")
    _bump()


def layernorm_bwd(dy, xin, gamma, mean, rstd, dres, dx, dgamma, dbeta, accumulate: bool = False, rows_per_block: int = 32):
    """dx = dLN(dy) + dres; dgamma / dbeta (bf16) written or accumulated."""
    rows, Cc = dy.shape
    nblocks = (rows + rows_per_block - 1) // rows_per_block
    ws = _workspace(2 * nblocks * Cc, dy.device)
    _chk(N.ops_lib().piccl_ops_ln_bwd(_p(dy), _p(xin), _p(gamma), _p(mean), _p(rstd), _p(dres), _p(dx), _p(dgamma), _p(dbeta), _p(ws), rows, Cc,
                                      rows_per_block, int(accumulate), C.c_void_p(_s())), "ln_bwd")
    _bump(3)


def bias_gelu_fwd(h, bias, h_out, g):
    rows, Cc = h.shape
    _chk(N.ops_lib().piccl_ops_bias_gelu_fwd(_p(h), _p(bias), _p(h_out), _p(g), C.c_longlong(rows), Cc, C.c_void_p(_s())), "bias_gelu_fwd")
    _bump()


def gelu_bwd(dg, h, dh):
    _chk(N.ops_lib().piccl_ops_gelu_bwd(_p(dg), _p(h), _p(dh), C.c_longlong(dg.numel()), C.c_void_p(_s())), "gelu_bwd")
    _bump()


def colsum(x, out, accumulate: bool = False, rows_per_block: int = 256):
    """out[c] (+)= sum_r x[r, c]  (bias gradient)."""
    rows, Cc = x.shape
    nparts = (rows + rows_per_block - 1) // rows_per_block
    ws = _workspace(nparts * Cc, x.device)
    _chk(N.ops_lib().piccl_ops_colsum(_p(x), _p(out), _p(ws), rows, Cc, rows_per_block, int(accumulate), C.c_void_p(_s())), "colsum")
    _bump(2)


def cross_entropy_fwd_bwd(logits, targets, loss_rows, vocab: int, gscale: float):
    """loss_rows[r] = CE(logits[r, :vocab], targets[r]); logits <- d(loss)/d(logits) * gscale, in place."""
    rows, Vp = logits.shape
    _chk(N.ops_lib().piccl_ops_ce_fwd_bwd(_p(logits), _p(targets), _p(loss_rows), rows, vocab, Vp, C.c_float(gscale), C.c_void_p(_s())), "ce_fwd_bwd")
    _bump()


def adamw(p, master, m, v, g, lr: float, b1: float, b2: float, eps: float, wd: float, step: int, gscale: float = 1.0):
    _chk(N.ops_lib().piccl_ops_adamw(_p(p), _p(master), _p(m), _p(v), _p(g), C.c_longlong(p.numel()), C.c_float(lr), C.c_float(b1), C.c_float(b2),
                                     C.c_float(eps), C.c_float(wd), step, C.c_float(gscale), C.c_void_p(_s())), "adamw")
    _bump()


def adamw_devstep(p, master, m, v, g, lr: float, b1: float, b2: float, eps: float, wd: float, step_dev, gscale: float = 1.0):
    """AdamW with the step number in a device int32 tensor (replayable from a CUDA graph)."""
    _chk(N.ops_lib().piccl_ops_adamw_devstep(_p(p), _p(master), _p(m), _p(v), _p(g), C.c_longlong(p.numel()), C.c_float(lr), C.c_float(b1), C.c_float(b2),
                                             C.c_float(eps), C.c_float(wd), _p(step_dev), C.c_float(gscale), C.c_void_p(_s())), "adamw_devstep")
    _bump()


def embed_fwd(idx, wte, wpe, out, seq: int):
    rows, Cc = out.shape
    _chk(N.ops_lib().piccl_ops_embed_fwd(_p(idx), _p(wte), _p(wpe), _p(out), rows, seq, Cc, C.c_void_p(_s())), "embed_fwd")
    _bump()


def wpe_bwd(dx, dwpe, batch: int, seq: int, accumulate: bool = False):
    _chk(N.ops_lib().piccl_ops_wpe_bwd(_p(dx), _p(dwpe), batch, seq, dx.shape[1], int(accumulate), C.c_void_p(_s())), "wpe_bwd")
    _bump()


def wte_bwd(idx, dx, stage, dwte):
    rows, Cc = dx.shape
    _chk(N.ops_lib().piccl_ops_wte_bwd(_p(idx), _p(dx), _p(stage), _p(dwte), rows, C.c_longlong(dwte.shape[0]), Cc, C.c_void_p(_s())), "wte_bwd")
    _bump(2)
