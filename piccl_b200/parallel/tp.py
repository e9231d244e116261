"""Fused tensor-parallel operations (tcgen05 GEMM + collective in one kernel, src/tp/tp_kernels.cu).

    gemm_rs(comm, A[M, K/n], B[N, K/n], out[M/n, N])      out = rows of rank r of  sum_r A_r @ B_r^T
    ag_gemm(comm, A[M/n, K], B[N/n, K], out[M, N/n])      out = concat_r(A_r) @ B^T

The communicator must have been created with a workspace (`make_config(tp_bytes=workspace_bytes(...))`).
`*_group` run virtual ranks of a LoopbackGroup in one cooperative launch (single-GPU testing).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N
from .comm import Communicator, LoopbackGroup, _stream_ptr


def _declare():
    lib = N.lib()
    if getattr(lib, "_tp_declared", False):
        return lib
    vp, i = C.c_void_p, C.c_int
    lib.piccl_tp_workspace_bytes.argtypes = [i, i, i, i, i]
    lib.piccl_tp_workspace_bytes.restype = C.c_longlong
    lib.piccl_gemm_rs.argtypes = [vp, vp, vp, vp, i, i, i, vp]
    lib.piccl_ag_gemm.argtypes = [vp, vp, vp, vp, i, i, i, vp]
    lib.piccl_gemm_rs_group.argtypes = [C.POINTER(vp), i, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), i, i, i, vp]
    lib.piccl_ag_gemm_group.argtypes = [C.POINTER(vp), i, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), i, i, i, vp]
    lib.piccl_tp_status.argtypes = [vp]
    lib._tp_declared = True
    return lib


def workspace_bytes(which: str, nranks: int, M: int, N_: int, K: int) -> int:
    return int(_declare().piccl_tp_workspace_bytes(0 if which == "gemm_rs" else 1, nranks, M, N_, K))


def _check(*ts):
    for t in ts:
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ValueError("operands must be contiguous bf16 tensors")


def gemm_rs(comm: Communicator, A: torch.Tensor, B: torch.Tensor, out: torch.Tensor, stream=None) -> torch.Tensor:
    _check(A, B, out)
    M, Kl = A.shape
    N.check(_declare().piccl_gemm_rs(comm._h, A.data_ptr(), B.data_ptr(), out.data_ptr(), M, B.shape[0], Kl, _stream_ptr(stream)), "piccl_gemm_rs")
    return out


def ag_gemm(comm: Communicator, A_shard: torch.Tensor, B: torch.Tensor, out: torch.Tensor, stream=None) -> torch.Tensor:
    _check(A_shard, B, out)
    Ms, K = A_shard.shape
    N.check(_declare().piccl_ag_gemm(comm._h, A_shard.data_ptr(), B.data_ptr(), out.data_ptr(), Ms * comm.nranks, B.shape[0], K, _stream_ptr(stream)), "piccl_ag_gemm")
    return out


def tp_status(comm_or_handle) -> int:
    h = comm_or_handle._h if isinstance(comm_or_handle, Communicator) else comm_or_handle
    return int(_declare().piccl_tp_status(h))


def _group(fn_name, g: LoopbackGroup, As, Bs, outs, M, N_, K, stream):
    lib = _declare()
    n = g.nranks
    comms = (C.c_void_p * n)(*[h.value for h in g._hs])
    a = (C.c_void_p * n)(*[t.data_ptr() for t in As])
    b = (C.c_void_p * n)(*[t.data_ptr() for t in Bs])
    o = (C.c_void_p * n)(*[t.data_ptr() for t in outs])
    N.check(getattr(lib, fn_name)(comms, n, a, b, o, M, N_, K, _stream_ptr(stream)), fn_name)


def gemm_rs_group(g: LoopbackGroup, As, Bs, outs, stream=None):
    _check(*As, *Bs, *outs)
    _group("piccl_gemm_rs_group", g, As, Bs, outs, As[0].shape[0], Bs[0].shape[0], As[0].shape[1], stream)


def ag_gemm_group(g: LoopbackGroup, As, Bs, outs, stream=None):
    _check(*As, *Bs, *outs)
    _group("piccl_ag_gemm_group", g, As, Bs, outs, As[0].shape[0] * g.nranks, Bs[0].shape[0], As[0].shape[1], stream)
