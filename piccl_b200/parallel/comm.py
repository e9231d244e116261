"""Communicators over the native peer-memory runtime.

`Communicator` is one rank of a multi-process job (one process per GPU); the
heap handles are exchanged through torch.distributed.  `LoopbackGroup` holds
several virtual ranks on ONE device inside one process and runs each collective
as a single cooperative kernel launch — the way to exercise the multi-rank
protocol when only one GPU is at hand.

The collectives mirror the reference's intercepted entry points
(src/piccl.c:29-173) but can also be called directly, with the algorithm and k
per call instead of through the environment.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from .. import _native as N

_TORCH_DTYPE = {
    torch.int8: "int8", torch.uint8: "uint8", torch.int32: "int32", torch.int64: "int64",
    torch.float16: "float16", torch.float32: "float32", torch.float64: "float64", torch.bfloat16: "bfloat16",
}


def _dt(t: torch.Tensor) -> int:
    try:
        return N.DTYPE[_TORCH_DTYPE[t.dtype]]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}")


def _stream_ptr(stream: Optional[torch.cuda.Stream]) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


def _algo(algo) -> int:
    return algo if isinstance(algo, int) else N.ALGO[algo.upper()]


def make_config(max_cta=0, nslot=0, slot_bytes=0, scratch_bytes=0, block_size=0, timeout_ms=0, tp_bytes=0, nvls_cta=0) -> N.Config:
    """0 everywhere: the library's defaults / PICCL_* environment.  nvls_cta: CTAs of the in-switch collectives (the default, 128,
    is for stand-alone bandwidth; 48 leaves room for a backward pass that runs at the same time)."""
    return N.Config(max_cta, nslot, slot_bytes, scratch_bytes, block_size, timeout_ms, tp_bytes, nvls_cta)


class _CommBase:
    def __init__(self):
        self._lib = N.lib()

    def _check_contig(self, *ts):
        for t in ts:
            if t is not None and not t.is_contiguous():
                raise ValueError("tensors must be contiguous")


class Communicator(_CommBase):
    """One rank.  `exchange(handle_bytes) -> list of all ranks' handle bytes` may be given;
    by default torch.distributed (already initialised) is used."""

    def __init__(self, rank: Optional[int] = None, nranks: Optional[int] = None, device: Optional[int] = None,
                 config: Optional[N.Config] = None, exchange=None, group=None):
        super().__init__()
        import torch.distributed as dist
        if rank is None:
            rank, nranks = dist.get_rank(group), dist.get_world_size(group)
        if device is None:
            device = torch.cuda.current_device()
        self.rank, self.nranks, self.device = rank, nranks, device
        self._h = C.c_void_p()
        N.check(self._lib.piccl_comm_create(rank, nranks, device, C.byref(config) if config else None, C.byref(self._h)), "piccl_comm_create")
        mine = N.Handle()
        N.check(self._lib.piccl_comm_local_handle(self._h, C.byref(mine)), "piccl_comm_local_handle")
        blob = bytes(mine.bytes)
        if exchange is not None:
            blobs = exchange(blob)
        elif nranks == 1:
            blobs = [blob]
        else:
            blobs = [None] * nranks
            dist.all_gather_object(blobs, blob, group=group)
        arr = (N.Handle * nranks)()
        for i, b in enumerate(blobs):
            C.memmove(C.byref(arr[i]), b, 128)
        N.check(self._lib.piccl_comm_connect(self._h, arr), "piccl_comm_connect")
        if nranks > 1 and exchange is None:
            dist.barrier(group=group)   # nobody pushes before everybody has mapped

    # ---- collectives (stream ordered) ----
    def all_reduce(self, send: torch.Tensor, recv: Optional[torch.Tensor] = None, op: str = "sum", algo="AUTO", k: int = -1, stream=None):
        recv = send if recv is None else recv
        self._check_contig(send, recv)
        N.check(self._lib.piccl_allreduce(self._h, send.data_ptr(), recv.data_ptr(), send.numel(), _dt(send), N.OP[op], _algo(algo), k, _stream_ptr(stream)), "piccl_allreduce")
        return recv

    def all_gather(self, send: torch.Tensor, recv: torch.Tensor, algo="AUTO", k: int = -1, stream=None):
        self._check_contig(send, recv)
        assert recv.numel() == send.numel() * self.nranks
        N.check(self._lib.piccl_allgather(self._h, send.data_ptr(), recv.data_ptr(), send.numel(), _dt(send), _algo(algo), k, _stream_ptr(stream)), "piccl_allgather")
        return recv

    def reduce_scatter(self, send: torch.Tensor, recv: torch.Tensor, op: str = "sum", algo="AUTO", k: int = -1, stream=None):
        self._check_contig(send, recv)
        assert send.numel() == recv.numel() * self.nranks
        N.check(self._lib.piccl_reduce_scatter(self._h, send.data_ptr(), recv.data_ptr(), recv.numel(), _dt(send), N.OP[op], _algo(algo), k, _stream_ptr(stream)), "piccl_reduce_scatter")
        return recv

    def reduce(self, send: torch.Tensor, recv: Optional[torch.Tensor], root: int = 0, op: str = "sum", algo="AUTO", k: int = -1, stream=None):
        self._check_contig(send, recv)
        rp = recv.data_ptr() if recv is not None else 0
        N.check(self._lib.piccl_reduce(self._h, send.data_ptr(), rp, send.numel(), _dt(send), N.OP[op], root, _algo(algo), k, _stream_ptr(stream)), "piccl_reduce")
        return recv

    def broadcast(self, tensor: torch.Tensor, root: int = 0, recv: Optional[torch.Tensor] = None, algo="AUTO", k: int = -1, stream=None):
        recv = tensor if recv is None else recv
        self._check_contig(tensor, recv)
        N.check(self._lib.piccl_broadcast(self._h, tensor.data_ptr(), recv.data_ptr(), tensor.numel(), _dt(tensor), root, _algo(algo), k, _stream_ptr(stream)), "piccl_broadcast")
        return recv

    # ---- state ----
    def status(self) -> N.Status:
        s = N.Status()
        self._lib.piccl_comm_status(self._h, C.byref(s))
        return s

    def stats(self) -> N.Stats:
        s = N.Stats()
        self._lib.piccl_get_stats(self._h, C.byref(s))
        return s

    def abort(self):
        self._lib.piccl_comm_abort(self._h)

    def unmatched_wait(self, timeout_ms: int = 200, stream=None):
        """Launches a kernel that waits for data nobody sends (bounded); see piccl_test_unmatched_wait."""
        N.check(self._lib.piccl_test_unmatched_wait(self._h, timeout_ms, _stream_ptr(stream)), "piccl_test_unmatched_wait")

    def close(self):
        if self._h:
            self._lib.piccl_comm_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class LoopbackGroup(_CommBase):
    """`nranks` virtual ranks on one device; every collective is one cooperative launch."""

    def __init__(self, nranks: int, device: Optional[int] = None, config: Optional[N.Config] = None):
        super().__init__()
        if device is None:
            device = torch.cuda.current_device()
        self.nranks, self.device = nranks, device
        self._hs = []
        blobs = []
        for r in range(nranks):
            h = C.c_void_p()
            N.check(self._lib.piccl_comm_create(r, nranks, device, C.byref(config) if config else None, C.byref(h)), "piccl_comm_create")
            self._hs.append(h)
            mine = N.Handle()
            N.check(self._lib.piccl_comm_local_handle(h, C.byref(mine)), "piccl_comm_local_handle")
            blobs.append(bytes(mine.bytes))
        arr = (N.Handle * nranks)()
        for i, b in enumerate(blobs):
            C.memmove(C.byref(arr[i]), b, 128)
        for h in self._hs:
            N.check(self._lib.piccl_comm_connect(h, arr), "piccl_comm_connect")

    def run(self, coll: str, send: Sequence[torch.Tensor], recv: Sequence[Optional[torch.Tensor]], count: int, op: str = "sum",
            root: int = 0, algo="RING", k: int = -1, stream=None):
        n = self.nranks
        comms = (C.c_void_p * n)(*[h.value for h in self._hs])
        sp = (C.c_void_p * n)(*[t.data_ptr() for t in send])
        rp = (C.c_void_p * n)(*[(t.data_ptr() if t is not None else 0) for t in recv])
        N.check(self._lib.piccl_group_collective(comms, n, N.COLL[coll], sp, rp, count, _dt(send[0]), N.OP[op], root, _algo(algo), k, _stream_ptr(stream)),
                f"piccl_group_collective({coll})")

    def status(self, rank: int = 0) -> N.Status:
        s = N.Status()
        self._lib.piccl_comm_status(self._hs[rank], C.byref(s))
        return s

    def stats(self, rank: int = 0) -> N.Stats:
        s = N.Stats()
        self._lib.piccl_get_stats(self._hs[rank], C.byref(s))
        return s

    def close(self):
        for h in self._hs:
            self._lib.piccl_comm_destroy(h)
        self._hs = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
