"""Bucketed data-parallel gradient averaging over a flat gradient buffer.

The model reports, during its backward pass, that `flat_g[:end]` is final; every
bucket (25 MiB by default, the size PyTorch DDP uses) that became complete is
averaged across ranks on a separate stream by the fused all-reduce, overlapping
the rest of the backward pass.  The optimizer waits for the last bucket.

This is what the reference gets from torch DDP calling the intercepted
ncclAllReduce; here the buckets are slices of one buffer, so there is no
gradient copy in or out.
"""
from __future__ import annotations

from typing import Optional

import torch

from .comm import Communicator


class GradAverager:
    def __init__(self, flat_g: torch.Tensor, comm: Optional[Communicator], bucket_bytes: int = 25 * 1024 * 1024, algo: str = "AUTO", k: int = -1):
        self.flat_g = flat_g
        self.comm = comm
        self.algo, self.k = algo, k
        self.bucket_elems = max(1, bucket_bytes // flat_g.element_size()) // 8 * 8
        self.n = flat_g.numel()
        self.done = 0
        self.stream = torch.cuda.Stream() if comm is not None and comm.nranks > 1 else None
        self.launched = 0

    def begin_step(self) -> None:
        self.done = 0

    def ready(self, end: int) -> None:
        """flat_g[:end] is final."""
        if self.stream is None:
            return
        final = end >= self.n
        while self.done < end:
            nxt = min(self.done + self.bucket_elems, self.n)
            if nxt > end and not final:
                break
            nxt = min(nxt, end) if final else nxt
            ev = torch.cuda.Event()
            ev.record()
            self.stream.wait_event(ev)
            bucket = self.flat_g[self.done:nxt]
            self.comm.all_reduce(bucket, op="avg", algo=self.algo, k=self.k, stream=self.stream)
            self.launched += 1
            self.done = nxt

    def finish(self) -> None:
        """Make the current stream wait for all bucket reductions."""
        if self.stream is None:
            return
        torch.cuda.current_stream().wait_stream(self.stream)
