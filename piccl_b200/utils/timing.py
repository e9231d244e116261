"""Device-side timing helpers: CUDA events on the launching stream, warm-up, L2 flush."""
from __future__ import annotations

import torch

_flush_buf = None


def l2_flush() -> None:
    """Writes a buffer larger than the 126 MB L2 so the next kernel starts cold."""
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def time_cuda(fn, iters: int = 10, warmup: int = 3, flush: bool = True) -> float:
    """Median milliseconds of `fn()` over `iters` runs, each bracketed by events."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            l2_flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]
