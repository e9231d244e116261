"""Host-side executor of the action programs over torch.distributed point-to-point messages.

The same per-rank programs the GPU kernel runs (src/coll/*.cc, obtained as JSON through the schedule
layer) are executed here on CPU tensors, one process per rank, FIFO entries travelling as ordered
`isend`/`recv` pairs of the process group (gloo on machines without GPUs).  It exists to check the
schedules in a real multi-process setting and to let the algorithms be tried where no GPU is present;
it is not a fast path.
"""
from __future__ import annotations

import json
from typing import Optional

import torch
import torch.distributed as dist

from .. import schedule as S

_OPS = {
    "sum": lambda a, b: a + b,
    "prod": lambda a, b: a * b,
    "max": torch.maximum,
    "min": torch.minimum,
}


def run_program(prog: dict, send: torch.Tensor, recv: Optional[torch.Tensor], op: str = "sum", group=None) -> None:
    """Executes one rank's program.  `send` / `recv` are flat CPU tensors (recv may be None where the
    collective defines no output on this rank)."""
    rank = prog["rank"]
    scratch = torch.empty(max(int(prog["scratch_elems"]), 1), dtype=send.dtype)
    bufs = {"in": send, "out": recv, "scratch": scratch}
    red = _OPS[op]
    pending = []
    for a in prog["actions"]:
        n = a["count"]
        parts = []          # (rank of the contributor, tensor) — combined in rank order like the device kernel
        if a["src"] != "none":
            parts.append((rank, bufs[a["src"]][a["src_off"]:a["src_off"] + n].clone()))
        for p in a["recv"]:
            t = torch.empty(n, dtype=send.dtype)
            dist.recv(t, src=p, group=group)
            parts.append((p, t))
        parts.sort(key=lambda x: x[0])
        val = parts[0][1]
        for _, t in parts[1:]:
            val = red(val, t)
        if a["dst"] != "none":
            bufs[a["dst"]][a["dst_off"]:a["dst_off"] + n] = val
        for p in a["send"]:
            pending.append(dist.isend(val.clone(), dst=p, group=group))
    for w in pending:
        w.wait()


def host_collective(coll: str, algo: str, send: torch.Tensor, recv: Optional[torch.Tensor], count: int, k: int = -1, root: int = 0,
                    op: str = "sum", group=None) -> None:
    """`count`: elements per rank for allgather / reduce_scatter, total elements otherwise (as in the C API)."""
    rank, n = dist.get_rank(group), dist.get_world_size(group)
    prog = json.loads(S.schedule_json(coll, algo, n, count, rank, k=k, root=root, elem_size=send.element_size()))
    run_program(prog, send, recv, op=op, group=group)
