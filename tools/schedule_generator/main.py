#!/usr/bin/env python
"""Schedule generator: writes the transfer list of a collective algorithm as schedule XML.

Same command line and output format as the reference's tools/schedule_generator/main.py:14-44
(`--collective --num_nodes --buffer_size --algorithm --k --output`), but the transfers come from
the native schedule compiler that also drives the GPU executor (src/coll/*.cc through
piccl_sched_xml), so the model and the library cannot drift apart.  All six algorithms exist for
all five collectives, sizes are integers and the XML is well formed (the reference's generator
fails for several combinations: allreduce/reduce_scatter `ring`, every RD/RM/PRD/PRM of
bcast/reduce/reduce_scatter).

`--buffer_size` is the size in bytes of the whole buffer; for allgather and reduce_scatter each
node contributes buffer_size / num_nodes.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from piccl_b200 import schedule as S  # noqa: E402

COLLECTIVES = {"allgather": "allgather", "allreduce": "allreduce", "reduce": "reduce", "bcast": "broadcast", "broadcast": "broadcast",
               "reduce_scatter": "reduce_scatter"}
ALGORITHMS = {"ring": "RING", "k_ring": "K_RING", "rd": "RD", "rm": "RM", "prd": "PRD", "prm": "PRM", "direct": "DIRECT"}


def generate(collective: str, num_nodes: int, buffer_size: int, algorithm: str = "ring", k: int = 1, root: int = 0) -> str:
    if collective not in COLLECTIVES:
        raise ValueError(f"Unsupported collective operation: {collective}")
    algo = ALGORITHMS.get(algorithm.lower())
    if algo is None:
        raise ValueError(f"Unsupported algorithm: {algorithm}")
    coll = COLLECTIVES[collective]
    count = buffer_size // num_nodes if coll in ("allgather", "reduce_scatter") else buffer_size
    if count < 1:
        raise ValueError("buffer_size is too small for the number of nodes")
    return S.schedule_xml(coll, algo, num_nodes, count, k=k, root=root, elem_size=1)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Generate collective communication schedules.")
    ap.add_argument("--collective", type=str, required=True, help="allgather, allreduce, reduce, bcast, reduce_scatter")
    ap.add_argument("--num_nodes", type=int, required=True)
    ap.add_argument("--buffer_size", type=int, required=True, help="bytes of the whole buffer")
    ap.add_argument("--algorithm", type=str, default="ring", help="ring, k_ring, RD, RM, PRD, PRM, direct")
    ap.add_argument("--k", type=int, default=1, help="group size (k_ring) or radix (RM, PRM)")
    ap.add_argument("--root", type=int, default=0)
    ap.add_argument("--output", type=str, required=True)
    a = ap.parse_args(argv)
    xml = generate(a.collective, a.num_nodes, a.buffer_size, a.algorithm, a.k, a.root)
    with open(a.output, "w") as f:
        f.write(xml)
    print(f"Schedule generated and saved to {a.output}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
