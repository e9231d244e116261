#!/usr/bin/env python
"""Per-rank send / receive lists of a schedule, and the matcher that joins them into schedule XML.

The reference keeps three unfinished experiments under tools/schedule_generator/saved/:
a per-rank ring allgather that returns `(sends, recvs)` lists of dictionaries
(saved/coll/allgather.py:16-62), a matcher that was meant to pair those lists into `<transfer>`
lines (saved/schedule_gen.py:3-70, does not parse) and a stand-alone k-ring generator
(saved/k-ring.py:3-285, allreduce missing).  This module finishes the idea for every collective
and algorithm of the library:

  rank_lists()  the ordered sends and receives of one rank, taken from that rank's compiled
                action program (the same program the GPU executor runs);
  match()       pairs the k-th send on every directed connection with the k-th receive,
                derives the dependencies (what the sending action had to receive first) and
                writes the transfer list in the simulator's XML format;
  k_ring_xml()  the stand-alone k-ring entry point of saved/k-ring.py, for all five collectives.

`match(all ranks' lists)` reproduces, transfer for transfer, what the native dump
(`piccl_sched --xml`, src/coll/dump.cc) writes; tests/test_tools_cpu.py checks that.
"""
from __future__ import annotations

import argparse
import json
import sys
from collections import defaultdict, deque
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from piccl_b200 import schedule as S  # noqa: E402

from tools.schedule_generator.main import ALGORITHMS, COLLECTIVES  # noqa: E402


def _program(coll: str, algo: str, n: int, count: int, rank: int, k: int, root: int) -> dict:
    return json.loads(S.schedule_json(coll, algo, n, count, rank, k=k, root=root, elem_size=1))


def _count(coll: str, n: int, buffer_size: int) -> int:
    count = buffer_size // n if coll in ("allgather", "reduce_scatter") else buffer_size
    if count < 1:
        raise ValueError("buffer_size is too small for the number of nodes")
    return count


def rank_lists(collective: str, num_nodes: int, buffer_size: int, rank: int, algorithm: str = "ring", k: int = 1, root: int = 0):
    """(sends, recvs) of `rank`, in program order.

    Every entry is a dictionary with the keys of the reference's lists (`from`, `to`, `size`,
    `tag`, `type`; receives also `offset`, sends also `deps`) plus `step` and `action`:
      tag     position of the message on its directed connection (k-th message from -> to);
      offset  byte offset in the receive buffer where the data lands, -1 if it is only forwarded;
      deps    the receives, as (from, tag) pairs, that the sending action consumes; if it consumes
              none, the receives of the latest earlier step that had any.
    """
    coll = COLLECTIVES[collective]
    algo = ALGORITHMS[algorithm.lower()]
    prog = _program(coll, algo, num_nodes, _count(coll, num_nodes, buffer_size), rank, k, root)
    sends, recvs = [], []
    send_tag, recv_tag = defaultdict(int), defaultdict(int)
    last_in, cur_in, last_step = [], [], None
    for ai, ac in enumerate(prog["actions"]):
        if ac["step"] != last_step:
            if cur_in:
                last_in = cur_in
            cur_in, last_step = [], ac["step"]
        incoming = []
        for p in ac["recv"]:
            t = recv_tag[p]
            recv_tag[p] += 1
            incoming.append((p, t))
            recvs.append({"from": p, "to": rank, "offset": ac["dst_off"] if ac["dst"] == "out" else -1, "size": ac["count"], "tag": t,
                          "type": "recv", "step": ac["step"], "action": ai})
        for p in ac["send"]:
            t = send_tag[p]
            send_tag[p] += 1
            sends.append({"from": rank, "to": p, "deps": list(incoming) if incoming else list(last_in), "size": ac["count"], "tag": t,
                          "type": "send", "step": ac["step"], "action": ai})
        cur_in.extend(incoming)
    return sends, recvs


def all_rank_lists(collective: str, num_nodes: int, buffer_size: int, algorithm: str = "ring", k: int = 1, root: int = 0):
    return [rank_lists(collective, num_nodes, buffer_size, r, algorithm, k, root) for r in range(num_nodes)]


def match(lists, collective: str, algorithm: str, buffer_size: int, k: int | None = None) -> str:
    """Joins the per-rank lists into schedule XML.

    Raises ValueError if a send has no receive (or the other way round), or if the two ends of a
    message disagree about its size: the checks the reference's matcher was going to make with its
    `send_waiting` / `recv_waiting` sets.
    """
    n = len(lists)
    posted = defaultdict(deque)          # (from, to) -> receives in posting order
    for r, (_, recvs) in enumerate(lists):
        for rc in recvs:
            posted[(rc["from"], r)].append(rc)
    # transfer ids in (step, rank, program order) order, like the native dump
    order = sorted(((s["step"], r, i) for r, (sends, _) in enumerate(lists) for i, s in enumerate(sends)))
    ids = {}
    for tid, (_, r, i) in enumerate(order):
        s = lists[r][0][i]
        ids[(r, s["to"], s["tag"])] = tid
    for r, (sends, _) in enumerate(lists):
        for s in sends:
            q = posted[(r, s["to"])]
            if not q:
                raise ValueError(f"send {r}->{s['to']} tag {s['tag']} has no matching receive")
            rc = q.popleft()
            if rc["tag"] != s["tag"] or rc["size"] != s["size"]:
                raise ValueError(f"send {r}->{s['to']} tag {s['tag']} size {s['size']} meets receive tag {rc['tag']} size {rc['size']}")
    left = [(key, len(q)) for key, q in posted.items() if q]
    if left:
        raise ValueError(f"receives without a send: {left}")
    head = f'<collective name="{COLLECTIVES[collective]}" algorithm="{algorithm.lower()}"'
    if k is not None and k > 0:
        head += f' k="{k}"'
    out = [head + f' nodes="{n}" buffer_size="{buffer_size}">']
    step = None
    for tid, (st, r, i) in enumerate(order):
        s = lists[r][0][i]
        if st != step:
            step = st
            out.append(f"\n    # (round {step})")
        deps = ",".join(str(ids[(p, r, t)]) for p, t in s["deps"]) or "-1"
        out.append(f'    <transfer id="{tid}" size="{s["size"]}" src="{r}" dst="{s["to"]}" deps="{deps}"/>')
    out.append("</collective>\n")
    return "\n".join(out)


def k_ring_xml(num_nodes: int, buffer_size: int, k: int, collective: str, root: int = 0) -> str:
    """Stand-alone k-ring generator (reference: saved/k-ring.py `KRingScheduleGenerator`), all five collectives."""
    if k < 1 or num_nodes % k != 0:
        raise ValueError("Number of nodes must be divisible by k.")
    return match(all_rank_lists(collective, num_nodes, buffer_size, "k_ring", k, root), collective, "k_ring", buffer_size, k)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Per-rank send/receive lists of a schedule; --xml joins them into schedule XML.")
    ap.add_argument("--collective", required=True)
    ap.add_argument("--num_nodes", type=int, required=True)
    ap.add_argument("--buffer_size", type=int, required=True)
    ap.add_argument("--algorithm", default="ring")
    ap.add_argument("--k", type=int, default=1)
    ap.add_argument("--root", type=int, default=0)
    ap.add_argument("--rank", type=int, default=None, help="print the lists of this rank (default: all ranks)")
    ap.add_argument("--xml", action="store_true", help="match the lists of all ranks and print schedule XML")
    a = ap.parse_args(argv)
    if a.xml:
        print(match(all_rank_lists(a.collective, a.num_nodes, a.buffer_size, a.algorithm, a.k, a.root), a.collective, a.algorithm, a.buffer_size), end="")
        return 0
    ranks = range(a.num_nodes) if a.rank is None else [a.rank]
    for r in ranks:
        sends, recvs = rank_lists(a.collective, a.num_nodes, a.buffer_size, r, a.algorithm, a.k, a.root)
        print(json.dumps({"rank": r, "sends": sends, "recvs": recvs}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
