#!/usr/bin/env python
"""LogGP(+contention) simulator for collective schedules.

    python tools/loggp_sim/sim.py --schedule S.xml --topo T.xml --radix R [--compat] [--output stats.json]

prints one line: the finish time of the last transfer in microseconds (same contract as the
reference's tools/loggp_sim/sim.py:156-165, which this replaces).  File formats are the
reference's (tools/loggp_sim/README.md:13-55): schedule XML (<transfer id size src dst deps/>),
hierarchical topology XML (<group level id param_file [ports]> / <node id>), LogGP CSV
(s,L,o_s,o_r,g,G; linear interpolation, clamped at both ends).

Model.  A transfer of s bytes from a to b:
    start (all deps done) -> +o_s -> wait for one of the `radix` send ports of a (and, if a and b are
    in different level-0 groups, one of the source group's NICs) -> the bytes take G(s-1) ->
    +L -> wait for the destination group's NIC / a receive port of b -> +o_r -> done.
  default ("clean", the classical LogGP of the fixture comments): the per-byte term is charged
    once (done = start + o_s + G(s-1) + L + o_r when nothing is contended), consecutive messages
    on a port are at least max(g, G s) apart, a NIC is busy for G s per message.  Optional
    --gamma adds a reduction cost per received byte, --alpha a fixed cost per transfer (kernel
    launch of the reference's one-launch-per-step design).
  --compat reproduces the behaviour of the simulator the reference ships, including its quirks:
    G(s-1) is charged on the send side and again on the receive side; the send gap g counts from
    the END of the previous send on the port, the receive gap from the START of the previous
    receive; a NIC is busy for G s.
Large transfers cost the same closed form (no per-4-KiB events), so 1 GiB schedules simulate
instantly.  A NIC serves whole messages in arrival order; the reference streams 4096-byte chunks
through its NIC queues (schedulers/loggpc_scheduler.py:22,284-377), which interleaves messages that
share a NIC: the LAST of them ends at the same time in both models (the NIC is never idle), the
earlier ones end later there.  tests/test_tools_cpu.py compares the two on large transfers.

Contention statistics (--output; reference: sim.py:124-153, loggpc_scheduler.py:272-291,411-428)
are kept per level-0 group of the topology, for the send side (the group of the source) and the
receive side (the group of the destination): attempts (one per transfer), success (started without
waiting for a port or a NIC), the time waited, and the largest number of transfers that were
waiting at the same time.  --output x.json writes them with the per-transfer times; any other
name gets a text report in the layout of the reference's.
"""
from __future__ import annotations

import argparse
import heapq
import json
import sys
import xml.etree.ElementTree as ET
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parents[2]


def get_path(p: str) -> Path:
    q = Path(p)
    if q.is_absolute() or q.exists():
        return q
    return REPO / p


# ------------------------------------------------------------------ inputs
@dataclass
class Task:
    id: int
    src: int
    dst: int
    size: int
    deps: set
    children: list = field(default_factory=list)
    start: float = -1.0
    done: float = -1.0


def parse_schedule(path) -> tuple[dict, dict]:
    # free text such as "# (round 3)" between the elements is character data and is ignored
    root = ET.parse(get_path(str(path))).getroot()
    tasks: dict[int, Task] = {}
    for t in root.iter("transfer"):
        size = t.get("size")
        try:
            nbytes = int(size)
        except (TypeError, ValueError):
            raise ValueError(f"transfer {t.get('id')}: size {size!r} is not an integer")
        deps = {int(d) for d in (t.get("deps") or "-1").split(",") if d.strip() and int(d) >= 0}
        tid = int(t.get("id"))
        if tid in tasks:
            raise ValueError(f"duplicate transfer id {tid}")
        tasks[tid] = Task(tid, int(t.get("src")), int(t.get("dst")), nbytes, deps)
    for t in tasks.values():
        for d in t.deps:
            if d not in tasks:
                raise ValueError(f"transfer {t.id} depends on unknown transfer {d}")
            tasks[d].children.append(t.id)
    return tasks, dict(root.attrib)


class Profile:
    """One LogGP CSV, interpolated per parameter."""

    def __init__(self, path):
        data = np.genfromtxt(get_path(str(path)), delimiter=",", names=True)
        data = np.atleast_1d(data)
        self.s = np.asarray(data["s"], dtype=float)
        order = np.argsort(self.s)
        self.s = self.s[order]
        self.cols = {k: np.asarray(data[k], dtype=float)[order] for k in ("L", "o_s", "o_r", "g", "G")}

    def __call__(self, name: str, size: float) -> float:
        return float(np.interp(size, self.s, self.cols[name]))


@dataclass
class Topology:
    nodes: list
    group0: dict                 # node -> level-0 group key
    nics: dict                   # level-0 group key -> NIC count (None: unlimited)
    chain: dict                  # node -> list of (level, group key, param file) from innermost outwards

    def pair_profile_file(self, a: int, b: int) -> str:
        keys_b = {k for _, k, _ in self.chain[b]}
        for _, k, f in self.chain[a]:
            if k in keys_b:
                return f
        raise ValueError(f"nodes {a} and {b} share no group")


def parse_topology(path) -> Topology:
    root = ET.parse(get_path(str(path))).getroot()
    nodes, group0, nics, chain = [], {}, {}, {}

    def walk(el, stack):
        for ch in el:
            if ch.tag == "group":
                key = (int(ch.get("level")), ch.get("id"), len(stack), id(ch))
                entry = (int(ch.get("level")), key, ch.get("param_file"))
                if int(ch.get("level")) == 0:
                    p = ch.get("ports")
                    nics[key] = int(p) if p is not None and int(p) > 0 else None
                walk(ch, stack + [entry])
            elif ch.tag == "node":
                n = int(ch.get("id"))
                nodes.append(n)
                chain[n] = list(reversed(stack))
                lvl0 = [e for e in stack if e[0] == 0]
                group0[n] = lvl0[-1][1] if lvl0 else ("flat",)

    walk(root, [])
    return Topology(sorted(nodes), group0, nics, chain)


def flat_topology_xml(n: int, param_file: str) -> str:
    nodes = "".join(f'<node id="{i}"/>' for i in range(n))
    return f'<topo num_nodes="{n}" num_levels="1"><group level="0" id="0" param_file="{param_file}">{nodes}</group></topo>'


# ------------------------------------------------------------------ engine
class Ports:
    """`count` interchangeable ports with a minimum spacing between uses."""

    def __init__(self, count):
        self.free = [0.0] * count          # busy until
        self.mark = [-1e300] * count       # reference point of the gap rule (start or end of the last use)
        self.after = [0.0] * count         # classical model: the gap the LAST use of the port imposes, max(g, G s) of that message

    def reserve(self, t: float, gap):
        """earliest (time, port) at which a use may start for a request made at t.
        gap: spacing from the port's mark; None = the spacing recorded by the port's previous use (`after`)"""
        best, bi = None, 0
        for i in range(len(self.free)):
            s = max(t, self.free[i], self.mark[i] + (self.after[i] if gap is None else gap))
            if best is None or s < best:
                best, bi = s, i
        return best, bi


class Simulator:
    def __init__(self, schedule, topo, radix: int = 1, compat: bool = False, gamma: float = 0.0, alpha: float = 0.0):
        self.tasks, self.meta = parse_schedule(schedule) if not isinstance(schedule, dict) else (schedule, {})
        self.topo = parse_topology(topo) if not isinstance(topo, Topology) else topo
        self.radix, self.compat, self.gamma, self.alpha = radix, compat, gamma, alpha
        self.profiles: dict[str, Profile] = {}
        self.send = {n: Ports(radix) for n in self.topo.nodes}
        self.recv = {n: Ports(radix) for n in self.topo.nodes}
        self.nic_s = {k: Ports(c) for k, c in self.topo.nics.items() if c}
        self.nic_r = {k: Ports(c) for k, c in self.topo.nics.items() if c}
        self.stats = {"send_wait": 0.0, "recv_wait": 0.0, "nic_wait": 0.0}
        self.group_stats: dict = {}                     # level-0 group id -> {"send": {...}, "recv": {...}}
        self._waits: dict = {}                          # (group id, side) -> [(asked, started)] of the transfers that waited
        for t in self.tasks.values():
            for n in (t.src, t.dst):
                if n not in self.send:
                    raise ValueError(f"transfer {t.id} uses node {n}, which is not in the topology")

    def _group_id(self, node) -> str:
        k = self.topo.group0[node]
        return str(k[1]) if len(k) > 1 else "flat"

    def _note(self, node, side: str, asked: float, started: float) -> None:
        gid = self._group_id(node)
        st = self.group_stats.setdefault(gid, {x: {"attempts": 0, "success": 0, "waited": 0.0, "max_queue_size": 0} for x in ("send", "recv")})[side]
        st["attempts"] += 1
        if started <= asked:
            st["success"] += 1
        else:
            st["waited"] += started - asked
            self._waits.setdefault((gid, side), []).append((asked, started))

    def _finish_group_stats(self) -> None:
        for (gid, side), iv in self._waits.items():
            ev = sorted([(a, 1) for a, _ in iv] + [(b, -1) for _, b in iv], key=lambda e: (e[0], e[1]))
            cur = best = 0
            for _, d in ev:
                cur += d
                best = max(best, cur)
            self.group_stats[gid][side]["max_queue_size"] = best

    def prof(self, a, b) -> Profile:
        f = self.topo.pair_profile_file(a, b)
        if f not in self.profiles:
            self.profiles[f] = Profile(f)
        return self.profiles[f]

    def run(self) -> float:
        q: list = []
        seq = 0

        def post(t, stage, task):
            nonlocal seq
            heapq.heappush(q, (t, seq, stage, task.id))
            seq += 1

        remaining = {t.id: len(t.deps) for t in self.tasks.values()}
        for t in self.tasks.values():
            if not t.deps:
                post(0.0, 0, t)
        finished, last = 0, 0.0
        arrive_state = {}
        while q:
            now, _, stage, tid = heapq.heappop(q)
            task = self.tasks[tid]
            p = self.prof(task.src, task.dst)
            s = task.size
            G, g = p("G", s), p("g", s)
            wire = G * max(s - 1, 0)
            inter = self.topo.group0[task.src] != self.topo.group0[task.dst]
            if stage == 0:                                   # dependencies done: sender overhead
                task.start = now
                post(now + self.alpha + p("o_s", s), 1, task)
            elif stage == 1:                                 # inject: send port (+ source NIC)
                # reference-compatible: g of this message after the end of the last use; classical: the gap belongs to the
                # message that used the port before (a short message does not make the next, longer one wait for its own length)
                st, pi = self.send[task.src].reserve(now, g if self.compat else None)
                nic = self.nic_s.get(self.topo.group0[task.src]) if inter else None
                if nic is not None:
                    ns, ni = nic.reserve(st, 0.0)
                    self.stats["nic_wait"] += ns - st
                    st = ns
                    nic.free[ni] = st + G * s
                self.stats["send_wait"] += st - now
                self._note(task.src, "send", now, st)
                ports = self.send[task.src]
                ports.free[pi] = st + wire
                ports.mark[pi] = st + wire if self.compat else st
                ports.after[pi] = max(g, G * s)
                arrive_state[tid] = st
                post(st + wire + p("L", s), 2, task)
            elif stage == 2:                                 # arrival: destination NIC, receive port
                if self.compat:
                    st, pi = self.recv[task.dst].reserve(now, g)
                else:
                    # classical: `now` is when the last byte would arrive on an idle port.  A port takes the bytes of one message
                    # at a time, so if another message was still arriving, this one ends max(g, G s) after that one ended.
                    rp = self.recv[task.dst]
                    pi = min(range(len(rp.free)), key=lambda i: rp.free[i])
                    st = max(now, rp.free[pi] + max(g, G * s)) if rp.free[pi] > 0.0 else now
                nic = self.nic_r.get(self.topo.group0[task.dst]) if inter else None
                if nic is not None and self.compat:
                    ns, ni = nic.reserve(st, 0.0)
                    self.stats["nic_wait"] += ns - st
                    st = ns
                    nic.free[ni] = st + G * s
                elif nic is not None:
                    # classical: the destination NIC carries the message WHILE it arrives, from its first byte (st - wire) on,
                    # not after its last byte; a message only waits if the NIC is still taking an earlier one
                    first = st - wire
                    ns, ni = nic.reserve(first, 0.0)
                    self.stats["nic_wait"] += ns - first
                    nic.free[ni] = ns + G * s
                    st += ns - first
                self.stats["recv_wait"] += st - now
                self._note(task.dst, "recv", now, st)
                ports = self.recv[task.dst]
                busy = wire if self.compat else 0.0          # the classical model charges the bytes once
                ports.free[pi] = st + busy
                ports.mark[pi] = st
                post(st + busy + p("o_r", s) + self.gamma * s, 3, task)
            else:                                            # done
                task.done = now
                last = max(last, now)
                finished += 1
                for c in task.children:
                    remaining[c] -= 1
                    if remaining[c] == 0:
                        post(now, 0, self.tasks[c])
        if finished != len(self.tasks):
            raise RuntimeError("Not all tasks completed (dependency cycle in the schedule?)")
        self._finish_group_stats()
        return last

    def output_stats(self, path, args=None) -> None:
        finish = max((t.done for t in self.tasks.values()), default=0.0)
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        if str(path).endswith(".json"):
            out = {"finish_time": finish, **self.stats, "groups": self.group_stats,
                   "tasks": {str(t.id): {"start": t.start, "done": t.done, "src": t.src, "dst": t.dst, "size": t.size} for t in self.tasks.values()}}
            Path(path).write_text(json.dumps(out, indent=1))
            return
        # the text report of the reference's simulator (same headings), per level-0 group
        lines = ["LogGP Simulation Output", "", "====================================", "", "Simulation args:"]
        if args is not None:
            lines += [f"  Schedule: {args.schedule}", f"  Topology: {args.topo}", f"  Device radix: {args.radix}", f"  Output file: {args.output}"]
        lines += ["", "====================================", "", "Simulation Overview:", f"  Simulation finished at time {finish * 1e6} us",
                  f"  Number of tasks: {len(self.tasks)}", f"  Number of completed tasks: {sum(1 for t in self.tasks.values() if t.done >= 0)}",
                  "", "====================================", "", "Scheduler Statistics:"]
        for side, title in (("send", "Send Contention"), ("recv", "Recv Contention")):
            lines.append(f"  {title}: ")
            for gid in sorted(self.group_stats):
                st = self.group_stats[gid][side]
                if st["attempts"]:
                    lines.append(f"    Group {gid}: {st['success']} / {st['attempts']} = {st['success'] / st['attempts']} attempts successful")
                    lines.append(f"    Max Queue Size: {st['max_queue_size']}")
                    lines.append(f"    Time waited: {st['waited'] * 1e6} us")
        Path(path).write_text("\n".join(lines) + "\n")


def simulate(schedule, topo, radix=1, compat=False, gamma=0.0, alpha=0.0) -> float:
    """Finish time in the time unit of the parameter files (seconds for measured profiles)."""
    return Simulator(schedule, topo, radix, compat, gamma, alpha).run()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="LogGP collective schedule simulator")
    ap.add_argument("--schedule", required=True)
    ap.add_argument("--topo", required=True)
    ap.add_argument("--radix", type=int, default=1, help="concurrent send ports and receive ports per device")
    ap.add_argument("--compat", action="store_true", help="reproduce the cost accounting of the simulator shipped with the reference")
    ap.add_argument("--gamma", type=float, default=0.0, help="reduction cost per received byte")
    ap.add_argument("--alpha", type=float, default=0.0, help="fixed cost per transfer")
    ap.add_argument("--output", default=None, help="write per-transfer times and contention statistics (JSON)")
    a = ap.parse_args(argv)
    sim = Simulator(a.schedule, a.topo, a.radix, a.compat, a.gamma, a.alpha)
    t = sim.run()
    if a.output:
        sim.output_stats(a.output, a)
    print(t * 1e6)
    return 0


if __name__ == "__main__":
    sys.exit(main())
