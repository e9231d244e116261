"""Exhaustive interleaving check of the counter / slot protocol of the in-switch collectives
(src/kernels/nvls_coll.cu, described in src/kernels/nvls.cuh), on a small model: two ranks, one CTA index with its
warp groups (fill, switch, out; the one that talks to the switch split in two) running on their own, a few chunks, several calls of different collectives in a row.

Every warp group runs the kernel's sequence of phases; the explorer tries every order in which the groups can advance and
in which counter arrivals can reach each rank (an arrival is delivered to every rank separately, in any order).  Data is
modelled as tags per (rank's copy, part of the slot, portion): a fill marks portions "in, chunk", the in-switch sum of an all-reduce
requires "in" in its portion of EVERY copy and marks it "sum" everywhere, a copy-out or a load-reduce requires what it
reads to be there and marks it "done".  Writing over anything that is not "done" is a violation, so a part that is
refilled too early (by the same or by another collective) shows up, and a lost wake-up shows up as a deadlock.  The
release ordering of the real kernel (data before the arrival) is what makes it legal to apply a phase's writes at once,
before its arrival is issued.  The reference has no counterpart."""
import sys
from pathlib import Path

import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

FILLED, REDUCED, CONSUMED = 0, 1, 2
MAX_DEPTH = 4
N_COUNTERS = MAX_DEPTH * 3          # counter index = part * 3 + kind


def ctr(part, kind):
    return part * 3 + kind


SUB = 2                 # groups the stage that talks to the switch is split into (3 in the kernel; 2 keeps the state space small)


def programs(coll, n, r, m, used, call, root=0, depth=2, broken=None):
    """The phases of the warp groups (fill, switch, out; the stage that issues the multimem instructions split into SUB groups
    that take the chunks in turn) of rank r for one call of `coll` with m chunks, exactly in the order of nvls_coll_kernel.
    used = fills so far of part 0..3, then reductions so far of part 0..3; returns (list of op lists, one per group, used')."""
    bu, by = used[:MAX_DEPTH], used[MAX_DEPTH:]
    split = {"allreduce": "switch", "allgather": "fill", "broadcast": "fill", "reduce_scatter": "out", "reduce": "out"}[coll]
    groups = {"fill": [[] for _ in range(SUB if split == "fill" else 1)], "switch": [[] for _ in range(SUB if split == "switch" else 1)],
              "out": [[] for _ in range(SUB if split == "out" else 1)]}
    g = lambda j: (call, j)
    allreduce = coll == "allreduce"
    filler = (r == root) if coll == "broadcast" else True
    consumer = (r == root) if coll == "reduce" else True
    fill_inc = n if coll == "broadcast" else 1
    cons_inc = n if coll == "reduce" else 1
    for j in range(m):
        p, u, uy = j % depth, bu[j % depth] + j // depth, by[j % depth] + j // depth
        fill, switch, out = (groups[k][j % len(groups[k])] for k in ("fill", "switch", "out"))
        if filler:
            if n * u and broken != "no_wait_consumed":
                fill.append(("wait", ctr(p, CONSUMED), n * u))
            if coll == "allgather":
                fill.append(("fill_all", g(j), p, (r,)))
            elif coll == "broadcast":
                fill.append(("fill_all", g(j), p, tuple(range(n))))
            else:
                fill.append(("fill_own", g(j), p))
            fill.append(("arrive", ctr(p, FILLED), fill_inc))
        if allreduce:
            if broken != "no_wait_filled":
                switch.append(("wait", ctr(p, FILLED), n * (u + 1)))
            switch.append(("reduce_all", g(j), p, r))
            switch.append(("arrive", ctr(p, REDUCED), 1))
        if consumer:
            if allreduce:
                if broken != "no_wait_reduced":
                    out.append(("wait", ctr(p, REDUCED), n * (uy + 1)))
                out.append(("copy_out", g(j), p, "sum"))
            else:
                if broken != "no_wait_filled":
                    out.append(("wait", ctr(p, FILLED), n * (u + 1)))
                if coll in ("allgather", "broadcast"):
                    out.append(("copy_out", g(j), p, "in"))
                elif coll == "reduce_scatter":
                    out.append(("reduce_local", g(j), p, (r,)))
                else:
                    out.append(("reduce_local", g(j), p, tuple(range(n))))
            out.append(("arrive", ctr(p, CONSUMED), cons_inc))
    cnt = [(m + depth - 1 - p) // depth if p < depth else 0 for p in range(MAX_DEPTH)]
    new = [bu[p] + cnt[p] for p in range(MAX_DEPTH)] + [by[p] + (cnt[p] if allreduce else 0) for p in range(MAX_DEPTH)]
    return groups["fill"] + groups["switch"] + groups["out"], new


def sequence(n, calls, depth=2, broken=None):
    """calls: list of (collective, chunks, root).  Returns the programs of the whole sequence, one per (rank, warp group):
    kernels of one rank run one after the other, so a group's ops of call k+1 follow ALL groups' ops of call k; that is
    modelled with a local barrier between calls."""
    G = 2 + SUB                                   # groups per rank
    procs = [[] for _ in range(G * n)]
    used = [0] * (2 * MAX_DEPTH)
    for ci, (coll, m, root) in enumerate(calls):
        nxt = None
        for r in range(n):
            roles, nxt = programs(coll, n, r, m, used, ci, root, depth, broken)
            for k in range(G):
                procs[G * r + k] += roles[k] + [("kernel_end", ci)]
        used = nxt
    return procs, used


def explore(n, procs, limit=6_000_000):
    """Returns the number of states visited; raises AssertionError naming the violation or the deadlock."""
    P = len(procs)
    # arrivals issued by process s on counter c, in program order, as (position in the program, increment)
    arrivals = [[[(i, op[2]) for i, op in enumerate(procs[s]) if op[0] == "arrive" and op[1] == c] for c in range(N_COUNTERS)] for s in range(P)]
    live = [(s, c) for s in range(P) for c in range(N_COUNTERS) if arrivals[s][c]]
    idx = {sc: k for k, sc in enumerate(live)}
    start = (tuple([0] * P), tuple([0] * (len(live) * n)), tuple([None] * (n * MAX_DEPTH * n)))
    seen = {start}
    stack = [start]
    free = lambda tag: tag is None or tag[0] == "done"
    at = lambda q, h, p: (q * MAX_DEPTH + h) * n + p
    while stack:
        pcs, deliv, tags = stack.pop()
        succ = []
        for (s_, c), k in idx.items():
            issued = sum(1 for pos, _ in arrivals[s_][c] if pos < pcs[s_])
            for dst in range(n):
                i = k * n + dst
                if deliv[i] < issued:
                    d = list(deliv); d[i] += 1
                    succ.append((pcs, tuple(d), tags))
        for pr in range(P):
            if pcs[pr] >= len(procs[pr]):
                continue
            G = P // n
            r = pr // G
            op = procs[pr][pcs[pr]]
            t = list(tags)
            if op[0] == "wait":
                have = sum(sum(inc for _, inc in arrivals[s_][c][:deliv[k * n + r]]) for (s_, c), k in idx.items() if c == op[1])
                if have < op[2]:
                    continue
            elif op[0] == "kernel_end":
                # the next kernel of this rank starts when every group of this one is done
                if any(not (pcs[G * r + k] < len(procs[G * r + k]) and procs[G * r + k][pcs[G * r + k]] == op) and
                       not any(o == op for o in procs[G * r + k][:pcs[G * r + k]]) for k in range(G)):
                    continue
            elif op[0] == "fill_own":
                _, g, h = op
                for p in range(n):
                    assert free(t[at(r, h, p)]), f"rank {r} fills part {h} with {g} over {t[at(r, h, p)]}"
                    t[at(r, h, p)] = ("in", g)
            elif op[0] == "fill_all":
                _, g, h, portions = op
                for q in range(n):
                    for p in portions:
                        assert free(t[at(q, h, p)]), f"rank {r} stores {g} into portion {p} of rank {q}'s part {h} over {t[at(q, h, p)]}"
                        t[at(q, h, p)] = ("in", g)
            elif op[0] == "reduce_all":
                _, g, h, p = op
                for q in range(n):
                    assert t[at(q, h, p)] == ("in", g), f"rank {r} sums {g} but rank {q}'s part {h} holds {t[at(q, h, p)]}"
                for q in range(n):
                    t[at(q, h, p)] = ("sum", g)
            elif op[0] == "copy_out":
                _, g, h, want = op
                for p in range(n):
                    assert t[at(r, h, p)] == (want, g), f"rank {r} copies {g} out of part {h} but portion {p} holds {t[at(r, h, p)]}"
                    t[at(r, h, p)] = ("done", g)
            elif op[0] == "reduce_local":
                _, g, h, portions = op
                for q in range(n):
                    for p in portions:
                        assert t[at(q, h, p)] == ("in", g), f"rank {r} load-reduces {g} but portion {p} of rank {q}'s part {h} holds {t[at(q, h, p)]}"
                for q in range(n):
                    for p in portions:
                        t[at(q, h, p)] = ("done", g)
            p2 = list(pcs); p2[pr] += 1
            succ.append((tuple(p2), deliv, tuple(t)))
        if not succ:
            assert all(pcs[k] == len(procs[k]) for k in range(P)), f"deadlock at {pcs}: {[procs[k][pcs[k]] for k in range(P) if pcs[k] < len(procs[k])]}"
        for st in succ:
            if st not in seen:
                seen.add(st)
                stack.append(st)
                assert len(seen) < limit, "state space larger than expected"
    return len(seen)


@pytest.mark.parametrize("calls,depth", [
    ([("allreduce", 3, 0)], 2),
    ([("allreduce", 2, 0), ("allreduce", 1, 0)], 2),
    ([("allreduce", 1, 0), ("allgather", 2, 0)], 2),
    ([("allgather", 3, 0)], 2),
    ([("allgather", 1, 0), ("allreduce", 1, 0)], 2),
    ([("reduce_scatter", 3, 0)], 2),
    ([("reduce_scatter", 1, 0), ("allreduce", 1, 0)], 2),
    ([("broadcast", 3, 1)], 2),
    ([("broadcast", 1, 1), ("reduce", 2, 0)], 2),
    ([("reduce", 3, 1)], 2),
    ([("reduce", 4, 1)], 3),
])
def test_every_interleaving_of_two_ranks_is_safe_and_terminates(calls, depth):
    procs, _ = sequence(2, calls, depth)
    assert explore(2, procs) > 20


def test_counts_of_uses_stay_in_step_for_any_number_of_chunks():
    # 3 chunks on a slot of 2 parts, then 2 chunks: part 0 was used twice, part 1 once, before the second call
    procs, used = sequence(2, [("allreduce", 3, 0), ("allgather", 2, 0)], depth=2)
    assert used == [3, 2, 0, 0, 2, 1, 0, 0]
    _, used = sequence(2, [("allreduce", 5, 0)], depth=4)
    assert used == [2, 1, 1, 1, 2, 1, 1, 1]


@pytest.mark.parametrize("calls,broken", [
    ([("allreduce", 3, 0)], "no_wait_filled"),
    ([("allreduce", 3, 0)], "no_wait_reduced"),
    ([("allreduce", 3, 0)], "no_wait_consumed"),          # the third chunk is staged over the first before it was copied out
    ([("allgather", 3, 0)], "no_wait_consumed"),          # ... or stored over it in a peer's copy
    ([("allreduce", 1, 0), ("allgather", 1, 0)], "no_wait_consumed"),   # another collective takes the part over too early
    ([("reduce_scatter", 3, 0)], "no_wait_consumed"),     # the own copy is refilled while a peer still load-reduces from it
    ([("broadcast", 2, 0)], "no_wait_filled"),
])
def test_the_checker_finds_a_missing_wait(calls, broken):
    procs, _ = sequence(2, calls, depth=2, broken=broken)
    with pytest.raises(AssertionError):
        explore(2, procs)
