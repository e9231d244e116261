"""Exhaustive interleaving check of the counter / half-slot protocol of the in-switch collectives
(src/kernels/nvls_coll.cu, described in src/kernels/nvls.cuh), on a small model: a few ranks, one CTA index, a few chunks,
several calls of different collectives in a row.

Each rank runs the kernel's sequence of phases; the explorer tries every order in which ranks can advance and in which
counter arrivals can reach each rank (an arrival is delivered to every rank separately, in any order).  Data is modelled
as tags per (rank's copy, half slot, portion): a fill marks portions "in, chunk", the in-switch sum of an all-reduce
requires "in" in its portion of EVERY copy and marks it "sum" everywhere, a copy-out or a load-reduce requires what it
reads to be there and marks it "done".  Writing over anything that is not "done" is a violation, so a half slot that is
refilled too early (by the same or by another collective) shows up, and a lost wake-up shows up as a deadlock.  The
release ordering of the real kernel (data before the arrival) is what makes it legal to apply a phase's writes at once,
before its arrival is issued.  The reference has no counterpart."""
import sys
from pathlib import Path

import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

FILLED, REDUCED, CONSUMED = 0, 1, 2
N_COUNTERS = 6          # counter index = half * 3 + kind


def ctr(half, kind):
    return half * 3 + kind


def program(coll, n, r, m, used, call, root=0, broken=None):
    """The phases of rank r for one call of `coll` with m chunks, exactly in the order of nvls_coll_kernel.
    used = [fills of half 0, fills of half 1, reductions of half 0, reductions of half 1] so far; returns (ops, used')."""
    bu, by = used[:2], used[2:]
    ops = []
    g = lambda j: (call, j)

    def wait_consumed(j):
        s = j & 1
        target = n * (bu[s] + (j >> 1))
        if target and broken != "no_wait_consumed":
            ops.append(("wait", ctr(s, CONSUMED), target))

    if coll == "allreduce":
        def fill(j):
            wait_consumed(j)
            ops.append(("fill_own", g(j), j & 1))
            ops.append(("arrive", ctr(j & 1, FILLED), 1))
        if m > 0:
            fill(0)
        for j in range(m):
            s = j & 1
            if broken != "no_wait_filled":
                ops.append(("wait", ctr(s, FILLED), n * (bu[s] + (j >> 1) + 1)))
            ops.append(("reduce_all", g(j), s, r))
            ops.append(("arrive", ctr(s, REDUCED), 1))
            if j + 1 < m:
                fill(j + 1)
            if broken != "no_wait_reduced":
                ops.append(("wait", ctr(s, REDUCED), n * (by[s] + (j >> 1) + 1)))
            ops.append(("copy_out", g(j), s, "sum"))
            ops.append(("arrive", ctr(s, CONSUMED), 1))
        new = [bu[0] + (m + 1) // 2, bu[1] + m // 2, by[0] + (m + 1) // 2, by[1] + m // 2]
        return ops, new
    filler = (r == root) if coll == "broadcast" else True
    consumer = (r == root) if coll == "reduce" else True
    fill_inc = n if coll == "broadcast" else 1
    cons_inc = n if coll == "reduce" else 1

    def fill(j):
        wait_consumed(j)
        s = j & 1
        if coll == "allgather":
            ops.append(("fill_all", g(j), s, (r,)))
        elif coll == "broadcast":
            ops.append(("fill_all", g(j), s, tuple(range(n))))
        else:
            ops.append(("fill_own", g(j), s))
        ops.append(("arrive", ctr(s, FILLED), fill_inc))

    if m > 0 and filler:
        fill(0)
    for j in range(m):
        s = j & 1
        if filler and j + 1 < m:
            fill(j + 1)
        if consumer:
            if broken != "no_wait_filled":
                ops.append(("wait", ctr(s, FILLED), n * (bu[s] + (j >> 1) + 1)))
            if coll in ("allgather", "broadcast"):
                ops.append(("copy_out", g(j), s, "in"))
            elif coll == "reduce_scatter":
                ops.append(("reduce_local", g(j), s, (r,)))
            else:
                ops.append(("reduce_local", g(j), s, tuple(range(n))))
            ops.append(("arrive", ctr(s, CONSUMED), cons_inc))
    return ops, [bu[0] + (m + 1) // 2, bu[1] + m // 2, by[0], by[1]]


def sequence(n, calls, broken=None):
    """calls: list of (collective, chunks, root).  Returns the per-rank programs of the whole sequence."""
    progs = [[] for _ in range(n)]
    used = [0, 0, 0, 0]
    for ci, (coll, m, root) in enumerate(calls):
        nxt = None
        for r in range(n):
            ops, nxt = program(coll, n, r, m, used, ci, root, broken)
            progs[r] += ops
        used = nxt
    return progs, used


def explore(n, programs, limit=4_000_000):
    """Returns the number of states visited; raises AssertionError naming the violation or the deadlock."""
    # arrivals issued by src on counter c, in program order, as (position in the program, increment)
    arrivals = [[[(i, op[2]) for i, op in enumerate(programs[src]) if op[0] == "arrive" and op[1] == c] for c in range(N_COUNTERS)] for src in range(n)]
    start = (tuple([0] * n), tuple([0] * (n * N_COUNTERS * n)), tuple([None] * (n * 2 * n)))
    seen = {start}
    stack = [start]
    free = lambda tag: tag is None or tag[0] == "done"
    while stack:
        pcs, deliv, tags = stack.pop()
        succ = []
        for src in range(n):
            for c in range(N_COUNTERS):
                issued = sum(1 for pos, _ in arrivals[src][c] if pos < pcs[src])
                for dst in range(n):
                    i = (src * N_COUNTERS + c) * n + dst
                    if deliv[i] < issued:
                        d = list(deliv); d[i] += 1
                        succ.append((pcs, tuple(d), tags))
        for r in range(n):
            if pcs[r] >= len(programs[r]):
                continue
            op = programs[r][pcs[r]]
            t = list(tags)
            at = lambda q, h, p: (q * 2 + h) * n + p
            if op[0] == "wait":
                have = sum(sum(inc for _, inc in arrivals[src][op[1]][:deliv[(src * N_COUNTERS + op[1]) * n + r]]) for src in range(n))
                if have < op[2]:
                    continue
            elif op[0] == "fill_own":
                _, g, h = op
                for p in range(n):
                    assert free(t[at(r, h, p)]), f"rank {r} fills half {h} with {g} over {t[at(r, h, p)]}"
                    t[at(r, h, p)] = ("in", g)
            elif op[0] == "fill_all":
                _, g, h, portions = op
                for q in range(n):
                    for p in portions:
                        assert free(t[at(q, h, p)]), f"rank {r} stores {g} into portion {p} of rank {q}'s half {h} over {t[at(q, h, p)]}"
                        t[at(q, h, p)] = ("in", g)
            elif op[0] == "reduce_all":
                _, g, h, p = op
                for q in range(n):
                    assert t[at(q, h, p)] == ("in", g), f"rank {r} sums {g} but rank {q}'s half {h} holds {t[at(q, h, p)]}"
                for q in range(n):
                    t[at(q, h, p)] = ("sum", g)
            elif op[0] == "copy_out":
                _, g, h, want = op
                for p in range(n):
                    assert t[at(r, h, p)] == (want, g), f"rank {r} copies {g} out of half {h} but portion {p} holds {t[at(r, h, p)]}"
                    t[at(r, h, p)] = ("done", g)
            elif op[0] == "reduce_local":
                _, g, h, portions = op
                for q in range(n):
                    for p in portions:
                        assert t[at(q, h, p)] == ("in", g), f"rank {r} load-reduces {g} but portion {p} of rank {q}'s half {h} holds {t[at(q, h, p)]}"
                for q in range(n):
                    for p in portions:
                        t[at(q, h, p)] = ("done", g)
            p2 = list(pcs); p2[r] += 1
            succ.append((tuple(p2), deliv, tuple(t)))
        if not succ:
            assert all(pcs[r] == len(programs[r]) for r in range(n)), f"deadlock at {pcs}: {[programs[r][pcs[r]] for r in range(n) if pcs[r] < len(programs[r])]}"
        for s in succ:
            if s not in seen:
                seen.add(s)
                stack.append(s)
                assert len(seen) < limit, "state space larger than expected"
    return len(seen)


@pytest.mark.parametrize("calls", [
    [("allreduce", 3, 0), ("allreduce", 2, 0)],
    [("allreduce", 2, 0), ("allgather", 3, 0)],
    [("allgather", 3, 0), ("allreduce", 2, 0)],
    [("reduce_scatter", 3, 0), ("allreduce", 2, 0)],
    [("broadcast", 3, 1), ("reduce", 3, 0)],
    [("reduce", 2, 1), ("allgather", 2, 0), ("broadcast", 2, 0)],
    [("allreduce", 1, 0), ("reduce_scatter", 2, 0), ("allgather", 1, 0)],
])
def test_every_interleaving_of_two_ranks_is_safe_and_terminates(calls):
    progs, _ = sequence(2, calls)
    assert explore(2, progs) > 50


@pytest.mark.parametrize("calls", [[("allreduce", 1, 0)], [("allgather", 1, 0)], [("reduce_scatter", 1, 0)], [("broadcast", 1, 2)], [("reduce", 1, 1)], [("broadcast", 1, 0), ("reduce", 1, 2)]])
def test_three_ranks(calls):
    progs, _ = sequence(3, calls)
    explore(3, progs)


def test_odd_and_even_chunk_counts_keep_the_half_slot_counters_in_step():
    # 3 chunks then 2 chunks: half slot 0 was used twice, half slot 1 once, before the second call
    progs, used = sequence(2, [("allreduce", 3, 0), ("allgather", 2, 0)])
    assert used == [3, 2, 2, 1]
    explore(2, progs)


@pytest.mark.parametrize("calls,broken", [
    ([("allreduce", 3, 0)], "no_wait_filled"),
    ([("allreduce", 3, 0)], "no_wait_reduced"),
    ([("allgather", 3, 0)], "no_wait_consumed"),          # the third chunk is stored over the first before it was copied out
    ([("allreduce", 1, 0), ("allgather", 1, 0)], "no_wait_consumed"),   # another collective takes the half slot over too early
    ([("reduce_scatter", 3, 0)], "no_wait_consumed"),     # the own copy is refilled while a peer still load-reduces from it
    ([("broadcast", 2, 0)], "no_wait_filled"),
])
def test_the_checker_finds_a_missing_wait(calls, broken):
    progs, _ = sequence(2, calls, broken=broken)
    with pytest.raises(AssertionError):
        explore(2, progs)
