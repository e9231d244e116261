"""Exhaustive interleaving check of the barrier / slot protocol of the in-switch all-reduce kernels
(src/kernels/nvls_allreduce.cu), on a small model: a few ranks, one CTA index, a few chunks, two calls in a row.

Each rank runs the kernel's sequence of phases; the explorer tries every order in which ranks can advance and in which
counter arrivals can reach each rank (an arrival is delivered to every rank separately, in any order).  Data is modelled
as tags: a copy-in marks the rank's slot "in, chunk j", the in-switch phase of rank x requires "in, j" in portion x of
EVERY rank's slot and marks it "sum, j" everywhere, a copy-out requires "sum, j" in all portions of the own slot.  A stale
or overwritten slot therefore shows up as a violation, a lost wake-up as a deadlock.  The release ordering of the real
kernel (data before the arrival) is what makes it legal to apply a phase's writes at once, before its arrival is issued.
The reference has no counterpart."""
import sys
from pathlib import Path

import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

# counters: 0 = plain kernel; 1, 2 = A of half slot 0 / 1; 3, 4 = B of half slot 0 / 1
N_COUNTERS = 5


def plain_program(n, m, base, call):
    """nvls_allreduce_kernel: one slot, one counter, two barriers per chunk."""
    ops, nbar = [], base
    for j in range(m):
        g = (call, j)
        ops.append(("ci", g, (0, 1)))
        nbar += 1
        ops += [("arrive", 0), ("wait", 0, nbar * n)]
        ops.append(("r", g, (0, 1)))
        nbar += 1
        ops += [("arrive", 0), ("wait", 0, nbar * n)]
        ops.append(("co", g, (0, 1)))
    return ops, nbar


def pipe_program(n, m, base, call, broken=None):
    """nvls_allreduce_pipe_kernel: two half slots, counters A0 A1 B0 B1.  `base` = uses of each half slot so far.
    The window slot of a CTA index is modelled as two halves; the plain kernel uses both for every chunk."""
    ops = []
    if m > 0:
        ops += [("ci", (call, 0), (0,)), ("arrive", 1)]
    for j in range(m):
        s = j & 1
        target = n * (base[s] + (j >> 1) + 1)
        g = (call, j)
        if broken != "no_wait_a":
            ops.append(("wait", 1 + s, target))
        ops += [("r", g, (s,)), ("arrive", 3 + s)]
        nxt = [("ci", (call, j + 1), (s ^ 1,)), ("arrive", 1 + (s ^ 1))] if j + 1 < m else []
        tail = [("wait", 3 + s, target), ("co", g, (s,))]
        if broken == "copy_in_after_copy_out_only":          # would be correct but serial: used as a sanity variant
            ops += tail + nxt
        elif broken == "no_wait_b":
            ops += nxt + [("co", g, (s,))]
        else:
            ops += nxt + tail
    used = [base[0] + (m + 1) // 2, base[1] + m // 2]
    return ops, used


def explore(n, programs, limit=3_000_000):
    """programs[r]: list of ops.  Returns the number of states visited; raises AssertionError naming the violation or the deadlock."""
    # state: pcs, delivered[src][c][dst], tags[rank][half][portion]
    start = (tuple([0] * n), tuple([0] * (n * N_COUNTERS * n)), tuple([None] * (n * 2 * n)))
    seen = {start}
    stack = [start]

    def issued(pcs, src, c):
        return sum(1 for op in programs[src][:pcs[src]] if op[0] == "arrive" and op[1] == c)

    while stack:
        pcs, deliv, tags = stack.pop()
        moved = False
        succ = []
        # deliveries
        for src in range(n):
            for c in range(N_COUNTERS):
                iss = issued(pcs, src, c)
                for dst in range(n):
                    i = (src * N_COUNTERS + c) * n + dst
                    if deliv[i] < iss:
                        d = list(deliv); d[i] += 1
                        succ.append((pcs, tuple(d), tags))
        # rank steps
        for r in range(n):
            if pcs[r] >= len(programs[r]):
                continue
            op = programs[r][pcs[r]]
            t = list(tags)
            if op[0] == "wait":
                have = sum(deliv[(src * N_COUNTERS + op[1]) * n + r] for src in range(n))
                if have < op[2]:
                    continue
            elif op[0] == "ci":
                _, g, halves = op
                for h in halves:
                    for p in range(n):
                        old = t[(r * 2 + h) * n + p]
                        # overwriting data that somebody still needs: contributions not yet summed, sums not yet copied out
                        assert old is None or old[0] == "done", f"rank {r} copies chunk {g} into half {h} over {old}"
                        t[(r * 2 + h) * n + p] = ("in", g)
            elif op[0] == "r":
                _, g, halves = op
                for h in halves:
                    for q in range(n):
                        old = t[(q * 2 + h) * n + r]
                        assert old == ("in", g), f"rank {r} sums chunk {g} but rank {q}'s half {h} holds {old}"
                    for q in range(n):
                        t[(q * 2 + h) * n + r] = ("sum", g)
            elif op[0] == "co":
                _, g, halves = op
                for h in halves:
                    for p in range(n):
                        old = t[(r * 2 + h) * n + p]
                        assert old == ("sum", g), f"rank {r} copies chunk {g} out of half {h} but portion {p} holds {old}"
                        t[(r * 2 + h) * n + p] = ("done", g)
            p2 = list(pcs); p2[r] += 1
            succ.append((tuple(p2), deliv, tuple(t)))
        for s in succ:
            moved = True
            if s not in seen:
                seen.add(s)
                stack.append(s)
                assert len(seen) < limit, "state space larger than expected"
        if not moved:
            assert all(pcs[r] == len(programs[r]) for r in range(n)), f"deadlock at {pcs}: {[programs[r][pcs[r]] for r in range(n) if pcs[r] < len(programs[r])]}"
    return len(seen)


def two_calls(n, kinds, m):
    """Every rank runs two kernels in a row (kinds: 'plain' / 'pipe'), m chunks each."""
    ops, nbar, used = [], 0, [0, 0]
    for call, kind in enumerate(kinds):
        if kind == "plain":
            o, nbar = plain_program(n, m, nbar, call)
        else:
            o, used = pipe_program(n, m, used, call)
        ops += o
    return [list(ops) for _ in range(n)]


@pytest.mark.parametrize("kinds,n,m", [(("plain", "plain"), 2, 2), (("pipe", "pipe"), 2, 3), (("pipe", "plain"), 2, 2), (("plain", "pipe"), 2, 3),
                                       (("pipe",), 3, 2), (("plain",), 3, 2)])
def test_every_interleaving_is_safe_and_terminates(kinds, n, m):
    states = explore(n, two_calls(n, kinds, m))
    assert states > 100


def test_odd_and_even_chunk_counts_keep_the_half_slot_counters_in_step():
    # 3 chunks then 2 chunks: half slot 0 was used twice, half slot 1 once, before the second call
    n = 2
    o1, used = pipe_program(n, 3, [0, 0], 0)
    o2, used2 = pipe_program(n, 2, used, 1)
    assert used == [2, 1] and used2 == [3, 2]
    explore(n, [o1 + o2 for _ in range(n)])


@pytest.mark.parametrize("broken", ["no_wait_b", "no_wait_a"])
def test_the_checker_finds_a_missing_wait(broken):
    n, m = 2, 3
    prog, _ = pipe_program(n, m, [0, 0], 0, broken=broken)
    with pytest.raises(AssertionError):
        explore(n, [list(prog) for _ in range(n)])


def test_serial_order_is_also_safe():
    n, m = 2, 3
    prog, _ = pipe_program(n, m, [0, 0], 0, broken="copy_in_after_copy_out_only")
    explore(n, [list(prog) for _ in range(n)])
