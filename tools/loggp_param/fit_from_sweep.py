#!/usr/bin/env python
"""LogGP profile from a measured ring all-reduce sweep (coll_bench CSV) instead of PRTT data.

A ring all-reduce of S bytes on n ranks is a chain of 2(n-1) dependent messages of S/n bytes, so
    c(m) = (T_ring(n*m) - launch) / (2(n-1))
is the cost of ONE message of m bytes as the library's executor really moves it (low-latency lines for small
messages, FIFO slots with flags above that, many CTAs for large ones).  The profile written here encodes that curve:
o_s = o_r = g = 0, G = the asymptotic time per byte, L(s) = c(s) - G (s - 1), one row per measured size.  The simulator then
reproduces the ring by construction and predicts the other schedules from it.  PRTT-based profiles (get_loggp_param.py, the
method of the reference's tools/loggp_param/get_loggp_param.py) describe a bare flag-and-fence message instead and over-predict
the per-step cost of the executor's low-latency path several times.

    python tools/loggp_param/fit_from_sweep.py benchmarks/results/sweep_8.csv --ranks 8 --output profile.csv
"""
from __future__ import annotations

import argparse
import csv
import sys


def message_costs(path: str, ranks: int, label: str = "ours-RING-k-1", dtype: str = "float", launch_us: float = 2.5):
    """[(message bytes, seconds)] sorted by size, from the rows `allreduce,<label>,<dtype>,sum,<ranks>,...`."""
    pts = {}
    with open(path) as f:
        for r in csv.reader(f):
            if len(r) < 8 or r[0] != "allreduce" or r[1] != label or r[2] != dtype or int(r[4]) != ranks:
                continue
            size, t_us = int(r[5]), float(r[7])
            if size < 16 * ranks:          # fewer than one 16-byte pack per rank: some hops carry nothing
                continue
            pts[size // ranks] = max(t_us - launch_us, 0.1) * 1e-6 / (2 * (ranks - 1))
    return sorted(pts.items())


def profile_rows(costs):
    """s, L, o_s, o_r, g, G rows: constant G from the two largest sizes, L(s) = c(s) - G (s - 1), never negative."""
    if len(costs) < 2:
        raise ValueError("need at least two message sizes")
    (m1, c1), (m2, c2) = costs[-2], costs[-1]
    G = max((c2 - c1) / (m2 - m1), 1e-15)
    rows = []
    for m, c in costs:
        rows.append((m, max(c - G * (m - 1), 0.0), 0.0, 0.0, 0.0, G))
    return rows


def write_profile(rows, out: str) -> None:
    with open(out, "w") as f:
        f.write("s,L,o_s,o_r,g,G\n")
        for r in rows:
            f.write(",".join([str(r[0])] + ["%.15e" % x for x in r[1:]]) + "\n")


def fit_gamma(path: str, profile: str, ranks: int, dtype: str = "float", launch_us: float = 2.5, min_bytes: int = 4 << 20):
    """Cost per received byte that best explains the measured recursive all-reduces (PRD / PRM rows of the sweep), given the
    profile fitted from the ring: those schedules send in one pass and receive-and-reduce in another, a ring hop does both
    at once (and that is inside the fitted message cost), so the term applies to them only (tools/selector/select.py: predict).
    Grid search on the squared log ratio; returns (gamma, median |log ratio|)."""
    import math
    import re
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
    from tools.selector import select as sel
    meas = []
    with open(path) as f:
        for r in csv.reader(f):
            m = re.match(r"ours-(PRD|PRM)-k(-?\d+)", r[1]) if len(r) > 8 and r[0] == "allreduce" and r[2] == dtype and int(r[4]) == ranks else None
            if m and int(r[5]) >= min_bytes:
                meas.append((m.group(1), int(m.group(2)), int(r[5]), float(r[7])))
    if not meas:
        raise ValueError("no PRD / PRM rows of that size in the sweep")
    base = [(1e6 * sel.predict(profile, "allreduce", ranks, b, a, k, radix=1, gamma=0.0), 1e6 * sel.predict(profile, "allreduce", ranks, b, a, k, radix=1, gamma=1e-12))
            for a, k, b, _ in meas]        # the prediction is linear in gamma: two points give the line
    best = None
    for i in range(0, 201):
        g = i * 1e-14
        errs = [abs(math.log((launch_us + p0 + (p1 - p0) * g / 1e-12) / t)) for (p0, p1), (_, _, _, t) in zip(base, meas)]
        score = sum(e * e for e in errs)
        if best is None or score < best[0]:
            best = (score, g, sorted(errs)[len(errs) // 2])
    return best[1], best[2]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="LogGP profile from a measured ring all-reduce sweep")
    ap.add_argument("sweep", help="coll_bench CSV")
    ap.add_argument("--ranks", type=int, required=True)
    ap.add_argument("--label", default="ours-RING-k-1")
    ap.add_argument("--dtype", default="float")
    ap.add_argument("--launch-us", type=float, default=2.5, help="time of an empty launch, subtracted before dividing by the hop count")
    ap.add_argument("--output", required=True)
    ap.add_argument("--fit-gamma", action="store_true", help="also fit the reduction cost per received byte (for --gamma of the simulator and the selector)")
    a = ap.parse_args(argv)
    rows = profile_rows(message_costs(a.sweep, a.ranks, a.label, a.dtype, a.launch_us))
    write_profile(rows, a.output)
    print(f"{len(rows)} sizes, G = {rows[0][5]:.3e} s/B ({1e-9 / rows[0][5]:.0f} GB/s) -> {a.output}")
    if a.fit_gamma:
        g, med = fit_gamma(a.sweep, a.output, a.ranks, a.dtype, a.launch_us)
        print(f"gamma = {g:.2e} s/B (median |log ratio| of the recursive all-reduces from 4 MiB: {med:.3f})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
