#!/usr/bin/env python
"""Algorithm / radix selector: writes the tuning table PICCL_TUNE_FILE points to
(CSV rows `collective,nranks,max_bytes,algorithm,k`; for a message of b bytes the first row of its
collective and rank count with max_bytes >= b wins; see src/runtime/selector.cc).

Two sources:
  --profile P.csv     predict every candidate with the LogGP simulator (tools/loggp_sim) on a flat
                      topology whose links use the fitted profile P (from tools/loggp_param)
  --from-bench F.csv  take the fastest measured candidate per size from coll_bench output
                      (label column `ours-<ALGO>-k<K>`; --alias LABEL=ALGO:K[:MAX_BYTES] names what a run with
                      another label measured, e.g. nvls=NVLS:-1, or ours-AUTO-k-1=PRM:8:65536 for the sizes at
                      which AUTO is known to have run that algorithm)
With --profile, --nvls-bench F.csv adds the in-switch path as a candidate.  It is not a schedule of point-to-point transfers, so
the LogGP simulator cannot replay it; its cost is fitted from measurements instead: T(bytes) = a + bytes / B per collective and rank
count (least squares over the rows of F whose label, after --alias, names NVLS), a = the fill / switch / out pipeline's start-up,
B = its steady-state rate.
The reference has no selector; its user sets PICCL_<COLL>_ALGO by hand (README.md:46-68).
"""
from __future__ import annotations

import argparse
import csv
import re
import sys
import tempfile
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from tools.loggp_sim import sim as S  # noqa: E402
from tools.schedule_generator import main as gen  # noqa: E402

COLLS = ["allgather", "allreduce", "broadcast", "reduce", "reduce_scatter"]


def candidates(n: int):
    out = [("RING", -1), ("PRD", -1)]
    if 2 < n <= 8:
        out.append(("DIRECT", -1))
    for k in (2, 4, 8):
        if 2 <= k <= n:
            out.append(("PRM", k))
            if n % k == 0 and k < n:
                out.append(("K_RING", k))
    return out


def predict(profile: str, coll: str, n: int, nbytes: int, algo: str, k: int, radix: int, gamma: float) -> float:
    with tempfile.TemporaryDirectory() as d:
        topo = Path(d) / "t.xml"
        topo.write_text(S.flat_topology_xml(n, profile))
        sched = Path(d) / "s.xml"
        total = nbytes * n if coll in ("allgather", "reduce_scatter") else nbytes
        sched.write_text(gen.generate("bcast" if coll == "broadcast" else coll, n, max(total, n), algo, max(k, 1)))
        # gamma: cost per received byte of the separate receive-and-reduce pass of the recursive and direct schedules; a ring hop
        # reduces while it forwards, and that is already part of a message cost fitted from a ring (fit_from_sweep.py)
        reducing = coll in ("allreduce", "reduce", "reduce_scatter") and algo not in ("RING", "K_RING")
        return S.simulate(sched, topo, radix=radix, gamma=gamma if reducing else 0.0)


def compress(rows):
    """(bytes, algo, k) per size -> ranges"""
    out = []
    for b, a, k in rows:
        if out and out[-1][1] == a and out[-1][2] == k:
            out[-1] = (b, a, k)
        else:
            out.append((b, a, k))
    if out:
        out[-1] = (1 << 62, out[-1][1], out[-1][2])
    return out


def fit_nvls(paths, aliases):
    """(collective, ranks) -> (a seconds, B bytes per second) of T = a + bytes / B, from coll_bench rows that measured NVLS."""
    import numpy as np
    pts: dict = {}
    for p in paths:
        with open(p) as f:
            for r in csv.reader(f):
                if len(r) < 9 or r[0].startswith("#") or (len(r) > 10 and r[10] == "FAIL"):
                    continue
                algo = aliases[r[1]][0] if r[1] in aliases else (re.match(r"ours-([A-Z_]+)-k", r[1]) or [None, None])[1]
                if algo == "NVLS":
                    pts.setdefault((r[0], int(r[4])), []).append((int(r[5]), float(r[7]) * 1e-6))
    out = {}
    for key, v in pts.items():
        if len(v) < 2:
            continue
        b, t = np.array(sorted(v)).T
        slope, a = np.polyfit(b, t, 1, w=1.0 / t)               # relative errors: the small sizes pin a, the large ones B
        if slope > 0:
            out[key] = (max(float(a), 0.0), 1.0 / float(slope))
    return out


def table_from_profile(profile: str, ranks, min_b: int, max_b: int, gamma: float, nvls=None):
    rows = []
    nvls = nvls or {}
    for coll in COLLS:
        for n in ranks:
            per = []
            b = min_b
            while b <= max_b:
                best = None
                if (coll, n) in nvls:
                    a_, B_ = nvls[(coll, n)]
                    best = (a_ + b / B_, "NVLS", -1)
                for algo, k in candidates(n):
                    # small messages: injections overlap (radix n); large: the egress link is shared (one port)
                    t = predict(profile, coll, n, b, algo, k, radix=n if b <= 16384 else 1, gamma=gamma)
                    if best is None or t < best[0]:
                        best = (t, algo, k)
                per.append((b, best[1], best[2]))
                b *= 4
            rows += [(coll, n, mb, a, k) for mb, a, k in compress(per)]
    return rows


def table_from_bench(paths, aliases=None):
    aliases = aliases or {}
    best: dict = {}
    for p in paths:
        with open(p) as f:
            for r in csv.reader(f):
                if len(r) < 9 or r[0].startswith("#") or (len(r) > 10 and r[10] == "FAIL"):
                    continue
                if r[1] in aliases:
                    algo, k, max_b = aliases[r[1]]
                    if max_b is not None and int(r[5]) > max_b:
                        continue
                else:
                    m = re.match(r"ours-([A-Z_]+)-k(-?\d+)", r[1])
                    if not m or m.group(1) == "AUTO":
                        continue
                    algo, k = m.group(1), int(m.group(2))
                key = (r[0], int(r[4]), int(r[5]))
                t = float(r[7])
                if key not in best or t < best[key][0]:
                    best[key] = (t, algo, k)
    rows = []
    for coll, n in sorted({(c, n) for c, n, _ in best}):
        per = [(b, best[(coll, n, b)][1], best[(coll, n, b)][2]) for b in sorted(b for c, m, b in best if c == coll and m == n)]
        rows += [(coll, n, mb, a, k) for mb, a, k in compress(per)]
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Build the algorithm selection table")
    ap.add_argument("--profile", help="fitted LogGP CSV (s,L,o_s,o_r,g,G)")
    ap.add_argument("--from-bench", nargs="*", help="coll_bench CSV files with ours-<ALGO>-k<K> labels")
    ap.add_argument("--alias", action="append", default=[], help="LABEL=ALGO:K[:MAX_BYTES]: rows with this label measured that algorithm (up to that size)")
    ap.add_argument("--ranks", default="2,4,8")
    ap.add_argument("--min", type=int, default=8)
    ap.add_argument("--max", type=int, default=1 << 30)
    ap.add_argument("--gamma", type=float, default=0.0, help="reduction cost per byte (s/B)")
    ap.add_argument("--nvls-bench", nargs="*", default=[], help="with --profile: coll_bench CSV files with rows that measured the in-switch path (label ours-NVLS-k-1 or an --alias)")
    ap.add_argument("--output", required=True)
    a = ap.parse_args(argv)
    aliases = {}
    for spec in a.alias:
        label, what = spec.split("=", 1)
        parts = what.split(":")
        aliases[label] = (parts[0], int(parts[1]) if len(parts) > 1 else -1, int(parts[2]) if len(parts) > 2 else None)
    if a.from_bench:
        rows = table_from_bench(a.from_bench, aliases)
    elif a.profile:
        nvls = fit_nvls(a.nvls_bench, aliases) if a.nvls_bench else None
        if nvls:
            for (coll, n), (a_, B_) in sorted(nvls.items()):
                print(f"in-switch {coll} on {n} ranks: T = {a_ * 1e6:.1f} us + bytes / {B_ / 1e9:.0f} GB/s")
        rows = table_from_profile(a.profile, [int(x) for x in a.ranks.split(",")], a.min, a.max, a.gamma, nvls)
    else:
        ap.error("give --profile or --from-bench")
    with open(a.output, "w") as f:
        f.write("# collective,nranks,max_bytes,algorithm,k\n")
        for r in rows:
            f.write(",".join(str(x) for x in r) + "\n")
    print(f"{len(rows)} rows written to {a.output}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
