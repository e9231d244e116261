#!/usr/bin/env python
"""Summary of the per-rank traces the library writes with PICCL_TRACE=<prefix> (Chrome-trace JSON, one file
`<prefix>.<rank>.json` per rank, one complete event per collective call: name `<collective>/<ALGO>`, device duration in µs,
args bytes / k / ctas; written by src/runtime/trace.cu when a communicator is destroyed).

    python tools/trace/summarize.py /tmp/run.0.json /tmp/run.1.json ...     # or a prefix: /tmp/run

Prints, per (collective, algorithm, size bucket): calls, total and mean device time, and the bandwidth the mean corresponds
to (bytes / time, the `algbw` of the benchmark tables); and per rank the share of traced time.  The files also load in
chrome://tracing or Perfetto as they are.  The reference has an NVTX range around one collective and nothing else
(src/piccl.c:32,55,60)."""
from __future__ import annotations

import glob
import json
import sys
from collections import defaultdict


def bucket(nbytes: int) -> str:
    """power-of-four size classes: <=1K, <=4K, ... <=1G, >1G"""
    b, names = 1024, ["1K", "4K", "16K", "64K", "256K", "1M", "4M", "16M", "64M", "256M", "1G"]
    for n in names:
        if nbytes <= b:
            return "<=" + n
        b *= 4
    return ">1G"


def load(paths):
    files = []
    for p in paths:
        files += sorted(glob.glob(p + ".*.json")) if not p.endswith(".json") else [p]
    events = []
    for f in files:
        with open(f) as fh:
            for e in json.load(fh).get("traceEvents", []):
                if e.get("ph") == "X":
                    events.append(e)
    return files, events


def summarize(events):
    groups = defaultdict(lambda: [0, 0.0, 0])          # calls, µs, bytes
    per_rank = defaultdict(float)
    for e in events:
        coll, _, algo = e["name"].partition("/")
        nbytes = int(e.get("args", {}).get("bytes", 0))
        g = groups[(coll, algo, bucket(nbytes))]
        g[0] += 1
        g[1] += float(e["dur"])
        g[2] += nbytes
        per_rank[int(e.get("pid", 0))] += float(e["dur"])
    rows = []
    for (coll, algo, b), (calls, us, nbytes) in sorted(groups.items(), key=lambda kv: -kv[1][1]):
        rows.append({"collective": coll, "algorithm": algo, "size": b, "calls": calls, "total_ms": us / 1e3, "mean_us": us / calls,
                     "algbw_GBs": (nbytes / calls) / (us / calls) / 1e3 if us > 0 else 0.0})
    return rows, dict(per_rank)


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if not argv:
        print(__doc__)
        return 2
    files, events = load(argv)
    if not events:
        print("no events found in", files or argv)
        return 1
    rows, per_rank = summarize(events)
    print(f"{len(events)} calls in {len(files)} file(s)")
    print(f"{'collective':15s} {'algorithm':8s} {'size':>6s} {'calls':>7s} {'total ms':>10s} {'mean us':>10s} {'GB/s':>8s}")
    for r in rows:
        print(f"{r['collective']:15s} {r['algorithm']:8s} {r['size']:>6s} {r['calls']:7d} {r['total_ms']:10.3f} {r['mean_us']:10.2f} {r['algbw_GBs']:8.1f}")
    total = sum(per_rank.values()) or 1.0
    print("device time per rank: " + ", ".join(f"rank {r}: {us / 1e3:.2f} ms ({100 * us / total:.0f} %)" for r, us in sorted(per_rank.items())))
    return 0


if __name__ == "__main__":
    sys.exit(main())
