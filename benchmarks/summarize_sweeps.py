"""Turns coll_bench sweep CSVs (benchmarks/run_sweeps.sh) into markdown tables:
per collective / dtype / rank count, latency at small sizes and bus bandwidth at large sizes for
stock NCCL, the reference build and every algorithm of this library.

    python benchmarks/summarize_sweeps.py results/sweep_8.csv [more.csv ...]
"""
from __future__ import annotations

import csv
import sys
from collections import defaultdict


def load(paths):
    rows = defaultdict(dict)      # (coll, dtype, ranks, bytes) -> label -> (us, busbw, check)
    for p in paths:
        with open(p) as f:
            for r in csv.reader(f):
                if len(r) < 11 or r[0].startswith("#"):
                    continue
                try:
                    rows[(r[0], r[2], int(r[4]), int(r[5]))][r[1]] = (float(r[7]), float(r[9]), r[10])
                except ValueError:
                    continue
    return rows


def fmt(v, check, bw):
    if v is None:
        return "–"
    s = f"{v[1]:.0f}" if bw else f"{v[0]:.1f}"
    return s + ("†" if v[2] == "FAIL" else "")


def main(paths):
    rows = load(paths)
    keys = sorted({(c, d, n) for c, d, n, _ in rows})
    for coll, dt, n in keys:
        sizes = sorted(b for c, d, m, b in rows if (c, d, m) == (coll, dt, n))
        labels = sorted({l for (c, d, m, b), v in rows.items() if (c, d, m) == (coll, dt, n) for l in v},
                        key=lambda l: (0 if l == "nccl" else 1 if l.startswith("ref") else 2, l))
        small = [b for b in sizes if b <= 65536]
        large = [b for b in sizes if b >= (1 << 20)]
        if len(small) > 6:
            small = small[::2][:6]
        if len(large) > 7:
            large = large[::2]
        print(f"\n#### {coll}, {dt}, {n} GPUs — latency µs (small) / busBW GB/s (large); † = failed the data check\n")
        print("| impl | " + " | ".join(f"{b} B" for b in small) + " | " + " | ".join((f"{b >> 30} GiB" if b >= (1 << 30) else f"{b >> 20} MiB") for b in large) + " |")
        print("|---|" + "---|" * (len(small) + len(large)))
        for l in labels:
            cells = [fmt(rows[(coll, dt, n, b)].get(l), None, False) for b in small] + [fmt(rows[(coll, dt, n, b)].get(l), None, True) for b in large]
            print(f"| {l} | " + " | ".join(cells) + " |")


if __name__ == "__main__":
    main(sys.argv[1:])
