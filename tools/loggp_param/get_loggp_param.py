#!/usr/bin/env python
"""LogGP parameter fit from PRTT measurements (the method of Hoefler et al.).

Input: whitespace separated rows  `size n d PRTT(1,0,s) PRTT(n,0,s) PRTT(n,d,s) PRTT_server(n-1,d,s)`
(a header line is allowed), as written by tools/loggp_bench.  Output: CSV `s,L,o_s,o_r,g,G` in
seconds and seconds per byte, one row per message size.  Same maths as the reference's
tools/loggp_param/get_loggp_param.py:24-44:
    g, G  intercept and slope of (PRTT(n,0,s) - PRTT(1,0,s)) / (n-1) against (s-1)
    L     PRTT(1,0,s) of the smallest size / 2
    o_s   (PRTT(n,d,s) - PRTT(1,0,s)) / (n-1) - d          per size
    o_r   (PRTT_server(n-1,d,s) - d(n-1)) / (n-1)          per size
The fit is a plain least-squares line (numpy); no pandas / scikit-learn needed.
"""
from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

import numpy as np


def read_raw(path) -> np.ndarray:
    rows = []
    with open(path) as f:
        for line in f:
            parts = line.split()
            if len(parts) < 7:
                continue
            try:
                rows.append([float(x) for x in parts[:7]])
            except ValueError:
                continue      # header
    if not rows:
        raise ValueError(f"{path}: no data rows")
    a = np.array(rows)
    return a[np.argsort(a[:, 0], kind="stable")]


def fit(raw: np.ndarray) -> np.ndarray:
    size, n, d, p1, pn0, pnd, psrv = raw.T
    if np.any(n < 2):
        raise ValueError("PRTT rows need n >= 2 messages per train (the gap is (PRTT(n,0,s) - PRTT(1,0,s)) / (n - 1))")
    gap = (pn0 - p1) / (n - 1)
    if len(size) >= 2 and np.ptp(size) > 0:
        G, g = np.polyfit(size - 1, gap, 1)
    else:
        G, g = 0.0, float(gap[0])
    L = p1[0] / 2
    o_s = (pnd - p1) / (n - 1) - d
    o_r = (psrv - d * (n - 1)) / (n - 1)
    out = np.empty((len(size), 6))
    out[:, 0] = size; out[:, 1] = L; out[:, 2] = o_s; out[:, 3] = o_r; out[:, 4] = g; out[:, 5] = G
    return out


def write_csv(path, table: np.ndarray) -> None:
    with open(path, "w") as f:
        f.write("s,L,o_s,o_r,g,G\n")
        for r in table:
            f.write(f"{int(r[0])}," + ",".join(f"{x:.15e}" for x in r[1:]) + "\n")


def process_file(src, dst) -> np.ndarray:
    t = fit(read_raw(src))
    write_csv(dst, t)
    return t


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Fit LogGP parameters from PRTT measurements.")
    ap.add_argument("inputs", nargs="*", help="raw PRTT files (default: $PICCL_HOME/data/osu_loggp_raw/*.csv)")
    ap.add_argument("--out-dir", default=None, help="default: $PICCL_HOME/data/loggp_param, or next to the input")
    a = ap.parse_args(argv)
    inputs = [Path(p) for p in a.inputs]
    home = os.environ.get("PICCL_HOME")
    if not inputs:
        if not home:
            print("give input files or set PICCL_HOME", file=sys.stderr)
            return 2
        inputs = sorted((Path(home) / "data" / "osu_loggp_raw").glob("*.csv"))
    for src in inputs:
        out_dir = Path(a.out_dir) if a.out_dir else (Path(home) / "data" / "loggp_param" if home and not a.inputs else src.parent)
        out_dir.mkdir(parents=True, exist_ok=True)
        dst = out_dir / (src.stem + "_loggp.csv")
        t = process_file(src, dst)
        print(f"{src} -> {dst}: L={t[0, 1]:.3e}s g={t[0, 4]:.3e}s G={t[0, 5]:.3e}s/B ({1 / t[0, 5] / 1e9 if t[0, 5] > 0 else float('inf'):.1f} GB/s)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
