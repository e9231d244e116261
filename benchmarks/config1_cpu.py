#!/usr/bin/env python
"""CPU-only schedule check (no GPU): all-reduce on p = 8 ranks with RING, K_RING (k = 2, 4), PRD, PRM (k = 2, 8) and DIRECT, fp32 sum,
message sizes 8 B - 1 GiB in powers of two.

For every (algorithm, size): the programs of all ranks are executed against each other by the data-flow validator
(src/coll/validate.cc) on buffers drawn from seed-0 uniform[-1,1) and compared with a serial sum (up to --data-max bytes; above
that the same execution runs without data: every output element covered, FIFO order, bounded FIFOs), the schedule is written
by tools/schedule_generator and its finish time is predicted by tools/loggp_sim with the B200 profile fitted from the measured
ring sweep.  Writes a CSV and prints a summary; exit code 1 if any schedule fails.

    python benchmarks/config1_cpu.py [--out benchmarks/results/config1_cpu.csv] [--data-max 67108864]
"""
from __future__ import annotations

import argparse
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from piccl_b200 import schedule as S  # noqa: E402
from tools.selector import select  # noqa: E402

ALGOS = [("RING", -1), ("K_RING", 2), ("K_RING", 4), ("PRD", -1), ("PRM", 2), ("PRM", 8), ("DIRECT", -1)]
PROFILE = "tools/loggp_sim/profiles/b200_executor_8gpu_loggp.csv"
GAMMA = 5.8e-13          # reduction cost per received byte fitted by tools/loggp_param/fit_from_sweep.py --fit-gamma


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(ROOT / "benchmarks" / "results" / "config1_cpu.csv"))
    ap.add_argument("--data-max", type=int, default=64 << 20, help="largest message validated with real data (bytes)")
    ap.add_argument("--ranks", type=int, default=8)
    a = ap.parse_args(argv)
    n, rows, bad, t0 = a.ranks, [], 0, time.time()
    size = 8
    while size <= 1 << 30:
        count = size // 4
        for algo, k in ALGOS:
            with_data = size <= a.data_max
            v = S.validate("allreduce", algo, n, count, k=k, op="sum", fifo_cap=2, seg_elems=(512 * 1024) // 4, n_cta=4 if with_data else 64, symbolic=not with_data)
            pred = 1e6 * select.predict(PROFILE, "allreduce", n, size, algo, k, radix=n if size <= 16384 else 1, gamma=GAMMA)
            rows.append((algo, k, size, "data" if with_data else "symbolic", "ok" if v.ok else "FAIL: " + v.error, v.max_abs_err, v.bytes_sent_max_rank, pred))
            bad += 0 if v.ok else 1
        size *= 2
    with open(a.out, "w") as f:
        f.write("# algorithm,k,bytes,check,result,max_abs_err,bytes_sent_per_rank,predicted_us\n")
        for r in rows:
            f.write(f"{r[0]},{r[1]},{r[2]},{r[3]},{r[4]},{r[5]:.3g},{r[6]},{r[7]:.2f}\n")
    print(f"{len(rows)} schedules checked in {time.time() - t0:.1f} s, {bad} failed -> {a.out}")
    for sz in (8, 1 << 20, 1 << 30):
        best = min((r for r in rows if r[2] == sz), key=lambda r: r[7])
        print(f"  {sz:>11d} B: fastest predicted {best[0]}{'' if best[1] < 0 else ' k=' + str(best[1])} {best[7]:.1f} us")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
