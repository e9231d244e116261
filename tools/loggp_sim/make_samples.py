#!/usr/bin/env python
"""Regenerates the sample inputs that ship with the simulator:

  profiles/b200_l1_mock_loggp.csv   a MOCK second network level: every parameter of the measured NVLink profile
                                    (profiles/b200_nvlink_prtt_cta16_loggp.csv) times 10, for multi-node what-if runs
                                    without a cluster (the reference ships the same kind of stand-in,
                                    tools/loggp_sim/profiles/nccl_l1_simple_loggp_mock.csv)
  topo/8_flat.xml                   8 GPUs in one NVSwitch domain
  topo/2x8_two_level.xml            2 nodes of 8 GPUs, 4 NICs per node, mock profile between the nodes
  schedules/*.xml                   a few schedules from the schedule generator (8 x 4097-byte all-gathers like the
                                    reference's samples, tools/loggp_sim/schedules/8_*_allgather.xml, and 16 MiB all-reduces)
"""
from __future__ import annotations

import csv
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))
from tools.schedule_generator import main as gen  # noqa: E402

PROFILE = "tools/loggp_sim/profiles/b200_nvlink_prtt_cta16_loggp.csv"
MOCK = "tools/loggp_sim/profiles/b200_l1_mock_loggp.csv"
SAMPLES = [("8_ring_allgather", "ring", 1, 8), ("8_kring_k_2_allgather", "k_ring", 2, 8), ("8_kring_k_4_allgather", "k_ring", 4, 8),
           ("8_direct_allgather", "direct", 1, 8), ("8_direct_allreduce", "direct", 1, 8), ("16_kring_k_8_allreduce", "k_ring", 8, 16),
           ("16_ring_allreduce", "ring", 1, 16)]


def nodes(a: int, b: int) -> str:
    return "".join(f'<node id="{i}"/>' for i in range(a, b))


def main() -> int:
    rows = list(csv.reader(open(HERE / "profiles" / Path(PROFILE).name)))
    with open(HERE / "profiles" / Path(MOCK).name, "w") as f:
        f.write(",".join(rows[0]) + "\n")
        for r in rows[1:]:
            f.write(",".join([r[0]] + ["%.15e" % (float(x) * 10) for x in r[1:]]) + "\n")
    (HERE / "topo").mkdir(exist_ok=True)
    (HERE / "schedules").mkdir(exist_ok=True)
    (HERE / "topo" / "8_flat.xml").write_text(f'<topo num_nodes="8" num_levels="1">\n  <group level="0" id="0" param_file="{PROFILE}">{nodes(0, 8)}</group>\n</topo>\n')
    (HERE / "topo" / "2x8_two_level.xml").write_text(
        f'<topo num_nodes="16" num_levels="2">\n  <group level="1" id="0" param_file="{MOCK}">\n'
        f'    <group level="0" id="0" ports="4" param_file="{PROFILE}">{nodes(0, 8)}</group>\n'
        f'    <group level="0" id="1" ports="4" param_file="{PROFILE}">{nodes(8, 16)}</group>\n  </group>\n</topo>\n')
    for name, algo, k, n in SAMPLES:
        coll = name.split("_")[-1]
        (HERE / "schedules" / f"{name}.xml").write_text(gen.generate(coll, n, n * 4097 if coll == "allgather" else 1 << 24, algo, k))
    print(f"wrote {len(SAMPLES)} schedules, 2 topologies, 1 mock profile under {HERE}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
