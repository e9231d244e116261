"""Offline tool chain: schedule generator CLI, LogGP simulator (classical model and the mode that
reproduces the simulator shipped with the reference), parameter fitter, selector."""
import subprocess
import sys
import xml.etree.ElementTree as ET
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from tools.loggp_param import get_loggp_param as fitter  # noqa: E402
from tools.loggp_sim import sim as S  # noqa: E402
from tools.schedule_generator import main as gen  # noqa: E402


@pytest.fixture()
def world(tmp_path):
    """Two parameter files with round numbers and two topologies (2 or 4 groups of 4 nodes, one NIC per group)."""
    (tmp_path / "intra.csv").write_text("s,L,o_s,o_r,g,G\n1,10,5,6,8,1\n2,10,5,6,8,1\n")
    (tmp_path / "inter.csv").write_text("s,L,o_s,o_r,g,G\n1,100,5,6,80,10\n2,100,5,6,80,10\n")

    def topo(groups):
        body = ""
        for g in range(groups):
            nodes = "".join(f'<node id="{4 * g + i}"/>' for i in range(4))
            body += f'<group level="0" id="{g}" ports="1" param_file="{tmp_path / "intra.csv"}">{nodes}</group>'
        p = tmp_path / f"topo{groups}.xml"
        p.write_text(f'<topo num_nodes="{4 * groups}" num_levels="2"><group level="1" id="0" param_file="{tmp_path / "inter.csv"}">{body}</group></topo>')
        return p

    def sched(transfers, name="s"):
        p = tmp_path / f"{name}.xml"
        rows = "\n".join(f'  <transfer id="{i}" size="{sz}" src="{a}" dst="{b}" deps="{d}"/>' for i, (sz, a, b, d) in enumerate(transfers))
        p.write_text(f'<collective name="t" nodes="16" buffer_size="1">\n  # (round 0)\n{rows}\n</collective>\n')
        return p

    return topo, sched


CASES = {
    # name: (transfers, groups, clean radix1, compat radix 1, compat radix 4)
    "intra": ([(1024, 0, 1, "-1")], 2, 1044, 2067, 2067),
    "inter": ([(1024, 0, 4, "-1")], 2, 10341, 20571, 20571),
    "same_port_twice": ([(3, 0, 1, "-1"), (3, 0, 1, "-1")], 2, None, 35, 25),
    "independent": ([(1, 0, 1, "-1"), (1, 0, 1, "-1"), (1, 2, 3, "-1"), (1, 5, 6, "-1")], 2, None, 29, 21),
    "independent_inter": ([(2, 4, 0, "-1"), (2, 15, 8, "-1")], 4, 121, 131, 131),
    "chain": ([(1024, 0, 1, "-1"), (1024, 0, 1, "-1"), (1024, 2, 3, "-1"), (1024, 7, 5, "-1"), (1024, 5, 6, "3"), (1024, 6, 7, "4"), (1024, 3, 2, "2")], 2, 3 * 1044, 6201, 6201),
    "two_into_one": ([(2, 3, 0, "-1"), (2, 2, 0, "-1")], 2, None, 31, 23),
    "nic_contention": ([(2, 0, 4, "-1"), (2, 0, 4, "-1")], 2, None, 221, 151),
    "nic_same_sender": ([(2, 4, 0, "-1"), (2, 4, 8, "-1")], 4, None, 221, 151),
    "nic_then_dep": ([(5, 0, 4, "-1"), (5, 1, 5, "-1"), (5, 5, 8, "1")], 4, None, 432, 432),
    "join": ([(2, 0, 4, "-1"), (2, 1, 4, "-1"), (2, 5, 4, "1"), (2, 4, 1, "1,2")], 4, None, 365, 305),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_simulator_reproduces_recorded_and_classical_numbers(world, name):
    topo, sched = world
    transfers, groups, clean, c1, c4 = CASES[name]
    s, t = sched(transfers, name), topo(groups)
    assert S.simulate(s, t, radix=1, compat=True) == pytest.approx(c1)
    assert S.simulate(s, t, radix=4, compat=True) == pytest.approx(c4)
    if clean is not None:
        assert S.simulate(s, t, radix=1) == pytest.approx(clean)       # o_s + G(s-1) + L + o_r per hop


def test_simulator_cli_and_stats(world, tmp_path):
    topo, sched = world
    s, t = sched(CASES["intra"][0], "cli"), topo(2)
    r = subprocess.run([sys.executable, str(ROOT / "tools/loggp_sim/sim.py"), "--schedule", str(s), "--topo", str(t), "--radix", "1", "--output", str(tmp_path / "o/stats.json")],
                       capture_output=True, text=True)
    assert r.returncode == 0 and float(r.stdout.strip()) == pytest.approx(1044e6)
    assert "finish_time" in (tmp_path / "o/stats.json").read_text()


def test_contention_statistics_are_kept_per_group(world, tmp_path):
    """Reference: sim.py:124-153 prints attempts / successes / largest queue per level-0 group.  Two transfers leave group 0
    through its one NIC at the same time, a third stays inside group 1: group 0 shows one sender that had to wait."""
    topo, sched = world
    s, t = sched([(2, 0, 4, "-1"), (2, 1, 5, "-1"), (2, 6, 7, "-1")], "groups"), topo(2)
    sim = S.Simulator(s, t, radix=1)
    sim.run()
    g0, g1 = sim.group_stats["0"], sim.group_stats["1"]
    assert g0["send"] == {"attempts": 2, "success": 1, "waited": pytest.approx(20.0), "max_queue_size": 1}      # the NIC is busy for G s = 20
    assert g1["send"]["attempts"] == 1 and g1["send"]["success"] == 1 and g1["send"]["max_queue_size"] == 0
    assert g1["recv"]["attempts"] == 3 and g0["recv"]["attempts"] == 0
    sim.output_stats(tmp_path / "stats.json")
    assert '"groups"' in (tmp_path / "stats.json").read_text()
    sim.output_stats(tmp_path / "report.txt")
    rep = (tmp_path / "report.txt").read_text()
    assert "Send Contention" in rep and "Group 0: 1 / 2 = 0.5 attempts successful" in rep and "Max Queue Size: 1" in rep


def _chunked_nic_reference(sizes, G, mtu=4096):
    """What the reference's chunk-level scheduler does with transfers that share one NIC and are ready at the same time
    (schedulers/loggpc_scheduler.py:319-377): every transfer puts one chunk of at most `mtu` bytes into the NIC's FIFO, the NIC
    serves the queue head for G * bytes, and the owner of a served chunk queues its next one.  Returns when each transfer's
    last chunk has left the NIC."""
    left = list(sizes)
    queue = list(range(len(sizes)))
    t, done = 0.0, [0.0] * len(sizes)
    while queue:
        i = queue.pop(0)
        b = min(mtu, left[i])
        t += G * b
        left[i] -= b
        if left[i] > 0:
            queue.append(i)
        else:
            done[i] = t
    return done


def test_whole_message_nic_model_against_chunked_interleaving_for_large_transfers(world):
    """Two 64 MiB transfers and a 16 MiB one leave a group through its single NIC at the same time.  The NIC is never idle in
    either model, so the LAST transfer ends at the same time whether the NIC takes whole messages in order (this simulator) or
    4096-byte chunks round robin (the reference); the earlier ones end later with chunks.  The makespan of a schedule whose
    steps wait for all their transfers is therefore the same, which is what the fixtures above check on small messages."""
    topo, sched = world
    sizes = [64 << 20, 64 << 20, 16 << 20]
    s, t = sched([(sizes[0], 0, 4, "-1"), (sizes[1], 1, 5, "-1"), (sizes[2], 2, 6, "-1")], "big"), topo(2)
    sim = S.Simulator(s, t, radix=1)
    sim.run()
    G = 10.0
    chunked = _chunked_nic_reference(sizes, G)
    # time at which each transfer's bytes have left the source NIC in this simulator: it started o_s = 5 after time 0 and waited for the NIC
    fixed = 5 + 100 + 6                                                   # o_s + L + o_r of the inter-group profile
    left_nic = sorted(tk.done - fixed + G for tk in sim.tasks.values())   # done = nic start + G (s - 1) + L + o_r
    assert left_nic[-1] - 5 == pytest.approx(max(chunked), rel=1e-6)      # the last one: same time, the NIC was busy throughout
    assert left_nic[-1] - 5 == pytest.approx(G * sum(sizes), rel=1e-6)
    # the earlier ones: whole messages in order let the first finish after its own bytes; with chunks the 16 MiB transfer shares
    # the NIC three ways and needs almost three times its own bytes
    assert left_nic[0] - 5 == pytest.approx(G * sizes[0], rel=1e-6)
    assert min(chunked) > G * sizes[2] * 2.9


def test_simulator_rejects_bad_schedules(world):
    topo, sched = world
    bad = sched([("1024.0", 0, 1, "-1")], "float_size")
    with pytest.raises(ValueError):
        S.simulate(bad, topo(2))
    cyc = sched([(8, 0, 1, "1"), (8, 1, 0, "0")], "cycle")
    with pytest.raises(RuntimeError):
        S.simulate(cyc, topo(2))


def test_generator_cli_all_combinations_are_well_formed(tmp_path):
    for coll in ["allgather", "allreduce", "reduce", "bcast", "reduce_scatter"]:
        for algo in ["ring", "k_ring", "RD", "RM", "PRD", "PRM"]:
            out = tmp_path / f"{coll}_{algo}.xml"
            assert gen.main(["--collective", coll, "--num_nodes", "8", "--buffer_size", "8192", "--algorithm", algo, "--k", "2", "--output", str(out)]) == 0
            root = ET.parse(out).getroot()
            ts = root.findall("transfer")
            assert ts and all(int(t.get("size")) > 0 for t in ts)
            assert root.get("nodes") == "8"


def test_generated_schedules_simulate_and_rank_as_the_cost_model_says(tmp_path):
    # one measured-style profile: L 2 us, g 1 us, 100 GB/s; flat 8-node topology
    prof = tmp_path / "p.csv"
    prof.write_text("s,L,o_s,o_r,g,G\n1,2e-6,5e-7,5e-7,1e-6,1e-11\n1073741824,2e-6,5e-7,5e-7,1e-6,1e-11\n")
    topo = tmp_path / "flat.xml"
    topo.write_text(S.flat_topology_xml(8, str(prof)))
    times = {}
    for algo, k in [("ring", 1), ("PRD", 2), ("PRM", 8)]:
        for size in [8 * 8, 1 << 30]:
            out = tmp_path / f"{algo}_{size}.xml"
            out.write_text(gen.generate("allreduce", 8, size, algo, k))
            # egress bandwidth is shared on an NVSwitch: one port for large messages, concurrent injection for tiny ones
            times[(algo, size)] = S.simulate(out, topo, radix=8 if size < 4096 else 1)
    # latency bound: fewer steps win; bandwidth bound: the ring moves the fewest bytes
    assert times[("PRM", 64)] < times[("PRD", 64)] < times[("ring", 64)]
    assert times[("ring", 1 << 30)] < times[("PRD", 1 << 30)] < times[("PRM", 1 << 30)]
    # 2(n-1)/n * S / beta within 5 % for the ring at 1 GiB
    assert times[("ring", 1 << 30)] == pytest.approx(2 * 7 / 8 * (1 << 30) * 1e-11, rel=0.05)


def test_fitter_round_trip(tmp_path):
    # synthesise PRTT measurements from known LogGP parameters and recover them
    L, o_s, o_r, g, G, n, d = 2e-6, 4e-7, 6e-7, 1.5e-6, 1.25e-11, 16, 5e-6
    rows = ["size n d PRTT(1,0,s) PRTT(n,0,s) PRTT(n,d,s) PRTT_server(n-1,d,s)"]
    for s in [1, 1024, 65536, 1 << 20, 1 << 24]:
        p1 = 2 * (L + o_s + o_r + (s - 1) * G)
        gap = g + (s - 1) * G
        rows.append(f"{s} {n} {d} {p1} {p1 + (n - 1) * gap} {p1 + (n - 1) * (o_s + d)} {(n - 1) * (o_r + d)}")
    raw = tmp_path / "raw.csv"
    raw.write_text("\n".join(rows) + "\n")
    t = fitter.process_file(raw, tmp_path / "fit.csv")
    assert t[0, 4] == pytest.approx(g, rel=1e-6) and t[0, 5] == pytest.approx(G, rel=1e-6)
    assert np.allclose(t[:, 2], o_s) and np.allclose(t[:, 3], o_r)
    assert t[0, 1] == pytest.approx((2 * (L + o_s + o_r)) / 2)
    prof = S.Profile(tmp_path / "fit.csv")
    assert prof("G", 5000) == pytest.approx(G, rel=1e-6)


def test_selector_tables(tmp_path):
    from tools.selector import select
    prof = tmp_path / "p.csv"
    prof.write_text("s,L,o_s,o_r,g,G\n1,2e-6,5e-7,5e-7,1e-6,1e-11\n1073741824,2e-6,5e-7,5e-7,1e-6,1e-11\n")
    out = tmp_path / "tune.csv"
    assert select.main(["--profile", str(prof), "--ranks", "8", "--min", "8", "--max", str(1 << 28), "--output", str(out)]) == 0
    rows = [l.split(",") for l in out.read_text().splitlines() if not l.startswith("#")]
    ar = [r for r in rows if r[0] == "allreduce"]
    assert ar[0][3] in ("PRM", "PRD") and ar[-1][3] in ("RING", "K_RING", "DIRECT")       # latency-optimal first, bandwidth-optimal last
    assert int(ar[-1][2]) >= 1 << 60
    bench = tmp_path / "b.csv"
    bench.write_text("# coll,label,dtype,op,ranks,bytes,iters,time_us,algbw_GBs,busbw_GBs,check\n"
                     "allreduce,ours-RING-k-1,float,sum,8,8,10,50.0,0,0,ok\nallreduce,ours-PRM-k8,float,sum,8,8,10,9.0,0,0,ok\n"
                     "allreduce,ours-RING-k-1,float,sum,8,1048576,10,60.0,0,0,ok\nallreduce,ours-PRM-k8,float,sum,8,1048576,10,90.0,0,0,ok\n")
    assert select.main(["--from-bench", str(bench), "--output", str(out)]) == 0
    rows = [l.split(",") for l in out.read_text().splitlines() if not l.startswith("#")]
    assert rows[0][:5] == ["allreduce", "8", "8", "PRM", "8"] and rows[1][3] == "RING"
    # the in-switch path enters the model-driven table through a fit of its measured times: T = 30 us + bytes / 400 GB/s here
    nv = tmp_path / "nv.csv"
    nv.write_text("".join(f"allreduce,sw,float,sum,8,{b},10,{30.0 + b / 400e3:.3f},0,0,ok\n" for b in (1 << 20, 1 << 24, 1 << 28)))
    fit = select.fit_nvls([str(nv)], {"sw": ("NVLS", -1, None)})
    assert fit[("allreduce", 8)][0] == pytest.approx(30e-6, rel=1e-3) and fit[("allreduce", 8)][1] == pytest.approx(400e9, rel=1e-3)
    assert select.main(["--profile", str(prof), "--ranks", "8", "--min", "8", "--max", str(1 << 28), "--nvls-bench", str(nv), "--alias", "sw=NVLS:-1",
                        "--output", str(out)]) == 0
    rows = [l.split(",") for l in out.read_text().splitlines() if not l.startswith("#")]
    ar = [r for r in rows if r[0] == "allreduce"]
    assert ar[0][3] != "NVLS" and ar[-1][3] == "NVLS"             # 100 GB/s links in the profile: the switch wins the large sizes
    assert all(r[3] != "NVLS" for r in rows if r[0] != "allreduce")


# ---------------------------------------------------------------- per-rank lists and the matcher
def _transfers(xml: str):
    import re
    return re.findall(r'<transfer id="(\d+)" size="(\d+)" src="(\d+)" dst="(\d+)" deps="([^"]*)"', xml)


@pytest.mark.parametrize("coll", ["allgather", "allreduce", "bcast", "reduce", "reduce_scatter"])
def test_matched_per_rank_lists_equal_the_native_dump(coll):
    """Reference idea: tools/schedule_generator/saved/schedule_gen.py (a matcher of per-rank send / receive lists)."""
    from tools.schedule_generator import per_rank as P
    for algo, k in [("ring", 1), ("k_ring", 2), ("rd", 1), ("rm", 3), ("prd", 1), ("prm", 2), ("prm", 8)]:
        for n in (2, 3, 4, 6, 8):
            if algo == "k_ring" and n % k:
                continue
            size = 4096 * n
            native = gen.generate(coll, n, size, algo, k)
            matched = P.match(P.all_rank_lists(coll, n, size, algo, k), coll, algo, size)
            assert _transfers(native) == _transfers(matched), (coll, algo, k, n)
            ET.fromstring("\n".join(l for l in matched.splitlines() if not l.strip().startswith("#")))


def test_per_rank_ring_allgather_lists_and_matcher_errors():
    """Reference: saved/coll/allgather.py:16-62 — ring allgather as (sends, recvs) per rank."""
    from tools.schedule_generator import per_rank as P
    n, size = 4, 4096
    for r in range(n):
        sends, recvs = P.rank_lists("allgather", n, size, r)
        assert [s["to"] for s in sends] == [(r + 1) % n] * (n - 1)
        assert [rc["from"] for rc in recvs] == [(r - 1) % n] * (n - 1)
        assert [s["tag"] for s in sends] == list(range(n - 1)) and all(s["size"] == size // n for s in sends)
        # block (r-1-i) mod n lands at its own offset
        assert [rc["offset"] for rc in recvs] == [((r - 1 - i) % n) * (size // n) for i in range(n - 1)]
        # what is forwarded in step i is what arrived in step i-1
        assert sends[0]["deps"] == [] and all(s["deps"] == [((r - 1) % n, i - 1)] for i, s in enumerate(sends) if i)
    lists = P.all_rank_lists("allgather", n, size)
    lists[2][1].pop()                      # rank 2 forgets its last receive
    with pytest.raises(ValueError, match="no matching receive"):
        P.match(lists, "allgather", "ring", size)
    lists = P.all_rank_lists("allgather", n, size)
    lists[1][0].pop()                      # rank 1 forgets its last send
    with pytest.raises(ValueError, match="without a send"):
        P.match(lists, "allgather", "ring", size)
    lists = P.all_rank_lists("allgather", n, size)
    lists[0][0][1]["size"] += 1
    with pytest.raises(ValueError, match="meets receive"):
        P.match(lists, "allgather", "ring", size)


def test_standalone_k_ring_generator(tmp_path):
    """Reference: saved/k-ring.py KRingScheduleGenerator (allgather / reduce / broadcast; allreduce was left empty)."""
    from tools.schedule_generator import per_rank as P
    for coll in ["allgather", "allreduce", "bcast", "reduce", "reduce_scatter"]:
        xml = P.k_ring_xml(8, 8 * 4097, 2, coll)
        assert 'algorithm="k_ring" k="2"' in xml and len(_transfers(xml)) > 0
    with pytest.raises(ValueError, match="divisible"):
        P.k_ring_xml(8, 4096, 3, "allgather")
    out = subprocess.run([sys.executable, str(ROOT / "tools/schedule_generator/per_rank.py"), "--collective", "allgather", "--num_nodes", "4",
                          "--buffer_size", "4096", "--rank", "1"], capture_output=True, text=True, check=True).stdout
    import json
    rec = json.loads(out.strip().splitlines()[-1])
    assert rec["rank"] == 1 and len(rec["sends"]) == 3 and len(rec["recvs"]) == 3


def test_shipped_samples_simulate(tmp_path):
    """Sample schedules, topologies and profiles under tools/loggp_sim (reference: tools/loggp_sim/schedules, profiles)."""
    sim = ROOT / "tools" / "loggp_sim"

    def run(sched, topo, radix=1):
        out = subprocess.run([sys.executable, str(sim / "sim.py"), "--schedule", str(sim / "schedules" / sched), "--topo", str(sim / "topo" / topo), "--radix", str(radix)],
                             capture_output=True, text=True, check=True, cwd=tmp_path).stdout
        return float(out.strip().splitlines()[-1])

    ring, k2, direct = run("8_ring_allgather.xml", "8_flat.xml"), run("8_kring_k_2_allgather.xml", "8_flat.xml"), run("8_direct_allgather.xml", "8_flat.xml")
    assert ring == pytest.approx(k2) and direct < ring                 # one switch: group size does not matter, fewer steps do
    flat_ring, flat_k8 = run("16_ring_allreduce.xml", "2x8_two_level.xml"), run("16_kring_k_8_allreduce.xml", "2x8_two_level.xml")
    assert flat_k8 < flat_ring                                         # two nodes: keeping most hops inside a node pays
    # the samples are what the generator writes today
    assert (sim / "schedules" / "8_direct_allreduce.xml").read_text() == gen.generate("allreduce", 8, 1 << 24, "direct", 1)
    assert (sim / "schedules" / "8_ring_allgather.xml").read_text() == gen.generate("allgather", 8, 8 * 4097, "ring", 1)


def _select_in_child(env_extra, queries):
    """AUTO's choice for (nranks, collective, bytes) in a fresh process (the tuning table is read once per process)."""
    code = ("import ctypes as C, sys, json; sys.path.insert(0, %r); from piccl_b200 import _native as N; l = N.lib(); out = []\n"
            "names = {v: k for k, v in N.ALGO.items()}\n"
            "for n, coll, b in json.loads(sys.argv[1]):\n"
            "    k = C.c_int(-9); a = l.piccl_select_algorithm(n, N.COLL[coll], C.c_ulonglong(b), C.byref(k)); out.append([names[a], k.value])\n"
            "print(json.dumps(out))") % str(ROOT)
    import json
    import os
    r = subprocess.run([sys.executable, "-c", code, json.dumps(queries)], env=dict(os.environ, **env_extra), capture_output=True, text=True, check=True)
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_builtin_rule_and_tuning_table_of_the_library():
    """src/runtime/selector.cc: the built-in rule, and a table given through PICCL_TUNE_FILE, which wins where it has a row."""
    q = [[8, "allreduce", 1024], [8, "allreduce", 1 << 20], [8, "allreduce", 1 << 28], [2, "allreduce", 16 << 20], [8, "allgather", 4096],
         [8, "allgather", 1 << 20], [8, "broadcast", 1 << 20], [4, "reduce_scatter", 8192]]
    got = _select_in_child({"PICCL_TUNE_FILE": ""}, q)
    assert got == [["PRM", 8], ["PRD", 2], ["RING", -1], ["RING", -1], ["PRM", 8], ["RING", -1], ["RING", -1], ["PRM", 4]]
    # the table derived from the 8-GPU sweep: first row of its collective and rank count with max_bytes >= size
    table = ROOT / "tools" / "selector" / "tables" / "b200_8gpu.csv"
    got = _select_in_child({"PICCL_TUNE_FILE": str(table)}, [[8, "allreduce", 1024], [8, "allreduce", 32768], [8, "allreduce", 2 << 20], [8, "allreduce", 1 << 30],
                                                           [4, "allreduce", 1024]])
    assert got[0] == ["PRM", 8] and got[1] == ["PRM", 2] and got[2] == ["PRD", -1] and got[3][0] == "RING"     # no window: the in-switch rows are skipped
    assert got[4] == ["PRM", 4]                                    # no row for 4 ranks in that table: the built-in rule
    # with an NVLink multicast window (piccl_select_algorithm_ex): large all-reduces and mid-size all-gathers / reduce-scatters go
    # through the switch from four ranks on; small ones, two ranks, broadcast and reduce do not
    code = ("import ctypes as C, sys, json; sys.path.insert(0, %r); from piccl_b200 import _native as N; l = N.lib(); out = []\n"
            "names = {v: k for k, v in N.ALGO.items()}\n"
            "for n, coll, b in json.loads(sys.argv[1]):\n"
            "    k = C.c_int(-9); a = l.piccl_select_algorithm_ex(n, N.COLL[coll], C.c_ulonglong(b), 1, C.byref(k)); out.append(names[a])\n"
            "print(json.dumps(out))") % str(ROOT)
    import json
    import os
    qs = [[8, "allreduce", 25 << 20], [8, "allreduce", 1 << 20], [2, "allreduce", 1 << 28], [4, "allreduce", 1 << 28], [8, "allgather", 1 << 20], [8, "allgather", 64 << 20],
          [8, "allgather", 32 << 10], [8, "reduce_scatter", 4 << 20], [8, "broadcast", 1 << 28], [8, "reduce", 1 << 28]]
    r = subprocess.run([sys.executable, "-c", code, json.dumps(qs)], env=dict(os.environ, PICCL_TUNE_FILE=""), capture_output=True, text=True, check=True)
    assert json.loads(r.stdout.strip().splitlines()[-1]) == ["NVLS", "PRD", "RING", "NVLS", "NVLS", "RING", "PRM", "NVLS", "RING", "RING"]
    # the same questions answered from the 8-GPU table: its in-switch rows apply when there is a window
    r = subprocess.run([sys.executable, "-c", code, json.dumps([q for q in qs if q[0] == 8])], env=dict(os.environ, PICCL_TUNE_FILE=str(table)), capture_output=True, text=True, check=True)
    assert json.loads(r.stdout.strip().splitlines()[-1]) == ["NVLS", "PRD", "NVLS", "RING", "PRM", "NVLS", "RING", "RING"]


def test_profile_fitted_from_a_measured_ring_sweep_predicts_the_other_schedules(tmp_path):
    """tools/loggp_param/fit_from_sweep.py on the committed 8-GPU sweep: the ring is reproduced by construction, the grouped ring within
    10 %, the recursive all-reduces from 4 MiB within 15 % (median) once the reduction cost per byte is fitted."""
    import csv
    import math
    import re
    from tools.loggp_param import fit_from_sweep as F
    from tools.selector import select
    sweep = str(ROOT / "benchmarks" / "results" / "sweep_8.csv")
    out = tmp_path / "p.csv"
    assert F.main([sweep, "--ranks", "8", "--output", str(out)]) == 0
    rows = [l.split(",") for l in out.read_text().splitlines()[1:]]
    G = float(rows[0][5])
    assert 550e9 < 1 / G < 700e9                                   # asymptotic bandwidth per hop, bytes/s: the 600+ GB/s the large ring runs at
    assert out.read_text() == (ROOT / "tools" / "loggp_sim" / "profiles" / "b200_executor_8gpu_loggp.csv").read_text()
    gamma, med = F.fit_gamma(sweep, str(out), 8)
    assert 2e-13 < gamma < 1.2e-12 and med < 0.15
    meas = {}
    for r in csv.reader(open(sweep)):
        m = re.match(r"ours-([A-Z_]+)-k(-?\d+)", r[1]) if len(r) > 8 and r[0] == "allreduce" and r[2] == "float" else None
        if m and int(r[5]) >= 1024:
            meas[(m.group(1), int(m.group(2)), int(r[5]))] = float(r[7])
    for (algo, k, b), t in meas.items():
        if algo in ("RING", "K_RING"):
            p = 2.5 + 1e6 * select.predict(str(out), "allreduce", 8, b, algo, k, radix=1, gamma=gamma)
            assert abs(math.log(p / t)) < (0.05 if algo == "RING" else 0.10), (algo, k, b, p, t)      # the ring was fitted without the reduction cost


def test_trace_summary(tmp_path, capsys):
    """tools/trace/summarize.py on files in the format src/runtime/trace.cu writes."""
    import json
    from tools.trace import summarize as T
    for rank in range(2):
        ev = [{"name": "allreduce/RING", "ph": "X", "pid": rank, "tid": 0, "ts": 10.0 * i, "dur": 100.0 + rank, "args": {"bytes": 26214400, "k": 0, "ctas": 64}} for i in range(3)]
        ev.append({"name": "allgather/PRM", "ph": "X", "pid": rank, "tid": 0, "ts": 99.0, "dur": 8.0, "args": {"bytes": 4096, "k": 8, "ctas": 1}})
        (tmp_path / f"run.{rank}.json").write_text(json.dumps({"traceEvents": ev}))
    files, events = T.load([str(tmp_path / "run")])
    assert len(files) == 2 and len(events) == 8
    rows, per_rank = T.summarize(events)
    assert rows[0]["collective"] == "allreduce" and rows[0]["algorithm"] == "RING" and rows[0]["size"] == "<=64M" and rows[0]["calls"] == 6
    assert abs(rows[0]["algbw_GBs"] - 26214400 / 100.5 / 1e3) < 0.5
    assert rows[1]["size"] == "<=4K" and per_rank[1] > per_rank[0]
    assert T.main([str(tmp_path / "run.0.json")]) == 0 and "4 calls in 1 file" in capsys.readouterr().out
    assert T.bucket(1 << 31) == ">1G" and T.bucket(1024) == "<=1K" and T.bucket(1025) == "<=4K"


def test_fitter_recovers_random_parameters_and_refuses_degenerate_input(tmp_path):
    """Synthetic PRTT data from known LogGP parameters (with the formulas of the docstring inverted) come back within rounding,
    for random parameter sets; a train of a single message cannot be fitted and says so."""
    rng = np.random.default_rng(7)
    for trial in range(20):
        L, g, G = rng.uniform(1e-6, 2e-5), rng.uniform(1e-7, 5e-6), rng.uniform(1e-12, 1e-10)
        n, d = int(rng.integers(2, 40)), rng.uniform(0, 1e-5)
        sizes = np.unique(rng.integers(1, 1 << 22, size=8))
        rows = []
        for s in sizes:
            o_s, o_r = rng.uniform(1e-7, 5e-6), rng.uniform(1e-7, 5e-6)
            p1 = 2 * L if s == sizes[0] else rng.uniform(1e-6, 1e-4)
            pn0 = p1 + (n - 1) * (g + G * (s - 1))
            pnd = p1 + (n - 1) * (o_s + d)
            psrv = (n - 1) * (o_r + d)
            rows.append((s, n, d, p1, pn0, pnd, psrv, o_s, o_r))
        raw = tmp_path / f"raw{trial}.txt"
        raw.write_text("size n d p1 pn0 pnd psrv\n" + "\n".join(" ".join(repr(float(x)) for x in r[:7]) for r in rows) + "\n")
        t = fitter.fit(fitter.read_raw(raw))
        assert t[0, 1] == pytest.approx(L, rel=1e-9) and t[0, 4] == pytest.approx(g, rel=1e-4, abs=1e-12) and t[0, 5] == pytest.approx(G, rel=1e-6)
        for row, r in zip(t, rows):
            assert row[2] == pytest.approx(r[7], rel=1e-6, abs=1e-12) and row[3] == pytest.approx(r[8], rel=1e-6, abs=1e-12)
    bad = tmp_path / "bad.txt"
    bad.write_text("64 1 0 1e-5 1e-5 1e-5 1e-5\n128 1 0 1e-5 1e-5 1e-5 1e-5\n")
    with pytest.raises(ValueError, match="n >= 2"):
        fitter.fit(fitter.read_raw(bad))
    with pytest.raises(ValueError, match="no data rows"):
        (tmp_path / "empty.txt").write_text("only a header\n")
        fitter.read_raw(tmp_path / "empty.txt")


def test_cpu_only_schedule_check_script(tmp_path):
    """benchmarks/config1_cpu.py: validator + generator + simulator over the headline sizes (data up to 1 MiB here to stay quick)."""
    out = tmp_path / "c1.csv"
    r = subprocess.run([sys.executable, str(ROOT / "benchmarks" / "config1_cpu.py"), "--out", str(out), "--data-max", str(1 << 20)], capture_output=True, text=True)
    assert r.returncode == 0 and "0 failed" in r.stdout, r.stdout + r.stderr
    rows = [l.split(",") for l in out.read_text().splitlines()[1:]]
    assert len(rows) == 28 * 7 and all(x[4] == "ok" for x in rows)
    assert {x[3] for x in rows if int(x[2]) <= 1 << 20} == {"data"} and {x[3] for x in rows if int(x[2]) > 1 << 20} == {"symbolic"}
