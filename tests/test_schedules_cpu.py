"""CPU data-flow validation of every collective x algorithm x k x rank count
(the reference ships no such test; its only check is the external OSU validation
run, README.md:40-44)."""
import itertools
import json
import xml.etree.ElementTree as ET

import pytest

from piccl_b200 import schedule as S

COLLS = ["allgather", "allreduce", "broadcast", "reduce", "reduce_scatter"]
ALGOS = ["RING", "K_RING", "RD", "RM", "PRD", "PRM", "DIRECT"]


@pytest.mark.parametrize("coll", COLLS)
@pytest.mark.parametrize("algo", ALGOS)
def test_all_rank_counts_and_radices(coll, algo):
    for n, k, in_place in itertools.product([1, 2, 3, 4, 5, 6, 7, 8, 9, 12, 16], [-1, 2, 3, 4, 8], [False, True]):
        v = S.validate(coll, algo, n, 257, k=k, root=n // 2, in_place=in_place, n_cta=3, seg_elems=32)
        assert v.ok, f"{coll} {algo} n={n} k={k} in_place={in_place}: {v.error}"


@pytest.mark.parametrize("algo", ALGOS)
def test_deferred_counter_updates_never_deadlock(algo):
    """The executor variant that publishes its FIFO counters only when it is about to block (exec_impl.cuh, DEFER):
    every schedule still terminates with the right data, also with the smallest FIFO."""
    for coll in COLLS:
        for n, k, in_place in itertools.product([2, 3, 4, 6, 8, 9, 16], [-1, 2, 4, 8], [False, True]):
            v = S.validate(coll, algo, n, 257, k=k, root=n - 1, in_place=in_place, n_cta=2, seg_elems=32, fifo_cap=2, deferred=True)
            assert v.ok, f"{coll} {algo} n={n} k={k} in_place={in_place}: {v.error}"


@pytest.mark.parametrize("op", ["sum", "prod", "max", "min"])
@pytest.mark.parametrize("integer", [False, True])
def test_ops_exact_for_integers(op, integer):
    for coll, algo in itertools.product(["allreduce", "reduce", "reduce_scatter"], ALGOS):
        v = S.validate(coll, algo, 8, 500, k=4, op=op, integer=integer, n_cta=2, seg_elems=64)
        assert v.ok, f"{coll} {algo} {op}: {v.error}"
        if integer:
            assert v.max_abs_err == 0.0


def test_headline_config_p8_fp32_sum_small_sizes_with_data():
    # allreduce, p = 8, RING / K_RING k=2,4 / PRD / PRM k=2,8, seed-0 uniform[-1,1) fp32 against a serial sum
    for algo, k in [("RING", -1), ("K_RING", 2), ("K_RING", 4), ("PRD", -1), ("PRM", 2), ("PRM", 8)]:
        for nbytes in [8, 64, 4096, 1 << 16, 1 << 20]:
            v = S.validate("allreduce", algo, 8, nbytes // 4, k=k, n_cta=4, seg_elems=4096)
            assert v.ok, f"{algo} k={k} {nbytes} B: {v.error}"
            assert v.max_abs_err < 1e-4


def test_headline_config_large_sizes_symbolic():
    # up to 1 GiB the programs are checked for FIFO order and complete output coverage without data
    for algo, k in [("RING", -1), ("K_RING", 2), ("K_RING", 4), ("PRD", -1), ("PRM", 2), ("PRM", 8)]:
        for nbytes in [1 << 24, 1 << 27, 1 << 30]:
            v = S.validate("allreduce", algo, 8, nbytes // 4, k=k, n_cta=32, symbolic=True)
            assert v.ok, f"{algo} k={k} {nbytes} B: {v.error}"


def test_traffic_matches_cost_model():
    n, count = 8, 8 * 1024
    S_bytes = count * 4
    v = S.validate("allreduce", "RING", n, count, n_cta=1, seg_elems=count)
    assert v.bytes_sent_max_rank == 2 * (n - 1) * S_bytes // n
    v = S.validate("allreduce", "PRD", n, count, n_cta=1, seg_elems=count)
    assert v.bytes_sent_max_rank == 3 * S_bytes
    v = S.validate("allreduce", "PRM", n, count, k=8, n_cta=1, seg_elems=count)
    assert v.bytes_sent_max_rank == 7 * S_bytes
    for algo in ALGOS:
        v = S.validate("allgather", algo, n, count, k=2, n_cta=1, seg_elems=count, elem_size=4)
        assert v.bytes_sent_max_rank == (n - 1) * S_bytes, algo


def test_direct_schedules_move_the_minimum_in_two_exchanges():
    n, count = 8, 7 * 8 * 1024
    S_bytes = count * 4
    # all-reduce: the ring's traffic in 3 steps (contributions out, reduce + sums out, sums stored)
    v = S.validate("allreduce", "DIRECT", n, count, n_cta=1, seg_elems=count)
    assert v.ok and v.bytes_sent_max_rank == 2 * (n - 1) * S_bytes // n
    assert json.loads(S.schedule_json("allreduce", "DIRECT", n, count, 3))["steps"] == 3
    prog = json.loads(S.schedule_json("allreduce", "DIRECT", n, count, 3))["actions"]
    assert [len(a["send"]) for a in prog] == [1] * 7 + [7] + [0] * 7 and [len(a["recv"]) for a in prog] == [0] * 7 + [7] + [1] * 7
    # broadcast: nobody sends more than the message, the root sends it exactly once
    v = S.validate("broadcast", "DIRECT", n, count, root=5, n_cta=1, seg_elems=count)
    assert v.ok and v.bytes_sent_max_rank == S_bytes
    # reduce: each rank sends at most its vector once
    v = S.validate("reduce", "DIRECT", n, count, root=2, n_cta=1, seg_elems=count)
    assert v.ok and v.bytes_sent_max_rank == S_bytes
    # all-gather / reduce-scatter resolve to one exchange with everybody
    r = S.resolve("allgather", "DIRECT", -1, n)
    assert (r.algo, r.k, r.radices) == ("PRM", 8, [8])
    # more than 8 ranks: one action cannot address everybody
    assert S.resolve("allreduce", "DIRECT", -1, 12).algo == "RING"


def test_permutation_oracle_vectors():
    # values of the reference's index formula (src/kernels/permutation_kernel.cu:166-207)
    assert S.permutation_index(0, 8, 2) == [0, 4, 2, 6, 1, 5, 3, 7]
    assert S.permutation_index(1, 8, 2) == [1, 5, 3, 7, 0, 4, 2, 6]
    assert S.permutation_index(3, 8, 2) == [3, 7, 1, 5, 2, 6, 0, 4]
    assert S.permutation_index(7, 8, 2) == [7, 3, 5, 1, 6, 2, 4, 0]
    assert S.permutation_index(5, 8, 8) == [5, 6, 7, 0, 1, 2, 3, 4]
    assert S.permutation_index(4, 9, 3) == [4, 7, 1, 5, 8, 2, 3, 6, 0]
    assert S.permutation_index(8, 9, 3) == [8, 2, 5, 6, 0, 3, 7, 1, 4]
    assert S.permutation_index(6, 16, 4) == [6, 10, 14, 2, 7, 11, 15, 3, 4, 8, 12, 0, 5, 9, 13, 1]
    assert S.permutation_index(5, 16, 2) == [5, 13, 1, 9, 7, 15, 3, 11, 4, 12, 0, 8, 6, 14, 2, 10]
    assert S.permutation_index(1, 8, 4) is None     # 8 is not a power of 4
    assert S.permutation_index(0, 6, 2) is None


def test_direct_placement_equals_permutation_table():
    # the block a permuted-recursive rank holds in receive order q is exactly perm[q]
    for n, b in [(8, 2), (4, 2), (16, 2), (9, 3), (16, 4), (8, 8)]:
        rad = S.resolve("allgather", "PRM", b, n).radices
        assert all(f == b for f in rad)
        for r in range(n):
            assert S.held_blocks(r, len(rad), rad, n, True) == S.permutation_index(r, n, b)


def test_resolve_defines_the_cases_the_reference_leaves_undefined():
    r = S.resolve("allgather", "PRM", 4, 8)          # reference: out-of-bounds writes
    assert sorted(r.radices) == [2, 4] and "mixed" in r.note
    r = S.resolve("allgather", "K_RING", 4, 2)       # reference: silently does nothing
    assert r.k == 2
    r = S.resolve("allreduce", "PRM", -1, 8)         # reference: K unset = -1, undefined behaviour
    assert r.k == 2 and r.radices == [2, 2, 2]
    r = S.resolve("allreduce", "K_RING", 3, 8)       # k does not divide n: plain ring, as the reference
    assert r.k == 8
    r = S.resolve("allreduce", "PRD", -1, 11)        # prime rank count: power-of-two core + followers
    assert r.core == 8
    r = S.resolve("allgather", "RD", -1, 11)
    assert r.algo == "RING"


def test_xml_is_well_formed_with_integer_sizes():
    for coll, algo, k in itertools.product(COLLS, ALGOS, [2, 4]):
        xml = S.schedule_xml(coll, algo, 8, 1024, k=k)
        root = ET.fromstring(xml)
        assert root.tag == "collective" and root.get("nodes") == "8"
        ids = set()
        for t in root.findall("transfer"):
            ids.add(int(t.get("id")))
            assert int(t.get("size")) > 0
            assert 0 <= int(t.get("src")) < 8 and 0 <= int(t.get("dst")) < 8 and t.get("src") != t.get("dst")
        for t in root.findall("transfer"):
            for d in t.get("deps").split(","):
                assert int(d) == -1 or int(d) in ids
        assert len(ids) > 0


def test_xml_transfer_counts():
    n = 8
    count = lambda **kw: len(ET.fromstring(S.schedule_xml(**kw)).findall("transfer"))
    assert count(coll="allgather", algo="RING", nranks=n, count=64) == n * (n - 1)
    assert count(coll="allreduce", algo="RING", nranks=n, count=64 * n) == 2 * n * (n - 1)
    assert count(coll="allreduce", algo="K_RING", nranks=n, count=64 * n, k=2) == 2 * n * (n - 1)
    assert count(coll="allreduce", algo="PRD", nranks=n, count=64) == 3 * n
    assert count(coll="allreduce", algo="PRM", nranks=n, count=64, k=8) == n * (n - 1)
    assert count(coll="broadcast", algo="RING", nranks=n, count=64) == n - 1
    assert count(coll="reduce", algo="PRD", nranks=n, count=64) == n - 1
