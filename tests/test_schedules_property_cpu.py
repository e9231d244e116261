"""Property tests of the schedule layer: random rank counts, radices, sizes, element sizes, CTA counts, segment sizes, roots and
strides, checked by the CPU data-flow validator (src/coll/validate.cc) with the smallest FIFO the runtime allows.  The reference
has no validator; its defects on such inputs are listed in the survey (K unset, rank counts that are no power of the radix, ...)."""
import sys
from pathlib import Path

import pytest
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from piccl_b200 import schedule as S  # noqa: E402

COLLS = ["allgather", "allreduce", "broadcast", "reduce", "reduce_scatter"]
ALGOS = ["RING", "K_RING", "RD", "RM", "PRD", "PRM", "DIRECT"]
COMMON = dict(deadline=None, derandomize=True, database=None, suppress_health_check=[HealthCheck.too_slow])


@settings(max_examples=400, **COMMON)
@given(coll=st.sampled_from(COLLS), algo=st.sampled_from(ALGOS), n=st.integers(1, 24), k=st.integers(-1, 9), count=st.integers(1, 700),
       elem_size=st.sampled_from([1, 2, 4, 8]), n_cta=st.integers(1, 5), seg=st.sampled_from([4, 16, 64, 1 << 20]), in_place=st.booleans(),
       root=st.integers(0, 23), deferred=st.booleans(), integer=st.booleans(), op=st.sampled_from(["sum", "max", "min"]))
def test_any_request_compiles_to_a_correct_program(coll, algo, n, k, count, elem_size, n_cta, seg, in_place, root, deferred, integer, op):
    v = S.validate(coll, algo, n, count, k=k, root=root % n, elem_size=elem_size, in_place=in_place, op=op, integer=integer,
                   fifo_cap=2, seg_elems=seg, n_cta=n_cta, deferred=deferred)
    assert v.ok, f"{coll} {algo} n={n} k={k} count={count} esz={elem_size} cta={n_cta} seg={seg} in_place={in_place} root={root % n} deferred={deferred}: {v.error}"
    if integer:
        assert v.max_abs_err == 0.0


@settings(max_examples=120, **COMMON)
@given(coll=st.sampled_from(["allgather", "reduce_scatter"]), algo=st.sampled_from(ALGOS), n=st.integers(2, 12), k=st.integers(2, 8), count=st.integers(1, 300),
       gap=st.integers(1, 64), n_cta=st.integers(1, 4))
def test_blocks_with_a_stride_never_touch_the_gaps(coll, algo, n, k, count, gap, n_cta):
    v = S.validate(coll, algo, n, count, k=k, stride=count + gap, n_cta=n_cta, seg_elems=32, fifo_cap=2)
    assert v.ok, f"{coll} {algo} n={n} k={k} count={count} stride={count + gap}: {v.error}"


@settings(max_examples=60, **COMMON)
@given(coll=st.sampled_from(COLLS), algo=st.sampled_from(ALGOS), n=st.integers(2, 64), k=st.integers(2, 8), mib=st.integers(1, 2048), n_cta=st.sampled_from([1, 16, 64, 128]))
def test_large_messages_symbolically(coll, algo, n, k, mib, n_cta):
    count = mib * (1 << 20) // 4
    if coll in ("allgather", "reduce_scatter"):
        count //= n
    v = S.validate(coll, algo, n, max(count, 1), k=k, n_cta=n_cta, fifo_cap=2, symbolic=True)
    assert v.ok, f"{coll} {algo} n={n} k={k} {mib} MiB cta={n_cta}: {v.error}"


@settings(max_examples=200, **COMMON)
@given(coll=st.sampled_from(COLLS), algo=st.sampled_from(ALGOS + ["AUTO", "NVLS", "DEFAULT"]), n=st.integers(1, 64), k=st.integers(-3, 70))
def test_resolve_is_total_and_consistent(coll, algo, n, k):
    r = S.resolve(coll, algo, k, n)
    assert r.algo in ALGOS and r.algo != "RD" or algo == "RD"          # a request only ever degrades to RING or to its own family
    if r.radices:
        prod = 1
        for f in r.radices:
            assert 2 <= f <= 8
            prod *= f
        assert prod == (r.core if coll == "allreduce" else n)
    assert 1 <= r.core <= n
