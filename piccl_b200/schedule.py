"""Python view of the native schedule layer: dumps, validation, placement tables."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

from . import _native as N

_COLL_ALIASES = {"bcast": "broadcast"}


def _coll(c) -> int:
    if isinstance(c, int):
        return c
    return N.COLL[_COLL_ALIASES.get(c, c)]


def _algo(a) -> int:
    if isinstance(a, int):
        return a
    return N.ALGO[a.upper()]


def schedule_xml(coll, algo, nranks: int, count: int, k: int = -1, root: int = 0, elem_size: int = 1) -> str:
    """Transfer list in the schedule-XML format read by tools/loggp_sim.
    `count` is the per-rank element count for allgather / reduce_scatter and the total otherwise."""
    l = N.lib()
    need = l.piccl_sched_xml(_coll(coll), _algo(algo), k, nranks, root, count, elem_size, None, 0)
    buf = C.create_string_buffer(need)
    l.piccl_sched_xml(_coll(coll), _algo(algo), k, nranks, root, count, elem_size, buf, need)
    return buf.value.decode()


def schedule_json(coll, algo, nranks: int, count: int, rank: int, k: int = -1, root: int = 0, elem_size: int = 1) -> str:
    l = N.lib()
    need = l.piccl_sched_json(_coll(coll), _algo(algo), k, nranks, root, count, elem_size, rank, None, 0)
    buf = C.create_string_buffer(need)
    l.piccl_sched_json(_coll(coll), _algo(algo), k, nranks, root, count, elem_size, rank, buf, need)
    return buf.value.decode()


@dataclass
class Resolved:
    algo: str
    k: int
    radices: list
    core: int
    note: str


def resolve(coll, algo, k: int, nranks: int) -> Resolved:
    l = N.lib()
    oa, ok, core = C.c_int(), C.c_int(), C.c_int()
    rad = (C.c_int * 16)()
    nr = C.c_int(16)
    note = C.create_string_buffer(256)
    l.piccl_sched_resolve(_coll(coll), _algo(algo), k, nranks, C.byref(oa), C.byref(ok), rad, C.byref(nr), C.byref(core), note, 256)
    names = {v: k_ for k_, v in N.ALGO.items()}
    return Resolved(names[oa.value], ok.value, [rad[i] for i in range(min(nr.value, 16))], core.value, note.value.decode())


@dataclass
class Validation:
    ok: bool
    error: str
    fifo_entries: int
    max_fifo_depth: int
    max_abs_err: float
    bytes_sent_max_rank: int


def validate(coll, algo, nranks: int, count: int, k: int = -1, root: int = 0, elem_size: int = 4, in_place: bool = False,
             op: str = "sum", integer: bool = False, fifo_cap: int = 2, seg_elems: int = 64, n_cta: int = 2,
             stride: int = 0, symbolic: bool = False, deferred: bool = False) -> Validation:
    """Runs all ranks' programs against each other on the CPU (see src/coll/validate.cc).
    `deferred` models the executor variant that publishes its FIFO counters only when it is about to block."""
    l = N.lib()
    ent, depth, err, sent = C.c_longlong(), C.c_int(), C.c_double(), C.c_longlong()
    msg = C.create_string_buffer(512)
    rc = l.piccl_sched_validate(_coll(coll), _algo(algo), k, nranks, root, count, stride, elem_size, int(in_place), N.OP[op], int(integer),
                                fifo_cap, seg_elems, n_cta, int(symbolic) | (2 if deferred else 0), C.byref(ent), C.byref(depth), C.byref(err), C.byref(sent), msg, 512)
    return Validation(rc == 0, msg.value.decode(), ent.value, depth.value, err.value, sent.value)


def permutation_index(r: int, n: int, b: int):
    out = (C.c_int * n)()
    if N.lib().piccl_permutation_index(r, n, b, out) != 0:
        return None
    return list(out)


def held_blocks(r: int, s: int, radices, n: int, permuted: bool):
    rad = (C.c_int * len(radices))(*radices)
    out = (C.c_int * n)()
    m = N.lib().piccl_held_blocks(r, s, rad, len(radices), n, int(permuted), out)
    return [out[i] for i in range(m)]


def counts(coll, algo, nranks: int, count: int, rank: int = 0, k: int = -1, root: int = 0, elem_size: int = 4):
    na, ns, sc = C.c_int(), C.c_int(), C.c_longlong()
    N.lib().piccl_sched_counts(_coll(coll), _algo(algo), k, nranks, root, count, elem_size, rank, C.byref(na), C.byref(ns), C.byref(sc))
    return na.value, ns.value, sc.value
