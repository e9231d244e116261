"""ctypes bindings of the native libraries (built in-tree by piccl_b200.build)."""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent / "lib"
_lock = threading.Lock()
_libs: dict[str, C.CDLL] = {}

# numeric values shared with src/include/piccl.h
COLL = {"allgather": 0, "allreduce": 1, "broadcast": 2, "reduce": 3, "reduce_scatter": 4}
ALGO = {"DEFAULT": 0, "RING": 1, "K_RING": 2, "RD": 3, "RM": 4, "PRD": 5, "PRM": 6, "AUTO": 7, "DIRECT": 8, "NVLS": 9}
OP = {"sum": 0, "prod": 1, "max": 2, "min": 3, "avg": 4}
# ncclDataType_t numbering
DTYPE = {"int8": 0, "uint8": 1, "int32": 2, "uint32": 3, "int64": 4, "uint64": 5, "float16": 6, "float32": 7, "float64": 8, "bfloat16": 9}


class Config(C.Structure):
    _fields_ = [("max_cta", C.c_int), ("nslot", C.c_int), ("slot_bytes", C.c_longlong), ("scratch_bytes", C.c_longlong),
                ("block_size", C.c_int), ("timeout_ms", C.c_int), ("tp_bytes", C.c_longlong), ("nvls_cta", C.c_int)]


class Handle(C.Structure):
    _fields_ = [("bytes", C.c_ubyte * 128)]


class Status(C.Structure):
    _fields_ = [("aborted", C.c_int), ("code", C.c_int), ("rank", C.c_int), ("cta", C.c_int), ("action", C.c_int),
                ("peer", C.c_int), ("segment", C.c_int), ("want", C.c_ulonglong), ("have", C.c_ulonglong)]


class Stats(C.Structure):
    _fields_ = [("calls", C.c_ulonglong * 5), ("bytes", C.c_ulonglong * 5), ("launches", C.c_ulonglong),
                ("program_cache_hits", C.c_ulonglong), ("program_cache_misses", C.c_ulonglong),
                ("fallbacks", C.c_ulonglong), ("timeouts", C.c_ulonglong), ("persistent_calls", C.c_ulonglong), ("nvls_calls", C.c_ulonglong)]


def _ensure_built(name: str) -> Path:
    path = _LIB_DIR / name
    if not path.exists() or os.environ.get("PICCL_REBUILD") == "1":
        from . import build as _build
        _build.build(only=[name])
    if not path.exists():
        raise RuntimeError(f"native library {name} is missing and could not be built (run python -m piccl_b200.build)")
    return path


def _declare(lib: C.CDLL) -> None:
    vp, i, ll, sz = C.c_void_p, C.c_int, C.c_longlong, C.c_size_t
    lib.piccl_last_error.restype = C.c_char_p
    lib.piccl_comm_create.argtypes = [i, i, i, C.POINTER(Config), C.POINTER(vp)]
    lib.piccl_comm_local_handle.argtypes = [vp, C.POINTER(Handle)]
    lib.piccl_comm_connect.argtypes = [vp, C.POINTER(Handle)]
    lib.piccl_comm_destroy.argtypes = [vp]
    lib.piccl_comm_abort.argtypes = [vp]
    lib.piccl_comm_status.argtypes = [vp, C.POINTER(Status)]
    lib.piccl_get_stats.argtypes = [vp, C.POINTER(Stats)]
    lib.piccl_allreduce.argtypes = [vp, vp, vp, sz, i, i, i, i, vp]
    lib.piccl_allgather.argtypes = [vp, vp, vp, sz, i, i, i, vp]
    lib.piccl_reduce_scatter.argtypes = [vp, vp, vp, sz, i, i, i, i, vp]
    lib.piccl_reduce.argtypes = [vp, vp, vp, sz, i, i, i, i, i, vp]
    lib.piccl_broadcast.argtypes = [vp, vp, vp, sz, i, i, i, i, vp]
    lib.piccl_group_collective.argtypes = [C.POINTER(vp), i, i, C.POINTER(vp), C.POINTER(vp), sz, i, i, i, i, i, vp]
    lib.piccl_test_unmatched_wait.argtypes = [vp, i, vp]
    lib.piccl_algo_from_string.argtypes = [C.c_char_p]
    lib.piccl_sched_xml.argtypes = [i, i, i, i, i, ll, i, C.c_char_p, ll]
    lib.piccl_sched_xml.restype = ll
    lib.piccl_sched_json.argtypes = [i, i, i, i, i, ll, i, i, C.c_char_p, ll]
    lib.piccl_sched_json.restype = ll
    lib.piccl_sched_resolve.argtypes = [i, i, i, i, C.POINTER(i), C.POINTER(i), C.POINTER(i), C.POINTER(i), C.POINTER(i), C.c_char_p, i]
    lib.piccl_sched_validate.argtypes = [i, i, i, i, i, ll, ll, i, i, i, i, i, ll, i, i, C.POINTER(ll), C.POINTER(i),
                                         C.POINTER(C.c_double), C.POINTER(ll), C.c_char_p, i]
    lib.piccl_permutation_index.argtypes = [i, i, i, C.POINTER(i)]
    lib.piccl_held_blocks.argtypes = [i, i, C.POINTER(i), i, i, i, C.POINTER(i)]
    lib.piccl_sched_counts.argtypes = [i, i, i, i, i, ll, i, i, C.POINTER(i), C.POINTER(i), C.POINTER(ll)]


def lib() -> C.CDLL:
    """The collectives library (piccl.so)."""
    with _lock:
        if "piccl" not in _libs:
            path = _ensure_built("piccl.so")
            l = C.CDLL(str(path), mode=C.RTLD_LOCAL)
            _declare(l)
            _libs["piccl"] = l
        return _libs["piccl"]


def ops_lib() -> C.CDLL:
    """The model-kernel library (libpiccl_ops.so)."""
    with _lock:
        if "ops" not in _libs:
            path = _ensure_built("libpiccl_ops.so")
            _libs["ops"] = C.CDLL(str(path), mode=C.RTLD_LOCAL)
        return _libs["ops"]


def gemm2_lib() -> C.CDLL:
    """The CTA-pair GEMM (libpiccl_gemm2.so); raises if the library or its source is not present."""
    with _lock:
        if "gemm2" not in _libs:
            path = _ensure_built("libpiccl_gemm2.so")
            _libs["gemm2"] = C.CDLL(str(path), mode=C.RTLD_LOCAL)
        return _libs["gemm2"]


def last_error() -> str:
    return (lib().piccl_last_error() or b"").decode()


class PicclError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"{what} failed with code {code}: {last_error()}")
        self.code = code


def check(code: int, what: str) -> None:
    if code != 0:
        raise PicclError(code, what)
