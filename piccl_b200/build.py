"""In-tree native build: compiles every C++/CUDA source for sm_100a and links

  piccl_b200/lib/piccl.so        collectives library + NCCL-ABI preload shim + fused TP kernels
  piccl_b200/lib/libpiccl_ops.so model kernels (tcgen05 GEMM, layer norm, cross entropy, AdamW, ...)
  piccl_b200/lib/piccl_sched     schedule dump / validation command line tool
  piccl_b200/lib/coll_bench      OSU-style collective benchmark (fork per GPU, no MPI)
  piccl_b200/lib/loggp_bench     PRTT measurements between two GPUs (input of tools/loggp_param)

The reference builds one piccl.so with a single nvcc call and no arch flag
(src/Makefile:7-17); here every translation unit is compiled separately (in
parallel, cached by mtime) with -gencode arch=compute_100a,code=sm_100a.

Run:  python -m piccl_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shlex
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "src"
OUT = ROOT / "piccl_b200" / "lib"
OBJ = ROOT / "build"

CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CXXFLAGS = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function,-fvisibility=default"]
INCLUDES = [f"-I{SRC / 'include'}", f"-I{CUDA_HOME}/include", f"-I{CUDA_HOME}/include/nvtx3", "-I/usr/include"]


def _sources(*patterns: str) -> list[Path]:
    out: list[Path] = []
    for p in patterns:
        out += sorted(SRC.glob(p))
    return out


def targets() -> dict[str, dict]:
    return {
        "piccl.so": {
            "src": _sources("coll/*.cc", "runtime/*.cc", "runtime/*.cu", "kernels/*.cu", "tp/*.cu", "piccl.cc"),
            "link": ["-shared", "-cudart", "static", "-ldl", "-lpthread", "-lrt"],
        },
        "libpiccl_ops.so": {
            "src": _sources("ops/*.cu", "ops/*.cc"),
            "link": ["-shared", "-cudart", "static", "-ldl", "-lpthread", "-lrt"],
        },
        # CTA-pair GEMM: a library of its own, left out of runs on several GPUs (see the header of its source)
        "libpiccl_gemm2.so": {
            "src": _sources("ops2/*.cu"),
            "link": ["-shared", "-cudart", "static", "-ldl", "-lpthread", "-lrt"],
        },
        "piccl_sched": {
            "src": _sources("coll/*.cc", "tools/piccl_sched.cc"),
            "link": [],
        },
        "loggp_bench": {
            "src": [ROOT / "tools" / "loggp_bench" / "loggp_bench.cu"],
            "link": ["-cudart", "static", "-ldl", "-lpthread", "-lrt"],
        },
        "coll_bench": {
            "src": [ROOT / "benchmarks" / "coll_bench.cc"],
            "link": ["-cudart", "static", "-ldl", "-lpthread", "-lrt", "-L/usr/lib/x86_64-linux-gnu", "-lnccl", "-Xcompiler", "-rdynamic"],
        },
    }


def _newer(a: Path, b: Path) -> bool:
    return (not b.exists()) or a.stat().st_mtime > b.stat().st_mtime


def _headers_mtime() -> float:
    m = 0.0
    for h in list(SRC.rglob("*.h")) + list(SRC.rglob("*.cuh")):
        m = max(m, h.stat().st_mtime)
    return m


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(shlex.quote(c) for c in cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(cmd)}\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}")
    if verbose and (r.stdout.strip() or r.stderr.strip()):
        print(r.stdout, r.stderr, flush=True)


def build(force: bool = False, verbose: bool = False, only: list[str] | None = None, ptxas_info: bool = False) -> dict[str, Path]:
    OUT.mkdir(parents=True, exist_ok=True)
    OBJ.mkdir(parents=True, exist_ok=True)
    hdr_m = _headers_mtime()
    jobs: dict[Path, list[str]] = {}
    plan = targets()
    if only:
        plan = {k: v for k, v in plan.items() if k in only}
    objs_of: dict[str, list[Path]] = {}
    for name, t in plan.items():
        objs = []
        for s in t["src"]:
            if not s.exists():
                continue
            o = OBJ / (str(s.relative_to(ROOT)).replace("/", "__") + ".o")
            objs.append(o)
            stale = force or _newer(s, o) or (o.exists() and hdr_m > o.stat().st_mtime)
            if stale and o not in jobs:
                cmd = [NVCC, *ARCH, *CXXFLAGS, *INCLUDES, "-c", str(s), "-o", str(o)]
                if ptxas_info:
                    cmd.insert(1, "-Xptxas=-v")
                jobs[o] = cmd
        objs_of[name] = objs
    if jobs:
        workers = max(1, min(len(jobs), (os.cpu_count() or 4)))
        with cf.ThreadPoolExecutor(workers) as ex:
            futs = {ex.submit(_run, cmd, verbose or ptxas_info): o for o, cmd in jobs.items()}
            for f in cf.as_completed(futs):
                f.result()
    built: dict[str, Path] = {}
    for name, t in plan.items():
        objs = objs_of[name]
        if not objs:
            continue
        dst = OUT / name
        if force or any(_newer(o, dst) for o in objs):
            _run([NVCC, *ARCH, *[str(o) for o in objs], *t["link"], "-o", str(dst)], verbose)
        built[name] = dst
    return built


def lib_path(name: str = "piccl.so") -> Path:
    return OUT / name


if __name__ == "__main__":
    force = "--force" in sys.argv
    verbose = "--verbose" in sys.argv
    info = "--ptxas-info" in sys.argv
    only = [a for a in sys.argv[1:] if not a.startswith("--")] or None
    res = build(force=force, verbose=verbose, only=only, ptxas_info=info)
    for k, v in res.items():
        print(f"built {k}: {v}")
