#!/usr/bin/env python
"""Headline benchmark: data-parallel GPT-2 medium training, tokens/s.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference .so preloaded under stock PyTorch DDP

Config (the end-to-end configuration of the baseline): GPT-2 medium (24 layers, d_model 1024,
16 heads, vocab 50257), sequence 1024, micro-batch 8 per GPU, bf16, random-init weights, token ids
uniform over the vocabulary, 25 MiB gradient buckets all-reduced every step, AdamW update inside
the timed region.  Weak scaling: the per-GPU batch is fixed.

Rank 0 prints one JSON line.  `value` is the aggregate tokens/s over all GPUs with the batch
already on the device, timed with CUDA events, max over ranks; `e2e` is the same through
`piccl_b200.train.DataParallelTrainer.step`, whose timed region includes, every step, the copy of
the batch from pinned host memory and the read-back of the loss.  For N > 1 the line also carries
`dropin`: stock PyTorch DDP on the SAME model code as the reference arm (benchmarks/torch_gpt2.py) with this
    library loaded through LD_PRELOAD and PICCL_ALLREDUCE_ALGO=AUTO, tokens/s and the interposer's counters of
    calls it ran itself / handed to NCCL;
`collectives`: all-reduce latency (us) per message size for every algorithm of this library, for stock NCCL and
    for the reference's own algorithms (fp32; it has no bf16), measured by benchmarks/coll_bench.cc (one process
    per GPU, CUDA events, maximum over ranks, 1000 / 100 iterations below / from 1 MB, data checked).
Both run as child processes of rank 0 once the training job has left the GPUs.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="piccl", choices=["piccl", "reference", "ddp"],
                    help="piccl: this framework's trainer; reference: stock PyTorch DDP under the reference .so; ddp: stock PyTorch DDP under --preload")
    ap.add_argument("--preload", default="", help="with --impl ddp: library to LD_PRELOAD (e.g. piccl_b200/lib/piccl.so; PICCL_*_ALGO from the environment); empty: none")
    ap.add_argument("--model", default="medium", choices=["medium", "tiny"])
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--algo", default=None, help="all-reduce algorithm of the bucket reductions (RING, K_RING, RD, RM, PRD, PRM, DIRECT, AUTO)")
    ap.add_argument("--k", type=int, default=-1)
    ap.add_argument("--no-collectives", action="store_true", help="skip the all-reduce tables for N > 1")
    ap.add_argument("--no-dropin", action="store_true", help="skip the LD_PRELOAD drop-in run for N > 1")
    return ap.parse_args()


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def max_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def timed_region(step_fn, steps: int, warmup: int, world: int):
    """W untimed + K timed steps; barrier + synchronize on both sides; CUDA events; max over ranks (ms per step)."""
    import torch
    import torch.distributed as dist
    for _ in range(warmup):
        step_fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    t0.record()
    last = None
    for _ in range(steps):
        last = step_fn()
    t1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - wall0) * 1e3
    ms = max(t0.elapsed_time(t1), 0.0)
    return max_over_ranks(ms, world) / steps, max_over_ranks(wall, world) / steps, last


def model_config(name: str):
    from piccl_b200.models.gpt2 import GPT2Config
    return GPT2Config.medium() if name == "medium" else GPT2Config.tiny()


def host_batches(cfg, micro_batch: int, n: int, seed: int):
    import torch
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        tok = torch.randint(0, cfg.vocab_size, (micro_batch, cfg.seq_len + 1), generator=g, dtype=torch.int64)
        out.append((tok[:, :-1].contiguous().pin_memory(), tok[:, 1:].contiguous().pin_memory()))
    return out


def _child_env(extra=None):
    """Environment for a child job: nothing of this torchrun's rendezvous, nothing preloaded unless asked for."""
    env = {k: v for k, v in os.environ.items() if not (k.startswith("TORCHELASTIC") or k in (
        "RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "ROLE_RANK", "ROLE_WORLD_SIZE", "GROUP_WORLD_SIZE", "ROLE_NAME",
        "MASTER_PORT", "LD_PRELOAD", "PICCL_BENCH_UNDER_REFERENCE", "PICCL_BENCH_LABEL"))}
    env["MASTER_ADDR"] = "127.0.0.1"
    env.update(extra or {})
    return env


def _free_port():
    import socket
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


def run_dropin(args, world: int):
    """Stock PyTorch DDP (the reference arm's model and optimizer) with this library preloaded, AUTO all-reduce."""
    import subprocess
    from piccl_b200 import build
    so = str(build.lib_path("piccl.so"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           str(ROOT / "bench.py"), "--impl", "ddp", "--preload", so, "--gpus", str(world), "--steps", str(args.steps), "--warmup", str(args.warmup), "--model", args.model,
           "--micro-batch", str(args.micro_batch)]
    algo = args.algo or "AUTO"
    try:
        # PICCL_NVLS_CTA=48: the setting for all-reduces that overlap with compute (the library's default, 128, is for stand-alone bandwidth)
        r = subprocess.run(cmd, env=_child_env({"PICCL_ALLREDUCE_ALGO": algo, "PICCL_NVLS_CTA": os.environ.get("PICCL_NVLS_CTA", "48")}), capture_output=True, text=True, timeout=900)
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    for ln in reversed(r.stdout.strip().splitlines()):
        if ln.startswith("{"):
            try:
                d = json.loads(ln)
            except ValueError:
                continue
            keep = {"value": d.get("value"), "unit": d.get("unit"), "ms_per_step": d.get("ms_per_step"), "e2e": d.get("e2e"), "shim": d.get("shim"),
                    "stack": "torch DistributedDataParallel + fused AdamW on benchmarks/torch_gpt2.py, LD_PRELOAD=piccl.so", "allreduce_algo_env": algo, "nvls_cta_env": os.environ.get("PICCL_NVLS_CTA", "48")}
            return keep
    return {"unavailable": f"rc {r.returncode}: " + (r.stderr.strip().splitlines() or ["no output"])[-1][:200]}


COLL_SIZES = [8, 4096, 65536, 1 << 20, 16 << 20, 25 << 20, 256 << 20, 1 << 30]


def run_collectives(world: int):
    """All-reduce latency per size: every algorithm of this library, stock NCCL and the reference's algorithms (fp32 only),
    same harness binary, only LD_PRELOAD and PICCL_* differ."""
    import subprocess
    from piccl_b200 import build
    cb = build.lib_path("coll_bench")
    ours = str(build.lib_path("piccl.so"))
    if not cb.exists():
        return {"unavailable": "coll_bench not built"}
    ref_missing = ensure_reference()
    ref = str(reference_paths())
    sizes = ",".join(str(b) for b in COLL_SIZES)
    table = {"sizes_bytes": COLL_SIZES, "iters": "1000 below 1 MB, 100 from 1 MB", "unit": "us per call, max over ranks", "failed_checks": {"ours": 0, "nccl": 0, "ref": 0}}

    def bench(dtype, label, preload, env_extra, algos=None):
        cmd = [str(cb), "--gpus", str(world), "--coll", "allreduce", "--dtype", dtype, "--sizes", sizes, "--check", "--label", label]
        if algos:
            cmd += ["--algos", algos]
        env = _child_env(env_extra)
        if preload:
            env["LD_PRELOAD"] = preload
        try:
            r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
        except Exception as e:  # noqa: BLE001
            return {label: f"{type(e).__name__}"}
        rows = {}
        for ln in r.stdout.splitlines():
            f = ln.split(",")
            if len(f) == 11 and f[0] == "allreduce":
                rows.setdefault(f[1], {})[int(f[5])] = round(float(f[7]), 1)
                if f[10] == "FAIL":
                    table["failed_checks"][f[1].split("-")[0] if f[1].split("-")[0] in ("ours", "nccl", "ref") else "ours"] += 1
        if not rows:
            return {label: f"no rows (rc {r.returncode})"}
        return {k: [v.get(b) for b in COLL_SIZES] for k, v in rows.items()}

    algos = "RING,K_RING:2,K_RING:4,PRD,PRM:2,PRM:4,AUTO"
    for dtype in ("float", "bf16"):
        t = {}
        t.update(bench(dtype, "nccl", "", {}))
        t.update(bench(dtype, "ours", ours, {}, algos))
        if dtype == "float":
            if ref_missing:
                t["ref"] = ref_missing
            else:
                for algo, k in (("RING", None), ("K_RING", 2), ("K_RING", 4), ("PRD", None), ("PRM", 2), ("PRM", 4)):
                    e = {"PICCL_ALLREDUCE_ALGO": algo}
                    if k:
                        e["PICCL_ALLREDUCE_K"] = str(k)
                    t.update(bench(dtype, f"ref-{algo}" + (f"-k{k}" if k else ""), ref, e))
        table[dtype] = t
    # bus bandwidth of AUTO against the comparators at the sizes that matter for gradient buckets and large messages
    summary = {}
    for dtype in ("float", "bf16"):
        t = table.get(dtype, {})
        auto, nccl = t.get("ours-AUTO-k-1"), t.get("nccl")
        if isinstance(auto, list) and isinstance(nccl, list):
            summary[dtype] = {str(b): {"auto_busbw_gbs": round(2 * (world - 1) / world * b / a / 1e3, 1), "nccl_busbw_gbs": round(2 * (world - 1) / world * b / c / 1e3, 1)}
                              for b, a, c in zip(COLL_SIZES, auto, nccl) if a and c and b >= (1 << 20)}
    table["busbw_summary"] = summary
    return table


# ------------------------------------------------------------------------------------------------ our arm
def run_piccl(args):
    import torch
    rank, world, local = dist_env()
    if world != args.gpus and world == 1 and args.gpus > 1:
        print(json.dumps({"error": f"--gpus {args.gpus} needs torchrun with {args.gpus} processes"}))
        return 2
    torch.cuda.set_device(local)
    import torch.distributed as dist
    from piccl_b200 import ops
    from piccl_b200.parallel.comm import Communicator
    from piccl_b200.train import DataParallelTrainer
    from piccl_b200.utils.clocks import ClockSampler
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        from piccl_b200.parallel.comm import make_config
        # 48 CTAs for the bucket all-reduces: measured on 8 GPUs 32.4 ms per step against 33.8 ms with the 128 that stand-alone bandwidth wants
        comm = Communicator(config=make_config(nvls_cta=int(os.environ.get("PICCL_NVLS_CTA", "48"))))
    cfg = model_config(args.model)
    trainer = DataParallelTrainer(cfg, comm, algo=args.algo, k=args.k, seed=0)
    batches = host_batches(cfg, args.micro_batch, 4, seed=1234 + rank)
    dev = [(a.cuda(), b.cuda()) for a, b in batches]
    tokens_per_step = world * args.micro_batch * cfg.seq_len

    it = {"i": 0}

    def step_dev():
        i = it["i"] = it["i"] + 1
        a, b = dev[i % len(dev)]
        return trainer.step_device(a, b)

    def step_e2e():
        i = it["i"] = it["i"] + 1
        a, b = batches[i % len(batches)]
        return trainer.step(a, b)

    sampler = ClockSampler(local).start() if rank == 0 else None
    l0 = trainer.kernel_launches()
    ms_dev, _, last = timed_region(step_dev, args.steps, args.warmup, world)
    launches = (trainer.kernel_launches() - l0) // max(1, args.steps + args.warmup) * args.steps
    ms_e2e, wall_e2e, last_loss = timed_region(step_e2e, args.steps, max(1, args.warmup // 2), world)
    clocks = sampler.stop() if sampler else None
    h2d = 2 * args.micro_batch * cfg.seq_len * 8
    comm_stats = None
    if comm is not None:
        st = comm.stats()
        comm_stats = {"allreduce_calls": int(st.calls[1]), "in_switch_calls": int(st.nvls_calls), "kernel_launches": int(st.launches)}
    algo_name = trainer.averager.algo
    launch_mode = "CUDA graph replay" if trainer.use_graph else "eager"
    gemm_counts = None
    if rank == 0:
        from piccl_b200.ops import gemm
        gemm_counts = gemm.counts()
    # the training job leaves the GPUs before rank 0 starts the child jobs of the other sections
    if world > 1:
        dist.barrier()
        comm.close()
        dist.destroy_process_group()
    del trainer, dev
    torch.cuda.empty_cache()
    if rank == 0:
        line = {
            "metric": "DDP GPT-2 medium training throughput" if args.model == "medium" else "DDP GPT-2 tiny training throughput",
            "value": round(tokens_per_step / ms_dev * 1e3, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_dev, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: token ids uniform over the vocabulary, random-init weights", "impl": "piccl_b200",
            "config": {"model": f"gpt2-{args.model}", "layers": cfg.n_layer, "d_model": cfg.d_model, "heads": cfg.n_head, "vocab": cfg.vocab_size,
                       "global_batch": world * args.micro_batch, "micro_batch_per_gpu": args.micro_batch, "seq_len": cfg.seq_len,
                       "parallelism": f"dp{world}", "bucket_mb": 25, "allreduce_algo": algo_name, "optimizer": "AdamW (in timed region)", "launch_mode": launch_mode,
                       "l2": "working set per step (>= 7 GB of weights, activations and gradients) is far larger than the 126 MB L2; no explicit flush",
                       "gemm_calls": gemm_counts, "communicator": comm_stats},
            "e2e": {"value": round(tokens_per_step / ms_e2e * 1e3, 1), "unit": "tokens/s", "ms_per_step": round(ms_e2e, 3), "wall_ms_per_step": round(wall_e2e, 3),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "api": "piccl_b200.train.DataParallelTrainer.step", "last_loss": last_loss},
            "gpu_launches": int(launches), "clocks": clocks,
        }
        if world > 1:
            time.sleep(2.0)                               # the other ranks' processes end and free their memory
            if not args.no_dropin:
                line["dropin"] = run_dropin(args, world)
            if not args.no_collectives:
                line["collectives"] = run_collectives(world)
        print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------------------------------------ reference arm
def reference_paths():
    ref_so = ROOT / "baseline" / "_ref" / "piccl.so"
    return ref_so


def ensure_reference():
    """Builds baseline/_ref/piccl.so from the unmodified reference sources if it is not there."""
    import subprocess
    so = reference_paths()
    if so.exists():
        return None
    try:
        r = subprocess.run([str(ROOT / "baseline" / "build_ref.sh")], capture_output=True, text=True, timeout=300)
    except Exception as e:  # noqa: BLE001
        return f"reference build could not be started: {e}"
    if r.returncode != 0 or not so.exists():
        return "reference build failed: " + (r.stderr.strip().splitlines() or ["no output"])[-1][:160]
    return None


def reexec_under(preload: str):
    """Re-executes this process with `preload` in LD_PRELOAD (nothing if empty): the drop-in configuration, stock PyTorch DDP
    whose NCCL calls the preloaded library intercepts."""
    env = dict(os.environ)
    if preload:
        env["LD_PRELOAD"] = str(Path(preload).resolve())
    env["PICCL_BENCH_UNDER_REFERENCE"] = "1"
    env["PICCL_BENCH_LABEL"] = f"ddp:{preload or 'none'}"
    os.execve(sys.executable, [sys.executable] + sys.argv, env)


def reexec_under_reference():
    """Re-executes this process with the reference .so preloaded.  The reference opens "libnccl.so" in a
    constructor (src/piccl.c:206-211), so a directory whose libnccl.so / libnccl.so.2 point at the NCCL
    that PyTorch ships is put first on the library path; otherwise the loader would pin the system build."""
    import importlib.util
    spec = importlib.util.find_spec("nvidia.nccl")
    shim_dir = ROOT / "baseline" / "_ref" / "lib"
    shim_dir.mkdir(parents=True, exist_ok=True)
    torch_nccl = None
    if spec and spec.submodule_search_locations:
        cand = Path(list(spec.submodule_search_locations)[0]) / "lib" / "libnccl.so.2"
        if cand.exists():
            torch_nccl = cand
    if torch_nccl is None:
        return "PyTorch's bundled libnccl.so.2 not found"
    # all ranks of a node run this at the same time: make the links atomically and tolerate a rank that was faster
    for name in ("libnccl.so", "libnccl.so.2"):
        link = shim_dir / name
        try:
            if link.is_symlink() and os.readlink(link) == str(torch_nccl):
                continue
            tmp = shim_dir / f".{name}.{os.getpid()}"
            if tmp.is_symlink() or tmp.exists():
                tmp.unlink()
            tmp.symlink_to(torch_nccl)
            os.replace(tmp, link)
        except OSError:
            if not link.exists():
                return f"cannot create {link}"
    env = dict(os.environ)
    env["LD_PRELOAD"] = str(reference_paths())
    env["LD_LIBRARY_PATH"] = f"{shim_dir}:/usr/local/cuda/lib64:" + env.get("LD_LIBRARY_PATH", "")
    env["PICCL_BENCH_UNDER_REFERENCE"] = "1"
    os.execve(sys.executable, [sys.executable] + sys.argv, env)


def run_reference(args):
    rank, world, local = dist_env()
    if os.environ.get("PICCL_BENCH_UNDER_REFERENCE") != "1":
        if args.impl == "ddp":
            reexec_under(args.preload)
        why = ensure_reference()
        if why is None:
            why = reexec_under_reference()      # only returns on failure
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return 0
    import torch
    import torch.distributed as dist
    from benchmarks.torch_gpt2 import TorchGPT2
    from piccl_b200.utils.clocks import ClockSampler
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = model_config(args.model)
    torch.manual_seed(0)
    model = TorchGPT2(cfg.vocab_size, cfg.seq_len, cfg.n_layer, cfg.n_head, cfg.d_model).cuda().to(torch.bfloat16)
    net = model
    if world > 1:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], bucket_cap_mb=25, gradient_as_bucket_view=True)
    decay = [p for n_, p in model.named_parameters() if p.dim() >= 2]
    nodecay = [p for n_, p in model.named_parameters() if p.dim() < 2]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": nodecay, "weight_decay": 0.0}], lr=3e-4, betas=(0.9, 0.95), fused=True)
    batches = host_batches(cfg, args.micro_batch, 4, seed=1234 + rank)
    dev = [(a.cuda(), b.cuda()) for a, b in batches]
    tokens_per_step = world * args.micro_batch * cfg.seq_len
    it = {"i": 0}
    loss_host = torch.empty(1, dtype=torch.float32).pin_memory()
    idx_d = torch.empty_like(dev[0][0]); tgt_d = torch.empty_like(dev[0][1])

    def one(a, b):
        opt.zero_grad(set_to_none=True)
        loss = net(a, b)
        loss.backward()
        opt.step()
        return loss

    def step_dev():
        i = it["i"] = it["i"] + 1
        return one(*dev[i % len(dev)])

    def step_e2e():
        i = it["i"] = it["i"] + 1
        a, b = batches[i % len(batches)]
        idx_d.copy_(a, non_blocking=True); tgt_d.copy_(b, non_blocking=True)
        loss = one(idx_d, tgt_d)
        loss_host.copy_(loss.detach().float().reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return float(loss_host[0])

    sampler = ClockSampler(local).start() if rank == 0 else None
    ms_dev, _, _ = timed_region(step_dev, args.steps, args.warmup, world)
    ms_e2e, wall_e2e, last_loss = timed_region(step_e2e, args.steps, max(1, args.warmup // 2), world)
    clocks = sampler.stop() if sampler else None
    shim = None
    if args.impl == "ddp" and os.environ.get("LD_PRELOAD"):
        # calls the preloaded interposer ran itself / handed to NCCL, per collective (all-gather, all-reduce, broadcast, reduce, reduce-scatter)
        try:
            import ctypes
            lib = ctypes.CDLL(os.environ["LD_PRELOAD"])
            nat, pas = (ctypes.c_ulonglong * 5)(), (ctypes.c_ulonglong * 5)()
            lib.piccl_shim_counters(nat, pas)
            shim = {"fused": list(nat), "passed_to_nccl": list(pas), "order": ["allgather", "allreduce", "broadcast", "reduce", "reduce_scatter"]}
        except (OSError, AttributeError):
            shim = None
    if rank == 0:
        print(json.dumps({
            "impl": os.environ.get("PICCL_BENCH_LABEL", "reference"), "shim": shim, "metric": "DDP GPT-2 medium training throughput" if args.model == "medium" else "DDP GPT-2 tiny training throughput",
            "value": round(tokens_per_step / ms_dev * 1e3, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_dev, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: token ids uniform over the vocabulary, random-init weights",
            "config": {"model": f"gpt2-{args.model}", "global_batch": world * args.micro_batch, "seq_len": cfg.seq_len, "parallelism": f"dp{world}", "bucket_mb": 25,
                       "stack": ("stock PyTorch DDP + fused AdamW under LD_PRELOAD given below" if args.impl == "ddp" else
                                 "unmodified reference piccl.so preloaded (algorithms unset: its bf16-capable path is the NCCL passthrough) under stock PyTorch DDP + fused AdamW"),
                       "allreduce_algo_env": os.environ.get("PICCL_ALLREDUCE_ALGO", ""),
                       "preload": os.environ.get("LD_PRELOAD", "")},
            "e2e": {"value": round(tokens_per_step / ms_e2e * 1e3, 1), "unit": "tokens/s", "ms_per_step": round(ms_e2e, 3), "wall_ms_per_step": round(wall_e2e, 3),
                    "h2d_bytes_per_step": 2 * args.micro_batch * cfg.seq_len * 8, "d2h_bytes_per_step": 4, "last_loss": last_loss},
            "gpu_launches": 0, "clocks": clocks}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    a = parse()
    sys.exit(run_reference(a) if a.impl in ("reference", "ddp") else run_piccl(a))
