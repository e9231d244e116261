"""Public training entry point: data-parallel GPT-2 training steps.

    trainer = DataParallelTrainer(GPT2Config.medium())      # one process per GPU
    loss = trainer.step(tokens_cpu, targets_cpu)            # pinned host tensors in, python float out

`step` copies the batch from (pinned) host memory, runs forward, backward with
bucketed gradient averaging overlapped on a second stream, the fused AdamW
update, and reads the loss back.  `step_device` is the same without the two host
transfers.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import ops
from .models.gpt2 import GPT2, GPT2Config
from .parallel.comm import Communicator
from .parallel.ddp import GradAverager


class DataParallelTrainer:
    def __init__(self, cfg: GPT2Config, comm: Optional[Communicator] = None, lr: float = 3e-4, weight_decay: float = 0.1,
                 bucket_bytes: int = 25 * 1024 * 1024, algo: Optional[str] = None, k: int = -1, seed: int = 0, use_graph: Optional[bool] = None):
        self.cfg = cfg
        self.model = GPT2(cfg, device=torch.device("cuda", torch.cuda.current_device()), seed=seed)
        self.comm = comm
        algo = algo or os.environ.get("PICCL_ALLREDUCE_ALGO", "AUTO")
        if k < 0:
            k = int(os.environ.get("PICCL_ALLREDUCE_K", "-1"))
        self.averager = GradAverager(self.model.flat_g, comm, bucket_bytes, algo, k)
        self.lr, self.weight_decay = lr, weight_decay
        self._idx = None
        self._tgt = None
        # CUDA graph of the whole step (forward, backward with overlapped bucket reductions, AdamW): after two eager steps
        # the launches are captured once and replayed, which removes the per-launch host cost (about a thousand launches).
        # Off unless asked for (PICCL_TRAIN_GRAPH=1 or use_graph=True), on one GPU and on several alike, so that step times at
        # different GPU counts compare the same launch mode.
        env_graph = os.environ.get("PICCL_TRAIN_GRAPH")
        default_graph = env_graph == "1"
        self.use_graph = default_graph if use_graph is None else use_graph
        self._graph = None
        self._graph_loss = None
        self._eager_steps = 0
        self._launches_per_step = 0
        self._replayed = 0
        self._loss_host = torch.empty(1, dtype=torch.float32).pin_memory()
        if comm is not None and comm.nranks > 1:
            # identical parameters everywhere: rank 0's initial values (all ranks seed alike; this makes it explicit)
            comm.broadcast(self.model.flat_p, root=0, algo="RING")
            self.model.master.copy_(self.model.flat_p.float())

    def _eager_step(self, idx: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        self.averager.begin_step()
        loss = self.model.forward_backward(idx, targets, on_grads_ready=self.averager.ready)
        self.averager.finish()
        self.model.optimizer_step(lr=self.lr, weight_decay=self.weight_decay)
        return loss

    def _static_inputs(self, shape_i, shape_t):
        if self._idx is None or self._idx.shape != shape_i:
            self._idx = torch.empty(shape_i, dtype=torch.int64, device="cuda")
            self._tgt = torch.empty(shape_t, dtype=torch.int64, device="cuda")
            self._graph = None
            self._eager_steps = 0

    def step_device(self, idx: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One training step on a batch that is already on the device."""
        if not self.use_graph:
            return self._eager_step(idx, targets)
        self._static_inputs(idx.shape, targets.shape)
        if idx.data_ptr() != self._idx.data_ptr():
            self._idx.copy_(idx, non_blocking=True)
            self._tgt.copy_(targets, non_blocking=True)
        if self._graph is None:
            if self._eager_steps < 2:                      # warm-up: buffers, program caches, cuBLAS workspaces
                self._eager_steps += 1
                before = self.kernel_launches()
                loss = self._eager_step(self._idx, self._tgt)
                self._launches_per_step = self.kernel_launches() - before
                return loss
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._graph_loss = self._eager_step(self._idx, self._tgt)
            self._graph = g
            self.model.step_count -= 1                     # the capture itself did not run
        self.model.step_count += 1
        self._graph.replay()
        self._replayed += 1
        return self._graph_loss

    def step(self, idx_host: torch.Tensor, targets_host: torch.Tensor) -> float:
        self._static_inputs(idx_host.shape, targets_host.shape)
        self._idx.copy_(idx_host, non_blocking=True)
        self._tgt.copy_(targets_host, non_blocking=True)
        loss = self.step_device(self._idx, self._tgt)
        self._loss_host.copy_(loss.reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return float(self._loss_host[0])

    def kernel_launches(self) -> int:
        """Launches of this framework's own kernels so far (model kernels + collective executor); a replayed step
        counts the launches that were captured into its graph."""
        n = ops.launch_count()
        if self.comm is not None:
            n += int(self.comm.stats().launches)
        return n + self._replayed * self._launches_per_step
