"""piccl_b200 — a Blackwell (sm_100a) native collectives framework with the
capabilities and public interface of PICCL.

Layout
  lib/       built native artefacts (piccl.so: collectives + NCCL-ABI preload shim + fused
             tensor-parallel kernels; libpiccl_ops.so: model kernels)
  parallel/  communicators, collectives, bucketed data parallelism, tensor-parallel ops
  ops/       Python front ends of the model kernels (autograd functions)
  models/    GPT-2 written against those ops
  utils/     timing, clocks sampling, environment helpers
"""
from .version import __version__  # noqa: F401
