"""tcgen05 GEMM vs cuBLAS (torch.mm) on the shapes of GPT-2 medium and of the tensor-parallel
consumers; CUDA-event timing, L2 flushed between iterations.  Prints TFLOP/s and the fraction of the
measured cuBLAS bf16 peak (MEASURED_PEAKS.json, or 1590 TFLOP/s if the file is absent).
`--pair` adds the CTA-pair kernel (src/ops2, `tcgen05.mma.cta_group::2`) on the shapes it supports and checks it
against cuBLAS first; a bounded wait that ran out is reported instead of a time."""
from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from piccl_b200.ops import gemm_sm100  # noqa: E402
from piccl_b200.utils.timing import time_cuda  # noqa: E402


def main():
    peak = 1590.0
    src = "fallback"
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        peak = float(json.loads(p.read_text())["bf16_tflops"]); src = "measured"
    shapes = [(8192, 1024, 1024), (8192, 3072, 1024), (8192, 4096, 1024), (8192, 1024, 4096), (8192, 50304, 1024), (8192, 8192, 3584), (8192, 3584, 8192), (8192, 8192, 8192)]
    pair = "--pair" in sys.argv
    print(f"# M,N,K,ours_ms,ours_tflops,cublas_ms,cublas_tflops,ours_frac_of_{src}_peak" + (",pair_ms,pair_tflops,pair_max_abs_err" if pair else ""))
    for M, N, K in shapes:
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        o = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        o2 = torch.empty_like(o)
        t1 = time_cuda(lambda: gemm_sm100.gemm_nt(a, b, o), iters=10, warmup=3)
        t2 = time_cuda(lambda: torch.mm(a, b.t(), out=o2), iters=10, warmup=3)
        fl = 2.0 * M * N * K / 1e12
        line = f"{M},{N},{K},{t1:.4f},{fl / t1 * 1e3:.1f},{t2:.4f},{fl / t2 * 1e3:.1f},{fl / t1 * 1e3 / peak:.3f}"
        if pair and M % 256 == 0 and N % 256 == 0:
            o3 = torch.zeros_like(o)
            gemm_sm100.gemm_nt_pair(a, b, o3)
            st = gemm_sm100.pair_status()
            if st:
                line += f",wait ran out (role {st}),,"
            else:
                err = (o3.float() - o2.float()).abs().max().item()
                t3 = time_cuda(lambda: gemm_sm100.gemm_nt_pair(a, b, o3), iters=10, warmup=3)
                line += f",{t3:.4f},{fl / t3 * 1e3:.1f},{err:.4f}"
        print(line, flush=True)


if __name__ == "__main__":
    main()
