"""CTA-pair GEMM (src/ops2/gemm_sm100_2cta.cu, `tcgen05.mma.cta_group::2`) against a PyTorch fp32 reference.
The kernel has not run on a GPU yet, so the test only runs when PICCL_TEST_PAIR_GEMM=1 asks for it; every wait in the kernel
is bounded and a wait that ran out is reported through the status word."""
import os
import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
pytestmark = [pytest.mark.gpu, pytest.mark.skipif(os.environ.get("PICCL_TEST_PAIR_GEMM") != "1", reason="set PICCL_TEST_PAIR_GEMM=1 to run the CTA-pair GEMM")]


@pytest.mark.parametrize("M,N,K,with_bias", [(256, 256, 64, False), (256, 256, 512, True), (512, 768, 1024, False), (8192, 1024, 1024, True), (2048, 4096, 3584, False)])
def test_pair_gemm_matches_fp32_reference(M, N, K, with_bias):
    from piccl_b200.ops import gemm_sm100
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    bias = (torch.randn(N, device="cuda", generator=g) * 0.1).to(torch.bfloat16) if with_bias else None
    out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm_sm100.gemm_nt_pair(a, b, out, bias)
    assert gemm_sm100.pair_status() == 0, "a bounded wait ran out"
    ref = a.float() @ b.float().t()
    if bias is not None:
        ref = ref + bias.float()
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * max(scale, 1.0), (err, scale)
