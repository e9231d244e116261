"""tcgen05 GEMM against a plain PyTorch fp32 reference (A @ B^T + bias, optional GELU)."""
import ctypes as C

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _bf(*shape, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def _status():
    from piccl_b200 import _native as N
    return N.ops_lib().piccl_ops_gemm_status()


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 64), (256, 256, 256), (128, 384, 128), (1024, 1024, 1024), (384, 3072, 1024), (8192, 1024, 4096), (512, 50304, 1024)])
def test_gemm_matches_fp32_reference(M, N, K):
    from piccl_b200.ops import gemm_sm100
    assert gemm_sm100.available(), "the tcgen05 GEMM must be built and loadable on a B200"
    a, b = _bf(M, K, seed=1), _bf(N, K, seed=2, scale=0.05)
    out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm_sm100.gemm_nt(a, b, out)
    torch.cuda.synchronize()
    assert _status() == 0
    ref = a.float() @ b.float().t()
    err = (out.float() - ref).abs().max().item()
    assert torch.allclose(out.float(), ref, atol=0.02 * ref.abs().max().item() + 1e-2, rtol=2e-2), f"max abs err {err}"


def test_gemm_bias_and_gelu_epilogue():
    from piccl_b200 import _native as N
    from piccl_b200.ops import gemm_sm100
    M, Nn, K = 512, 1024, 256
    a, b, bias = _bf(M, K, seed=1), _bf(Nn, K, seed=2, scale=0.1), _bf(Nn, seed=3)
    out = torch.empty(M, Nn, device="cuda", dtype=torch.bfloat16)
    gemm_sm100.gemm_nt(a, b, out, bias=bias)
    ref = a.float() @ b.float().t() + bias.float()
    assert torch.allclose(out.float(), ref, atol=5e-2, rtol=2e-2)
    pre = torch.empty_like(out)
    rc = N.ops_lib().piccl_ops_gemm_bf16_nt_ex(C.c_void_p(a.data_ptr()), C.c_void_p(b.data_ptr()), C.c_void_p(out.data_ptr()), C.c_void_p(pre.data_ptr()),
                                               C.c_void_p(bias.data_ptr()), M, Nn, K, 1, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert _status() == 0
    assert torch.allclose(pre.float(), ref, atol=5e-2, rtol=2e-2)
    assert torch.allclose(out.float(), F.gelu(pre.float(), approximate="tanh"), atol=2e-2, rtol=2e-2)


def test_gemm_back_to_back_and_unsupported_shapes():
    from piccl_b200 import _native as N
    from piccl_b200.ops import gemm_sm100
    a, b = _bf(256, 512, seed=4), _bf(256, 512, seed=5)
    outs = []
    for _ in range(5):
        o = torch.empty(256, 256, device="cuda", dtype=torch.bfloat16)
        gemm_sm100.gemm_nt(a, b, o)
        outs.append(o)
    torch.cuda.synchronize()
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    # shapes the kernel does not cover are refused with an error code, not computed wrongly
    rc = N.ops_lib().piccl_ops_gemm_bf16_nt(C.c_void_p(a.data_ptr()), C.c_void_p(b.data_ptr()), C.c_void_p(outs[0].data_ptr()), C.c_void_p(0), 100, 256, 512, 0, C.c_void_p(0))
    assert rc != 0
