"""The allocation-free column sum (src/ops/colsum_noalloc.h) is for callers that cannot allocate
device memory when they call in — their HBM belongs to another allocator, or they cannot take the
device-wide stall of cudaMalloc.  It is reached here the way such a caller reaches it: through the
exported C symbol, passing only input, output and a stream.  Its result must agree with the regular
entry point (which gets a caller-provided workspace) on two calls in a row that share the built-in
workspace, and oversize requests must be refused."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from piccl_b200 import _native as N
    lib = N.ops_lib()
    fn = lib.piccl_ops_colsum_noalloc
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    return fn


def _regular(x, accumulate_into=None):
    from piccl_b200 import ops
    out = accumulate_into.clone() if accumulate_into is not None else torch.empty(x.shape[1], device="cuda", dtype=torch.bfloat16)
    ops.colsum(x, out, accumulate=accumulate_into is not None)
    return out


def test_matches_regular_entry_point_on_two_calls_in_a_row():
    fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(0)
    # two different shapes back to back: the second call reuses the workspace the first one left dirty
    shapes = [(8192, 4096), (1000, 1024), (300, 16384)]            # the last one is as wide as the built-in workspace allows
    xs = [(torch.randn(r, c, generator=g, device="cuda")).to(torch.bfloat16) for r, c in shapes]
    outs = [torch.full((c,), float("nan"), device="cuda", dtype=torch.bfloat16) for _, c in shapes]
    for x, o in zip(xs, outs):
        assert fn(x.data_ptr(), o.data_ptr(), x.shape[0], x.shape[1], 0, stream) == 0
    torch.cuda.synchronize()
    for x, o in zip(xs, outs):
        want = _regular(x)
        ref32 = x.float().sum(0)
        tol = 0.02 * ref32.abs().max().item() + 0.3
        assert torch.allclose(o.float(), want.float(), atol=tol, rtol=2e-2)
        assert torch.allclose(o.float(), ref32, atol=tol, rtol=2e-2)
    # accumulate mode, again right after another call
    base = torch.ones(1024, device="cuda", dtype=torch.bfloat16)
    acc = base.clone()
    assert fn(xs[1].data_ptr(), acc.data_ptr(), 1000, 1024, 1, stream) == 0
    torch.cuda.synchronize()
    assert torch.allclose(acc.float(), _regular(xs[1], accumulate_into=base).float(), atol=0.5, rtol=2e-2)


def test_rejects_what_does_not_fit(capfd):
    fn = _lib()
    x = torch.zeros(8, 8, device="cuda", dtype=torch.bfloat16)
    o = torch.zeros(8, device="cuda", dtype=torch.bfloat16)
    assert fn(x.data_ptr(), o.data_ptr(), 8, 16392, 0, 0) == -2        # wider than the built-in workspace
    assert fn(x.data_ptr(), o.data_ptr(), 8, 12, 0, 0) == -1
    assert fn(x.data_ptr(), o.data_ptr(), 0, 8, 0, 0) == -3
    assert fn(0, o.data_ptr(), 8, 8, 0, 0) == -4
    assert fn(x.data_ptr() + 2, o.data_ptr(), 7, 8, 0, 0) == -7         # a view that starts one element into the buffer
    assert "exceeds the built-in workspace" in capfd.readouterr().err
