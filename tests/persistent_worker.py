"""Runs small all-reduces through the persistent launcher (PICCL_LAUNCH=persistent must be in the environment
before the library is loaded) on virtual ranks of one GPU, with pauses longer than the server's idle limit in
between, so that the server leaves and is started again several times."""
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from piccl_b200.parallel.comm import LoopbackGroup, make_config  # noqa: E402

n = 4
g = LoopbackGroup(n, config=make_config(max_cta=4, nslot=2, slot_bytes=4096, scratch_bytes=1 << 16, timeout_ms=5000))
served_before = g.stats(0).persistent_calls
for round_ in range(3):
    for dtype, count in [(torch.float32, 1), (torch.bfloat16, 777), (torch.float32, 2000)]:
        gen = torch.Generator(device="cuda").manual_seed(round_ * 10 + count)
        xs = [(torch.rand(count, generator=gen, device="cuda") * 2 - 1).to(dtype) for _ in range(n)]
        outs = [torch.empty_like(x) for x in xs]
        for _ in range(5):
            g.run("allreduce", xs, outs, count, algo="PRD")
        y = outs[0].float() * 2                      # ordinary work queued behind the collective on the same stream
        torch.cuda.synchronize()
        assert g.status().aborted == 0
        ref = torch.stack([x.float() for x in xs]).sum(0)
        tol = 1e-4 if dtype == torch.float32 else 5e-2
        for r in range(n):
            assert torch.allclose(outs[r].float(), ref, atol=tol, rtol=tol), (round_, dtype, count, r)
        assert torch.allclose(y, ref * 2, atol=2 * tol, rtol=tol)
    time.sleep(0.05)                                 # far beyond the idle limit: the server has left
served = g.stats(0).persistent_calls - served_before
assert served == 45, served
g.close()
print("PERSISTENT_OK", served)
