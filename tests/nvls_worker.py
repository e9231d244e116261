"""Worker of tests/test_nvls_gpu.py: in-switch all-reduce on a communicator of ONE rank.
The multicast object then has a single device, so sums equal the input, but every part of the path runs:
window set-up, both views, multimem.ld_reduce / multimem.st / multimem.red, the barrier counters, chunking.
Prints NVLS_UNAVAILABLE when the driver gives no multicast window, NVLS_OK on success."""
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
os.environ["PICCL_NVLS"] = "1"
os.environ.setdefault("PICCL_LOG", "1")


def main():
    from piccl_b200.parallel.comm import Communicator, make_config
    torch.cuda.set_device(0)
    comm = Communicator(rank=0, nranks=1, device=0, config=make_config(timeout_ms=2000))
    probe = torch.ones(1024, device="cuda")
    comm.all_reduce(probe, algo="NVLS")
    torch.cuda.synchronize()
    if comm.stats().nvls_calls == 0:
        print("NVLS_UNAVAILABLE")
        return
    calls = 1
    g = torch.Generator(device="cuda").manual_seed(1)
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        # 1000: one partial chunk; 1 MiB + 3: a tail that is not a multiple of 16 bytes; 40 Mi elements: several chunks per CTA
        for count in (1, 1000, (1 << 20) + 3, 40 << 20):
            x = (torch.rand(count, generator=g, device="cuda") * 2 - 1).to(dtype)
            out = torch.empty_like(x)
            comm.all_reduce(x, out, algo="NVLS")
            calls += 1
            torch.cuda.synchronize()
            st = comm.status()
            assert st.aborted == 0, f"wait gave up: code {st.code} cta {st.cta} chunk {st.segment} want {st.want} have {st.have}"
            assert torch.equal(out, x), f"{dtype} {count}: {(out.float() - x.float()).abs().max().item()}"
        # in place, unaligned start, avg (scale 1/1)
        base = (torch.rand(70001, generator=g, device="cuda") * 2 - 1).to(dtype)
        y = base[1:]                      # starts 2 or 4 bytes past a 16-byte boundary: element-wise copies
        want = y.clone()
        comm.all_reduce(y, op="avg", algo="NVLS")
        calls += 1
        torch.cuda.synchronize()
        assert torch.equal(y, want), f"{dtype} in place"
    # unsupported type: the request runs the ring schedule instead
    z = torch.arange(5000, device="cuda", dtype=torch.int32)
    comm.all_reduce(z, algo="NVLS")
    torch.cuda.synchronize()
    assert torch.equal(z, torch.arange(5000, device="cuda", dtype=torch.int32))
    assert comm.stats().nvls_calls == calls, (comm.stats().nvls_calls, calls)
    # replay from a CUDA graph: the barrier counters live in device memory
    x = torch.randn(1 << 20, device="cuda")
    out = torch.empty_like(x)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        comm.all_reduce(x, out, algo="NVLS", stream=s)
        s.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            comm.all_reduce(x, out, algo="NVLS", stream=s)
        for i in range(3):
            x.fill_(float(i))
            graph.replay()
            s.synchronize()
            assert torch.equal(out, x)
    assert comm.status().aborted == 0
    comm.close()
    print("NVLS_OK")


if __name__ == "__main__":
    main()
