"""Worker of tests/test_nvls_gpu.py: the in-switch collectives (algorithm NVLS) with the switch EMULATED on one GPU.
All ranks are virtual ranks of one cooperative launch (LoopbackGroup); a multimem load-reduce becomes a loop over the
ranks' windows and a multicast store a loop of stores, everything else (chunking, half slots, counters, copies, the
handling of unaligned buffers and odd sizes) is the code that runs on real NVLink multicast windows.  Results are
compared with plain PyTorch fp32 arithmetic.  Small slots (PICCL_NVLS_CHUNK_KB) make every CTA wrap around the parts of its
slot many times, and the collectives are interleaved so that a part is reused by a different collective."""
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
os.environ.setdefault("PICCL_NVLS", "1")
os.environ.setdefault("PICCL_NVLS_CHUNK_KB", "8")
os.environ.setdefault("PICCL_NVLS_MIN_KB", "4")
os.environ.setdefault("PICCL_NVLS_CTA", "6")


def rand(count, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.rand(count, generator=g, device="cuda") * 2 - 1).to(dtype)


def tol(dtype, n):
    return {torch.float32: 2e-6 * n, torch.bfloat16: 1.6e-2 * n ** 0.5, torch.float16: 2e-3 * n ** 0.5}[dtype]


def reduce_ref(xs, op):
    st = torch.stack([x.float() for x in xs])
    return {"sum": st.sum(0), "avg": st.mean(0), "max": st.max(0).values, "min": st.min(0).values}[op]


def main():
    from piccl_b200.parallel.comm import LoopbackGroup, make_config
    torch.cuda.set_device(0)
    expected_switch_calls = 0
    for n in (2, 3, 8):
        grp = LoopbackGroup(n, config=make_config(max_cta=4, timeout_ms=4000))
        before = grp.stats().nvls_calls

        def healthy(what):
            torch.cuda.synchronize()
            st = grp.status()
            assert st.aborted == 0, f"{what}: wait gave up: code {st.code} rank {st.rank} cta {st.cta} chunk {st.segment} want {st.want} have {st.have}"

        calls = 0
        for dtype in (torch.float32, torch.bfloat16, torch.float16):
            es = torch.empty(0, dtype=dtype).element_size()
            ops = ("sum", "avg") if dtype == torch.float32 else ("sum", "avg", "max", "min")
            # element counts: one element; an odd size with a tail; several chunks per CTA (6 CTAs, parts of 8 KiB)
            for count in (1, 1001, (200 * 1024) // es + 3):
                for op in ops:
                    xs = [rand(count, dtype, 10 * r + count % 7) for r in range(n)]
                    outs = [torch.full_like(x, float("nan")) for x in xs]
                    grp.run("allreduce", xs, outs, count, op=op, algo="NVLS")
                    healthy(f"allreduce {dtype} {count} {op}")
                    calls += 1
                    want = reduce_ref(xs, op)
                    for r in range(n):
                        assert torch.allclose(outs[r].float(), want, atol=tol(dtype, n), rtol=1e-2), f"allreduce n={n} {dtype} {count} {op} rank {r}: {(outs[r].float() - want).abs().max().item()}"
                        assert torch.equal(outs[r], outs[0]), "ranks differ"
            # block collectives: blocks of a multiple of 16 bytes take the switch; interleaved so that the parts of a slot change hands
            for count in (16 // es, (48 * 1024) // es, (24 * 1024 + 16) // es):
                xs = [rand(count, dtype, 100 + r) for r in range(n)]
                # all-gather
                outs = [torch.full((n * count,), float("nan"), device="cuda", dtype=dtype) for _ in range(n)]
                grp.run("allgather", xs, outs, count, algo="NVLS")
                healthy("allgather")
                calls += 1
                want = torch.cat(xs)
                for r in range(n):
                    assert torch.equal(outs[r], want), f"allgather n={n} {dtype} {count} rank {r}"
                # reduce-scatter
                big = [rand(n * count, dtype, 200 + r) for r in range(n)]
                rs = [torch.full((count,), float("nan"), device="cuda", dtype=dtype) for _ in range(n)]
                grp.run("reduce_scatter", big, rs, count, op="sum", algo="NVLS")
                healthy("reduce_scatter")
                calls += 1
                want = reduce_ref(big, "sum")
                for r in range(n):
                    assert torch.allclose(rs[r].float(), want[r * count:(r + 1) * count], atol=tol(dtype, n), rtol=1e-2), f"reduce_scatter n={n} {dtype} {count} rank {r}"
                # broadcast from the last rank, in place
                root = n - 1
                bs = [x.clone() for x in xs]
                grp.run("broadcast", bs, bs, count, root=root, algo="NVLS")
                healthy("broadcast")
                calls += 1
                for r in range(n):
                    assert torch.equal(bs[r], xs[root]), f"broadcast n={n} {dtype} {count} rank {r}"
                # reduce to rank 1
                outs = [torch.full_like(x, float("nan")) for x in xs]
                op = "max" if dtype != torch.float32 else "sum"
                grp.run("reduce", xs, outs, count, op=op, root=1, algo="NVLS")
                healthy("reduce")
                calls += 1
                assert torch.allclose(outs[1].float(), reduce_ref(xs, op), atol=tol(dtype, n), rtol=1e-2), f"reduce n={n} {dtype} {count}"
                assert torch.isnan(outs[0].float()).all(), "only the root's receive buffer is written"
            # user buffers that start 2 or 4 bytes past a 16-byte boundary, and in-place all-gather / reduce-scatter
            count = (40 * 1024) // es
            bases = [rand(count * n + 1, dtype, 300 + r) for r in range(n)]
            xs = [b[1:1 + count] for b in bases]
            want = reduce_ref(xs, "sum")
            grp.run("allreduce", xs, xs, count, op="sum", algo="NVLS")
            healthy("allreduce unaligned in place")
            calls += 1
            for r in range(n):
                assert torch.allclose(xs[r].float(), want, atol=tol(dtype, n), rtol=1e-2)
            bases = [rand(count * n + 1, dtype, 400 + r) for r in range(n)]
            bufs = [b[1:] for b in bases]
            mine = [bufs[r][r * count:(r + 1) * count].clone() for r in range(n)]
            grp.run("allgather", [bufs[r][r * count:(r + 1) * count] for r in range(n)], bufs, count, algo="NVLS")
            healthy("allgather unaligned in place")
            calls += 1
            for r in range(n):
                assert torch.equal(bufs[r], torch.cat(mine)), f"in-place all-gather rank {r}"
            bases = [rand(count * n + 1, dtype, 500 + r) for r in range(n)]
            bufs = [b[1:] for b in bases]
            want = reduce_ref(bufs, "avg")
            grp.run("reduce_scatter", bufs, [bufs[r][r * count:(r + 1) * count] for r in range(n)], count, op="avg", algo="NVLS")
            healthy("reduce_scatter unaligned in place")
            calls += 1
            for r in range(n):
                assert torch.allclose(bufs[r][r * count:(r + 1) * count].float(), want[r * count:(r + 1) * count], atol=tol(dtype, n), rtol=1e-2), f"in-place reduce-scatter rank {r}"
        # every call above was eligible for the switch
        assert grp.stats().nvls_calls - before == calls, (grp.stats().nvls_calls - before, calls)
        expected_switch_calls += calls
        # what the switch cannot reduce (fp32 max, integers) and blocks that are not a multiple of 16 bytes: the peer-to-peer schedules run
        x32 = [rand(5000, torch.float32, 600 + r) for r in range(n)]
        outs = [torch.empty_like(x) for x in x32]
        grp.run("allreduce", x32, outs, 5000, op="max", algo="NVLS")
        healthy("fp32 max")
        assert torch.equal(outs[0], reduce_ref(x32, "max"))
        xi = [torch.arange(999, device="cuda", dtype=torch.int32) * (r + 1) for r in range(n)]
        outs = [torch.empty(n * 999, device="cuda", dtype=torch.int32) for _ in range(n)]
        grp.run("allgather", xi, outs, 999, algo="NVLS")
        healthy("int32 odd all-gather")
        assert torch.equal(outs[n - 1], torch.cat(xi))
        assert grp.stats().nvls_calls - before == calls
        # AUTO picks the switch for large messages when a window exists and there are at least four ranks
        big = [rand(1 << 20, torch.bfloat16, 700 + r) for r in range(n)]
        outs = [torch.empty_like(x) for x in big]
        grp.run("allreduce", big, outs, 1 << 20, op="sum", algo="AUTO")
        healthy("auto")
        assert grp.stats().nvls_calls - before == calls + (1 if n >= 4 else 0)
        assert torch.allclose(outs[0].float(), reduce_ref(big, "sum"), atol=tol(torch.bfloat16, n), rtol=1e-2)
        grp.close()
    print(f"NVLS_EMULATED_OK {expected_switch_calls} collectives through the emulated switch")


if __name__ == "__main__":
    main()
