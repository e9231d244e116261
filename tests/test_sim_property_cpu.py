"""Property tests of the LogGP simulator (tools/loggp_sim/sim.py): random acyclic schedules on a two-level topology always
finish (in the classical and in the reference-compatible accounting), never faster than their longest dependency chain allows,
deterministically; a single chain of dependent transfers costs exactly the sum of its uncontended message costs.  Malformed inputs are refused with
a message instead of a traceback from deep inside."""
import random
import sys
from pathlib import Path

import pytest
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from tools.loggp_sim import sim as S  # noqa: E402

COMMON = dict(deadline=None, derandomize=True, database=None, suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])


def _world(tmp_path):
    (tmp_path / "intra.csv").write_text("s,L,o_s,o_r,g,G\n1,10,5,6,8,1\n1000000,10,5,6,8,1\n")
    (tmp_path / "inter.csv").write_text("s,L,o_s,o_r,g,G\n1,100,5,6,80,10\n1000000,100,5,6,80,10\n")
    body = ""
    for g in range(2):
        nodes = "".join(f'<node id="{4 * g + i}"/>' for i in range(4))
        body += f'<group level="0" id="{g}" ports="1" param_file="{tmp_path / "intra.csv"}">{nodes}</group>'
    topo = tmp_path / "topo.xml"
    topo.write_text(f'<topo num_nodes="8" num_levels="2"><group level="1" id="0" param_file="{tmp_path / "inter.csv"}">{body}</group></topo>')
    return topo


def _write(tmp_path, transfers, name="s.xml"):
    rows = "\n".join(f'  <transfer id="{i}" size="{sz}" src="{a}" dst="{b}" deps="{",".join(map(str, d)) if d else "-1"}"/>' for i, (sz, a, b, d) in enumerate(transfers))
    p = tmp_path / name
    p.write_text(f'<collective name="t" nodes="8" buffer_size="1">\n  # (round 0)\n{rows}\n</collective>\n')
    return p


def _random_dag(seed, n_transfers):
    rnd = random.Random(seed)
    out = []
    for i in range(n_transfers):
        a = rnd.randrange(8)
        b = rnd.choice([x for x in range(8) if x != a])
        deps = sorted(rnd.sample(range(i), k=min(i, rnd.choice([0, 0, 1, 1, 2]))))
        out.append((rnd.choice([1, 2, 64, 1024, 5000]), a, b, deps))
    return out


@settings(max_examples=60, **COMMON)
@given(seed=st.integers(0, 10_000), n=st.integers(1, 24), radix=st.sampled_from([1, 2, 4]))
def test_random_schedules_finish_and_respect_the_model(tmp_path, seed, n, radix):
    topo = _world(tmp_path)
    tr = _random_dag(seed, n)
    t_clean = S.simulate(_write(tmp_path, tr), topo, radix=radix)
    t_compat = S.simulate(_write(tmp_path, tr), topo, radix=radix, compat=True)
    assert t_clean > 0 and t_compat > 0          # both accountings finish; they are different models, neither bounds the other
    # lower bound: the longest chain of dependent transfers, each at its uncontended intra-group cost o_s + G(s-1) + L + o_r
    best = [0.0] * n
    for i, (sz, a, b, deps) in enumerate(tr):
        best[i] = max([best[d] for d in deps], default=0.0) + 5 + (sz - 1) * 1 + 10 + 6
    assert t_clean >= max(best) - 1e-6
    # (no monotonicity claims: with first-come-first-served ports a longer message or a missing port can reorder the contention
    # and shorten the schedule, the classic list-scheduling anomaly)
    assert S.simulate(_write(tmp_path, tr, "again.xml"), topo, radix=radix) == t_clean            # deterministic
    # without contention (every transfer on its own pair of nodes is impossible here, so: a single chain) the bound is met exactly
    chain = [(sz, i % 4, (i + 1) % 4, [i - 1] if i else []) for i, (sz, _, _, _) in enumerate(tr)]
    exact = sum(5 + (sz - 1) * 1 + 10 + 6 for sz, _, _, _ in chain)
    assert S.simulate(_write(tmp_path, chain, "chain.xml"), topo, radix=radix) == pytest.approx(exact)


def test_malformed_inputs_are_refused(tmp_path):
    topo = _world(tmp_path)
    cyc = tmp_path / "cyc.xml"
    cyc.write_text('<collective name="t" nodes="8" buffer_size="1"><transfer id="0" size="4" src="0" dst="1" deps="1"/><transfer id="1" size="4" src="1" dst="2" deps="0"/></collective>')
    with pytest.raises((ValueError, RuntimeError)):
        S.simulate(cyc, topo)
    for body, what in [('<transfer id="0" size="4.0" src="0" dst="1" deps="-1"/>', "not an integer"),
                       ('<transfer id="0" size="4" src="0" dst="1" deps="7"/>', "unknown transfer"),
                       ('<transfer id="0" size="4" src="0" dst="1" deps="-1"/><transfer id="0" size="4" src="1" dst="2" deps="-1"/>', "duplicate")]:
        p = tmp_path / "bad.xml"
        p.write_text(f'<collective name="t" nodes="8" buffer_size="1">{body}</collective>')
        with pytest.raises(ValueError, match=what):
            S.simulate(p, topo)
    stranger = tmp_path / "stranger.xml"
    stranger.write_text('<collective name="t" nodes="8" buffer_size="1"><transfer id="0" size="4" src="0" dst="42" deps="-1"/></collective>')
    with pytest.raises((ValueError, KeyError)):
        S.simulate(stranger, topo)
