"""Hybrid decoders without a GPU: the host side (spec parsing, state slots, planned steps, page / slot / row addressing of
turbomind/hybrid.py and the engine) runs the scenarios of tests/hybrid_scenarios.py with the numpy stand-in for the CUDA
library, in float32, against the float64 oracle."""
import math

import pytest

import hybrid_cases as HC
import hybrid_scenarios as S
from lmdeploy_b200.turbomind.scheduler import Scheduler, Sequence
from lmdeploy_b200.turbomind.specs import RotarySpec, gulozen_spec


def _make(cfg, tensors, **kw):
    return HC.build_engine(cfg, tensors, device="cpu", dtype="f32", emulate=True, **kw)


@pytest.mark.parametrize("scenario", S.ALL, ids=lambda f: f.__name__)
def test_engine_scenario_on_the_emulated_library(scenario):
    scenario(_make, 2e-5)


def test_spec_reads_every_size_from_the_config():
    cfg = HC.config()
    spec = gulozen_spec(cfg)
    assert [l.mixer.kind for l in spec.layers] == ["lightning", "latent_attention", "latent_attention", "lightning"]
    assert spec.layers[2].mlp is None and spec.layers[1].mlp.top == 1 and spec.layers[0].mlp.experts == 5
    assert (spec.width, spec.vocab, spec.norm_groups, spec.conv_taps, spec.embedding_scale) == (48, 61, 3, 3, 0.7)
    m = spec.layers[1].mixer
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank, m.scale, m.rot.dims) == (3, 8, 12, 10, 20, 14, 0.3, 8)
    assert spec.layers[2].mixer.rot.scaling is None and spec.layers[3].mixer.decay == (0.99, 0.7, 1.0)
    with pytest.raises(NotImplementedError):
        gulozen_spec(HC.config(layers=[{"type": "sliding", "mixer": {}, "mlp": None}]))
    with pytest.raises(ValueError):
        gulozen_spec(HC.config(layers=[dict(HC.lightning(heads=3), mlp=None)]))          # two decays for three heads


def test_rotary_frequencies_follow_the_ramp():
    """Pairs that turn fast keep their frequency, slow ones are divided by the factor, the ramp in between is linear."""
    r = RotarySpec(dims=16, base=100.0, scaling=(4.0, 64.0, 8.0, 1.0))
    f, mag = r.frequencies()
    plain = [100.0 ** (-2.0 * i / 16) for i in range(8)]
    where = lambda turns: 16 * math.log(64.0 / (2 * math.pi * turns)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(where(8.0)), 0), min(math.ceil(where(1.0)), 15)
    assert (lo, hi) == (0, 5)
    for i in range(8):
        ramp = min(max((i - lo) / (hi - lo), 0.0), 1.0)
        assert f[i] == pytest.approx(plain[i] * (1 - ramp) + plain[i] / 4.0 * ramp, rel=1e-12)
    assert f[0] == plain[0] and f[7] == pytest.approx(plain[7] / 4.0) and mag == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert RotarySpec(dims=16, base=100.0).frequencies() == (plain, 1.0)


def _seq(sid, n):
    return Sequence(session_id=sid, prompt=list(range(n)), max_new_tokens=4, stop_token_ids=[], ignore_eos=True, eos_id=None)


def test_state_slots_limit_admission_and_return_on_retirement_and_preemption():
    sch = Scheduler(max_batch=4, block_len=64, num_blocks=4, session_len=512, prefill_chunk=64, token_budget=256, state_slots=2)
    a, b, c = _seq(1, 10), _seq(2, 10), _seq(3, 10)
    for s in (a, b, c):
        sch.add(s)
    batch = sch.schedule()
    assert batch == [a, b] and {a.slot, b.slot} == {0, 1} and c.slot == -1          # two slots: the third request waits
    sch.update(batch, [5, 5])
    a.finished = True
    freed = a.slot
    batch = sch.schedule()
    assert batch == [b, c] and c.slot == freed and a.slot == -1                      # the retired request's slot is handed out again
    sch._preempt(c)
    assert c.slot == -1 and c.cached == 0 and sorted(sch.slots) == [freed]           # a preempted sequence restarts from a fresh slot
    with pytest.raises(ValueError):
        Scheduler(max_batch=2, block_len=64, num_blocks=2, session_len=128, prefix_caching=True, state_slots=2)


def test_planned_steps_admit_skip_and_refuse():
    sch = Scheduler(max_batch=2, block_len=64, num_blocks=2, session_len=512, state_slots=2)
    a, b, c = _seq(1, 100), _seq(2, 30), _seq(3, 5)
    for s in (a, b, c):
        s.hold = True
        sch.add(s)
    assert sch.schedule_planned({1: 64}) == [a] and a.step_tokens == 64 and len(a.blocks) == 1
    sch.update([a], [0])
    assert sch.schedule_planned({2: 30}) == [b] and a in sch.active                 # a sits the step out and keeps its page
    sch.update([b], [0])
    with pytest.raises(MemoryError):
        sch.schedule_planned({1: 36})                                               # a's second page: both pages are taken
    with pytest.raises(MemoryError):
        sch.schedule_planned({3: 5})                                                # no batch / state slot left
    with pytest.raises(ValueError):
        sch.schedule_planned({2: 1})                                                # b has no token left to feed
    sch.finish(2)
    assert sch.alloc.num_free == 1 and len(sch.slots) == 1 and not b.blocks
    with pytest.raises(MemoryError):
        sch.schedule_planned({1: 36, 3: 5})                                         # a takes the freed page, none is left for c
    assert c.slot == -1 and c not in sch.active                                     # a refused request was not admitted
    assert sch.schedule_planned({1: 36}) == [a]
    sch.update([a], [0])
    assert not a.finished                                                           # open-ended requests end only from outside
    sch.finish(1)
    assert sch.schedule_planned({3: 5}) == [c] and c.slot >= 0
    sch.update([c], [0])
    sch.finish(3)
    assert sch.alloc.num_free == 2 and sorted(sch.slots) == [0, 1] and not sch.has_work
