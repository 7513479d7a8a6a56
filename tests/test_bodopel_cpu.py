"""Bodopel decoders without a GPU: the host side (spec parsing, runs of looped layers, state slots, page / slot / row
addressing of turbomind/hybrid.py and the engine) runs the scenarios of tests/bodopel_scenarios.py with the numpy stand-in for
the CUDA library, in float32, against the float64 oracle; and the oracle's own mechanisms are checked on cases worked by hand."""
import math

import pytest
import torch

import bodopel_cases as BC
import bodopel_scenarios as S
from oracle import bodopel as B


def _make(cfg, tensors, **kw):
    return BC.build_engine(cfg, tensors, device="cpu", dtype="f32", emulate=True, **kw)


@pytest.mark.parametrize("scenario", S.ALL, ids=lambda f: f.__name__)
def test_engine_scenario_on_the_emulated_library(scenario):
    scenario(_make, 2e-5)


def test_spec_reads_every_size_from_the_config():
    cfg = BC.config()
    spec = BC.spec_of(cfg)
    assert [l.mixer.kind for l in spec.layers] == ["window_attention"] * 4 and spec.block == "pre_norm"
    assert spec.layers[1].mlp is None and spec.layers[2].mlp.ff == 24 and spec.layers[0].mlp.kind == "dense"
    assert (spec.width, spec.vocab, spec.conv_taps, spec.embedding_scale, spec.max_positions, spec.loop) == (48, 61, 3, 3.0, 320, (1, 3, 2))
    m = spec.layers[1].mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.window, m.scale, m.softcap) == (4, 1, 12, 6, 70, 0.4, 2.0)
    assert spec.runs() == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (3, None)]
    assert BC.spec_of(BC.config(loop=None)).runs() == [(i, None) for i in range(4)]
    with pytest.raises(NotImplementedError):
        BC.spec_of(BC.config(layers=[{"type": "lightning", "mixer": {}, "mlp": None}]))
    with pytest.raises(NotImplementedError):
        BC.spec_of(BC.config(layers=[dict(BC.attention(), mlp={"kind": "moe"})]))
    with pytest.raises(ValueError):
        BC.spec_of(BC.config(layers=[dict(BC.attention(heads=5, kv_heads=2), mlp=None)]))
    with pytest.raises(ValueError):
        BC.spec_of(BC.config(loop=(2, 5, 2)))


def test_runs_own_caches_and_states_layers_own_weights():
    cfg = BC.config()
    eng = _make(cfg, BC.random_tensors(cfg))
    model = eng.model
    W, taps = cfg["width"], cfg["canon"]["taps"]
    assert len(model.cache_off) == 6 and len(set(model.cache_off.values())) == 6
    offs = sorted(list(model.conv_off.values()) + list(model.conv2_off.values()))
    assert len(offs) == 6 + 4 and offs == [k * (taps - 1) * W for k in range(10)] and model.slot_floats == 10 * (taps - 1) * W
    per_run = [64 * (2 * m["kv_heads"] * (m["dim"] + m["vdim"])) for m in (cfg["layers"][i]["mixer"] for i, _ in model.runs)]
    assert model.block_bytes == sum(4 * b // 2 for b in per_run)          # float32 keys and values of every run


def test_positions_past_the_table_are_refused():
    cfg = BC.config(max_positions=70)
    w = BC.random_tensors(cfg)
    eng = _make(cfg, w)
    assert eng.session_len == 71
    P = BC.prompts_for(cfg, {"a": 70})
    BC.replay(eng, P, [[("a", 70)]])
    from lmdeploy_b200.turbomind.scheduler import InputLengthError
    from lmdeploy_b200.turbomind.engine import TurboMindInstance
    with pytest.raises(InputLengthError):
        TurboMindInstance(eng).open(eng.new_session_id(), list(range(60)) + list(range(20)), None)
    held = TurboMindInstance(eng).open(eng.new_session_id(), P["a"], None)
    held.prompt.append(3)                                       # an open request grows past the table: the step itself refuses
    with pytest.raises(ValueError):
        eng.step({held.session_id: 71})


# ------------------------------------------------------------------------------------------------ the oracle on hand-worked cases
def test_oracle_offset_norm_and_taps():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    got = B.offset_norm(x, torch.tensor([0.5, -1.0], dtype=torch.float64), 0.0)
    assert torch.allclose(got, torch.tensor([[3.0 / math.sqrt(12.5) * 1.5, 0.0]], dtype=torch.float64))
    h = torch.tensor([[1.0], [10.0], [100.0]], dtype=torch.float64)
    out, keep = B.causal_taps(h, torch.tensor([[2.0, 3.0, 5.0]], dtype=torch.float64), torch.tensor([[7.0], [0.5]], dtype=torch.float64))
    # taps [2, 3, 5] weigh the inputs two back, one back and the present one
    assert out.reshape(-1).tolist() == [1 + 2 * 7 + 3 * 0.5 + 5 * 1, 10 + 2 * 0.5 + 3 * 1 + 5 * 10, 100 + 2 * 1 + 3 * 10 + 5 * 100]
    assert keep.reshape(-1).tolist() == [10.0, 100.0]


def test_oracle_scores_cap_penalty_and_softmax():
    m = {"scale": 2.0, "softcap": 3.0}
    q = torch.tensor([[1.0, 0.0]], dtype=torch.float64)
    keys = torch.tensor([[[5.0, 1.0]], [[0.5, 2.0]]], dtype=torch.float64)            # positions 6 and 7, query at 7
    r1, r2 = torch.tensor([0.7], dtype=torch.float64), torch.tensor([0.25], dtype=torch.float64)
    got = B.window_scores(q, keys, 7, 6, m, r1, r2)
    s0 = 3.0 * math.tanh(10.0 / 3.0) - 0.7 * math.log(1.25)
    s1 = 3.0 * math.tanh(1.0 / 3.0)
    e0, e1 = math.exp(s0), math.exp(s1)
    assert torch.allclose(got, torch.tensor([[e0 / (e0 + e1), e1 / (e0 + e1)]], dtype=torch.float64))


def test_oracle_layer_runs():
    cfg = {"layers": [0] * 5, "loop": {"start": 1, "stop": 3, "times": 3}}
    assert B.layer_runs(cfg) == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (1, 2), (2, 2), (3, None), (4, None)]
    assert B.layer_runs({"layers": [0] * 2}) == [(0, None), (1, None)]
