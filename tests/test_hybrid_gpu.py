"""Hybrid decoders on a device: each CUDA operator of libb200hybrid.so alone against its plain restatement (oracle/gulozen.py,
float64), then the engine scenarios of tests/hybrid_scenarios.py in float32 and bfloat16."""
import math

import numpy as np
import pytest
import torch

import hybrid_cases as HC
import hybrid_scenarios as S
from oracle import gulozen as G

pytestmark = pytest.mark.gpu

TOL = {"f32": 2e-5, "bf16": 6e-2}


def _make(dtype):
    return lambda cfg, tensors, **kw: HC.build_engine(cfg, tensors, device="cuda", dtype=dtype, **kw)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("scenario", S.ALL, ids=lambda f: f.__name__)
def test_engine_scenario(scenario, dtype):
    scenario(_make(dtype), TOL[dtype])


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_long_decoding_over_several_pages(dtype):
    S.prefill_then_decode(_make(dtype), TOL[dtype], n=330, tail=210)


# ------------------------------------------------------------------------------------------------ operators alone
def _alone(cfg, tensors, dtype, blocks=8):
    eng = HC.build_engine(cfg, tensors, device="cuda", dtype=dtype, blocks=blocks)
    return eng, eng.model


def _ctx(eng, start, n, pages, slot=2):
    """Step arrays of ONE sequence feeding rows [start, start + n), its pages in the given (shuffled) order."""
    from lmdeploy_b200.turbomind.hybrid import StepArrays
    dev = eng.model.device
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    ptrs = torch.tensor([eng.pool.base + b * eng.pool.block_bytes for b in pages], dtype=torch.int64, device=dev)
    return StepArrays(n=n, batch=1, tok_seq=i32([0] * n), tok_pos=i32(list(range(start, start + n))), cu_q=i32([0, n]), seq_slot=i32([slot]),
                      block_ptrs=ptrs, cu_blocks=i32([0, len(pages)]), state=eng.state, max_pos=start + n - 1)


def _bf(t):
    return t.to(torch.bfloat16).to(torch.float32)


def _close(got, want, tol, what):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
    assert err <= tol, f"{what}: {err:.3g} of the largest value (bound {tol})"


CUTS = [[3, 1, 2, 60, 64, 2, 1, 1], [134]]              # portions down to one and two rows / everything at once


@pytest.mark.parametrize("cuts", CUTS, ids=["portions", "whole"])
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_causal_convolution_carries_its_last_inputs(taps, cuts):
    cfg = HC.config(taps=taps)
    w = HC.random_tensors(cfg)
    eng, model = _alone(cfg, w, "f32")
    n = sum(cuts)
    x = torch.randn(n, cfg["width"], generator=torch.Generator().manual_seed(1))
    want, _ = G.causal_taps(x.double(), w["l1.canon1"].double(), torch.zeros(taps - 1, cfg["width"], dtype=torch.float64))
    got, at = [], 0
    for c in cuts:
        got.append(model.conv_input(1, x[at:at + c].cuda().contiguous(), _ctx(eng, at, c, [0, 1, 2])).cpu())
        at += c
    _close(torch.cat(got), want, 1e-6, f"taps {taps}")


@pytest.mark.parametrize("groups", [1, 3, 8])
def test_grouped_norm_adds_to_the_stream(groups):
    from lmdeploy_b200 import _hybrid_lib as H
    lib = H.load()
    n, W, parts = 5, 48, 3
    g = torch.Generator().manual_seed(groups)
    x, m, wn = torch.randn(n, W, generator=g), 3.0 * torch.randn(n, parts, W, generator=g), torch.randn(W, generator=g)
    want = x.double() + G.grouped_rms_norm(m.double().sum(1), wn.double(), groups, 1e-5)
    xd, md, wd = x.cuda(), m.cuda(), wn.cuda()
    xt = torch.empty(n, W, device="cuda")
    H.check(lib.b200h_residual_group_norm(xd.data_ptr(), md.data_ptr(), 1, parts, wd.data_ptr(), n, W, groups, 1e-5, xt.data_ptr(), H.F32, None))
    _close(xd.cpu(), want, 1e-6, "stream")
    _close(xt.cpu(), want, 1e-6, "its copy for the next projection")
    out = torch.empty(2, W, device="cuda")
    rows = torch.tensor([4, 1], dtype=torch.int32, device="cuda")
    H.check(lib.b200h_group_norm_rows(xd.data_ptr(), rows.data_ptr(), wd.data_ptr(), 2, W, groups, 1e-5, out.data_ptr(), H.F32, None))
    _close(out.cpu(), G.grouped_rms_norm(want[[4, 1]], wn.double(), groups, 1e-5), 1e-6, "norm of chosen rows")


def test_depth_mix_keeps_every_earlier_stream():
    from lmdeploy_b200 import _hybrid_lib as H
    lib = H.load()
    n, W, L = 4, 10, 3
    g = torch.Generator().manual_seed(0)
    hist = torch.zeros(L + 1, n, W)
    hist[0] = torch.randn(n, W, generator=g)
    hd = hist.cuda()
    keep = [hist[0].double()]
    for i in range(L):
        x = torch.randn(n, W, generator=g)
        coef = torch.randn(i + 2, generator=g)
        xd, cd = x.cuda(), coef.cuda()
        H.check(lib.b200h_depth_mix(xd.data_ptr(), hd.data_ptr(), n * W, cd.data_ptr(), i + 2, n * W, None))
        keep.append(x.double())
        _close(xd.cpu(), sum(coef[j].double() * keep[j] for j in range(i + 2)), 1e-6, f"after layer {i}")
    _close(hd.cpu(), torch.stack(keep), 0, "history")


@pytest.mark.parametrize("dtype,tol", [("f32", 2e-5), ("bf16", 3e-2)])
@pytest.mark.parametrize("cuts", [[130, 1, 1, 1, 60, 2, 1], [61, 3, 64, 1, 1, 66]], ids=["prompt_then_single", "portions"])
def test_latent_attention_finds_far_keys_and_counts_the_sink(cuts, dtype, tol):
    """One score is made to stand out: the inputs at positions 0, 63, 64 and 127 (first token, page borders) are scaled so
    that the shared rotated key part, which is not normed, is large there.  Sinks from -20 (never matters) to +6 (takes most
    of the weight) are in the softmax.  Pages are handed over in shuffled order."""
    layer = dict(HC.latent(heads=4, dim=8, rot_dim=12, rot_dims=8, vdim=10, kv_rank=36, q_rank=14), mlp=None)
    cfg = HC.config(layers=[layer])
    w = HC.random_tensors(cfg, seed=2)
    w["l0.mix.sink"] = torch.tensor([-20.0, 0.0, 3.0, 6.0])
    eng, model = _alone(cfg, w, dtype)
    n = sum(cuts)
    h = _bf(torch.randn(n, cfg["width"], generator=torch.Generator().manual_seed(5)))
    for far in (0, 63, 64, 127):
        h[far] *= 12.0
    m = cfg["layers"][0]["mixer"]
    p = {k: v.double() for k, v in G.sub(w, "l0.mix.").items()}
    want = G.latent_attention_mixer(h.double(), p, m, cfg["norm"]["eps"], list(range(n)),
                                    dict(c=torch.zeros(0, m["kv_rank"], dtype=torch.float64), kr=torch.zeros(0, m["rot_dim"], dtype=torch.float64)))
    got, at = [], 0
    for c in cuts:
        y = model.latent_mixer(0, h[at:at + c].to("cuda", model.T).contiguous(), _ctx(eng, at, c, [5, 1, 6, 0]))
        got.append(y.double().cpu() @ p["o"].T)
        at += c
    _close(torch.cat(got), want, tol, "latent attention")


@pytest.mark.parametrize("dtype,tol", [("f32", 2e-5), ("bf16", 3e-2)])
def test_decayed_linear_attention_carries_its_state(dtype, tol):
    """300 rows in portions and single rows with decays from 0.3 to exactly 1: what the first rows wrote is still in the state
    at the end (decay 1 and 0.999) or long gone (0.3)."""
    layer = dict(HC.lightning(heads=4, dim=40, vdim=9, decay=(1.0, 0.999, 0.9, 0.3)), mlp=None)
    cfg = HC.config(layers=[layer])
    w = HC.random_tensors(cfg, seed=3)
    eng, model = _alone(cfg, w, dtype)
    cuts = [2, 1, 100, 1, 1, 64, 131]
    n = sum(cuts)
    h = _bf(torch.randn(n, cfg["width"], generator=torch.Generator().manual_seed(6)))
    m = cfg["layers"][0]["mixer"]
    p = {k: v.double() for k, v in G.sub(w, "l0.mix.").items()}
    want = G.lightning_mixer(h.double(), p, m, cfg["norm"]["eps"], torch.zeros(m["heads"], m["dim"], m["vdim"], dtype=torch.float64))
    got, at = [], 0
    for c in cuts:
        y = model.decay_mixer(0, h[at:at + c].to("cuda", model.T).contiguous(), _ctx(eng, at, c, [0]))
        got.append(y.double().cpu() @ p["o"].T)
        at += c
    _close(torch.cat(got), want, tol, "decayed linear attention")


@pytest.mark.parametrize("dtype,tol", [("f32", 2e-5), ("bf16", 3e-2)])
@pytest.mark.parametrize("experts,top", [(7, 2), (3, 3), (1, 1), (6, 1)])
def test_routed_experts_take_the_largest_scores_unrenormalised(experts, top, dtype, tol):
    layer = dict(HC.lightning(), mlp=HC.moe(experts=experts, top=top, ff=20))
    cfg = HC.config(layers=[layer])
    w = HC.random_tensors(cfg, seed=4)
    eng, model = _alone(cfg, w, dtype)
    n = 33
    x = _bf(torch.randn(n, cfg["width"], generator=torch.Generator().manual_seed(7)))
    p = {k: v.double() for k, v in G.sub(w, "l0.mlp.").items()}
    want = G.routed_experts(x.double(), p, cfg["layers"][0]["mlp"])
    out = model.routed_experts(0, x.cuda(), x.to("cuda", model.T), n)
    _close(out.double().sum(1).cpu(), want, tol, "experts")
    ids, wts = model.last_routing
    scores = torch.softmax(x.double() @ p["router"].T, -1)
    assert (ids.cpu().long() == scores.topk(top, -1).indices).all()
    _close(wts.cpu(), scores.topk(top, -1).values, 1e-5, "router weights")
    assert top == experts or float(wts.sum(-1).min()) < 0.999        # the chosen scores are not renormalised


def test_argmax_takes_the_lowest_index_of_equal_logits():
    eng, model = _alone(HC.config(), HC.random_tensors(HC.config()), "f32")
    lg = torch.randn(5, 1000, generator=torch.Generator().manual_seed(0))
    lg[1, 7] = lg[1, 900] = 50.0
    lg[2, 999] = 60.0
    assert model.argmax(lg.cuda()).cpu().tolist() == [int(lg[0].argmax()), 7, 999, int(lg[3].argmax()), int(lg[4].argmax())]


def test_do_sample_through_the_engine_is_a_function_of_the_seed():
    """Sampling requests run the framework's device sampling stage on the hybrid decoder's logits."""
    from lmdeploy_b200.messages import GenerationConfig
    from lmdeploy_b200.turbomind.engine import batched_generate
    cfg = HC.config()
    w = HC.random_tensors(cfg, seed=9)
    P = HC.prompts_for(cfg, {"a": 9, "b": 20})
    run = lambda seed: [list(s.generated) for s in batched_generate(
        HC.build_engine(cfg, w, device="cuda", dtype="bf16"), [P["a"], P["b"]],
        [GenerationConfig(max_new_tokens=12, ignore_eos=True, do_sample=True, top_k=20, temperature=1.5, random_seed=seed),
         GenerationConfig(max_new_tokens=12, ignore_eos=True)])]
    a, b, c = run(1), run(1), run(2)
    assert a == b and a[0] != c[0] and a[1] == c[1]


def test_decode_graph_replay_equals_eager_launches(monkeypatch):
    """Steps of single decoded tokens replay from a CUDA graph per (batch size, key ranges); the tokens are those of eager launches."""
    from lmdeploy_b200.messages import GenerationConfig
    from lmdeploy_b200.turbomind.engine import batched_generate
    cfg = HC.config()
    w = HC.random_tensors(cfg, seed=11)
    P = HC.prompts_for(cfg, {"a": 9, "b": 70, "c": 3})
    out = {}
    for graphs in ("0", "1"):
        monkeypatch.setenv("B200_ENGINE_GRAPHS", graphs)
        eng = HC.build_engine(cfg, w, device="cuda", dtype="f32")
        seqs = batched_generate(eng, [P[k] for k in "abc"], GenerationConfig(max_new_tokens=80, ignore_eos=True))
        out[graphs] = [list(s.generated) for s in seqs]
        assert bool(eng._hybrid_graphs) == (graphs == "1")
    assert out["0"] == out["1"]


def _write_checkpoint(folder, cfg, tensors):
    """config.json + model.safetensors (bfloat16) as a Gulozen checkpoint is laid out."""
    import json
    from safetensors.torch import save_file
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))


def test_pipeline_serves_a_checkpoint_folder(tmp_path):
    """pipeline(<folder>) picks the hybrid model class by config.json, loads the safetensors and generates what an engine built
    from the same tensors generates; a checkpoint that lacks a tensor is refused by name."""
    import lmdeploy_b200 as lmdeploy
    from lmdeploy_b200.turbomind.engine import batched_generate
    cfg = HC.config()
    w = HC.random_tensors(cfg, seed=12)
    _write_checkpoint(tmp_path, cfg, w)
    P = HC.prompts_for(cfg, {"a": 9, "b": 70})
    gen = lmdeploy.GenerationConfig(max_new_tokens=8, ignore_eos=True)
    ecfg = lmdeploy.TurbomindEngineConfig(max_batch_size=2, session_len=256, cache_max_entry_count=8)
    pipe = lmdeploy.pipeline(str(tmp_path), ecfg)
    assert pipe.engine.hybrid and pipe.engine.spec.arch == "gulozen" and pipe.engine.spec.dtype == "bf16"
    got = [r.token_ids for r in pipe([P["a"], P["b"]], gen)]
    want = [list(s.generated) for s in batched_generate(HC.build_engine(cfg, w, device="cuda", dtype="bf16"), [P["a"], P["b"]], gen)]
    assert got == want and all(len(x) == 8 for x in got)
    bad = tmp_path / "bad"
    bad.mkdir()
    _write_checkpoint(bad, cfg, {k: v for k, v in w.items() if k != "l1.mix.sink"})
    with pytest.raises(KeyError, match="l1.mix.sink"):
        lmdeploy.pipeline(str(bad), ecfg)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 6e-2)])
def test_trace_runner_replays_a_schedule(tmp_path, dtype, tol):
    """bin/trace_run as a process: three requests over a pool of three pages, portions beside single tokens, a request that sits a
    step out, pages and slots given back at "end" and used again; the logits it writes against the oracle."""
    import json
    import os
    import subprocess
    import sys
    cfg = HC.config()
    w = HC.random_tensors(cfg, seed=13)
    model, out = tmp_path / "model", tmp_path / "out"
    model.mkdir()
    _write_checkpoint(model, cfg, w)
    P = HC.prompts_for(cfg, {"a": 100, "b": 6, "c": 64})
    steps = [[("a", 62, [0, 61]), ("b", 2, [1])], [("a", 3, [0, 1, 2]), ("b", 1, [0])], [("b", 3, [2])], [("a", 35, [34]), ("c", 2, [])],
             [("c", 62, [0, 61])], [("b2", 6, [5])]]
    at, lines, asked = {}, [], []
    for k, step in enumerate(steps):
        entries, end = [], []
        for name, count, want in step:
            toks = P[name.rstrip("2")]
            lo = at.get(name, 0)
            at[name] = lo + count
            entries.append({"id": name, "tokens": toks[lo:lo + count], "want": want})
            asked += [(k, name.rstrip("2"), lo + x) for x in want]
            if at[name] == len(toks):
                end.append(name)
        lines.append(json.dumps({"step": k, "entries": entries, "end": end}))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(model), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "192"], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [x for x in r.stdout.split("\n") if x.startswith("done")] == [f"done {k}" for k in range(len(steps))]
    oracle = {name: HC.oracle_logits(cfg, w, toks) for name, toks in P.items()}
    rows = {}
    for k in range(len(steps)):
        want_here = [(n, p) for kk, n, p in asked if kk == k]
        path = out / f"{k}.f32"
        if not want_here:
            assert not path.exists()
            continue
        got = np.fromfile(path, dtype="<f4").reshape(len(want_here), cfg["vocab"])
        for (n, p), row in zip(want_here, got):
            rows.setdefault(n, []).append((row, oracle[n][p]))
    for n, pairs in rows.items():
        err = HC.rel_error(np.stack([a for a, _ in pairs]), np.stack([b for _, b in pairs]))
        assert (err.max() if tol < 1e-3 else np.median(err)) <= tol, (n, err)
