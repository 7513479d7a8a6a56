"""Shared scaffolding of the hybrid-decoder tests: small Gulozen configurations with random weights, the engine built on
them (on a GPU with the CUDA library, or on the CPU with tests/hybrid_emulator.py standing in for it), a replay of
hand-written schedules through TurboMind.step, and the same tokens through the plain oracle (oracle/gulozen.py, float64)."""
import dataclasses

import numpy as np
import torch

from oracle import gulozen as G

BLOCK = 64


def latent(heads=3, dim=8, rot_dim=12, rot_dims=8, vdim=10, kv_rank=20, q_rank=14, scale=0.3, scaling=True, base=1000.0):
    rot = {"dims": rot_dims, "base": base}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
                      "rot": rot}}


def lightning(heads=2, dim=12, vdim=6, decay=(0.9, 0.5)):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def moe(experts=5, top=3, ff=24):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(layers=None, width=48, vocab=61, groups=3, taps=3, scale=0.7, eps=1e-5):
    """A Gulozen config.json as a dict.  The default stack starts with the recurrent mixer, has a layer without a
    feed-forward, a router that takes one expert, and sizes that are neither equal to each other nor powers of two."""
    if layers is None:
        layers = [dict(lightning(), mlp=moe()), dict(latent(), mlp=moe(experts=4, top=1, ff=16)), dict(latent(scaling=False, rot_dims=12), mlp=None),
                  dict(lightning(heads=3, dim=40, vdim=5, decay=(0.99, 0.7, 1.0)), mlp=moe(experts=3, top=3, ff=8))]
    return {"architecture": "Gulozen", "canon": {"taps": taps}, "embedding": {"scale": scale}, "layers": layers,
            "norm": {"eps": eps, "groups": groups}, "vocab": vocab, "width": width}


def random_tensors(cfg, seed=0):
    """name -> float32 tensor with bf16-representable values (so bf16 and float32 engines and the float64 oracle share them)."""
    from lmdeploy_b200.turbomind.hybrid import HybridModel
    from lmdeploy_b200.turbomind.specs import gulozen_spec
    shapes = HybridModel.tensor_shapes(_Shapes(gulozen_spec(cfg)))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in shapes.items():
        if name.endswith(("norm1", "norm2", ".norm")):
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif name.endswith("canon1"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif name.endswith("dwa"):
            t = torch.softmax(torch.randn(shape, generator=g), 0) * 1.2
        elif name.endswith("sink"):
            t = 2.0 * torch.randn(shape, generator=g)
        elif name.endswith("router"):
            t = torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (1.5 / shape[-1] ** 0.5)
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


class _Shapes:
    """Enough of a HybridModel for tensor_shapes()."""

    def __init__(self, spec):
        self.spec = spec


def build_engine(cfg, tensors, *, device, dtype="f32", blocks=8, max_batch=4, emulate=False, prefill_tokens=None):
    """TurboMind over a HybridModel holding `tensors`.  emulate: the numpy stand-in replaces the CUDA library (CPU only)."""
    from lmdeploy_b200 import _hybrid_lib as H
    from lmdeploy_b200.messages import TurbomindEngineConfig
    from lmdeploy_b200.turbomind.engine import TurboMind
    from lmdeploy_b200.turbomind.hybrid import HybridModel
    from lmdeploy_b200.turbomind.specs import gulozen_spec
    spec = dataclasses.replace(gulozen_spec(cfg), dtype=dtype)
    real = H.load
    if emulate:
        from hybrid_emulator import EmulatedHybridLib
        H.load = lambda: EmulatedHybridLib()
    try:
        model = HybridModel(spec, block_len=BLOCK, max_batch=max_batch, device=device)
    finally:
        H.load = real
    model.load_weights(lambda k: tensors[k])
    ecfg = TurbomindEngineConfig(cache_max_entry_count=blocks, max_batch_size=max_batch,
                                 session_len=blocks * BLOCK + 1, max_prefill_token_num=prefill_tokens or blocks * BLOCK)
    return TurboMind(spec, ecfg, model=model)


def replay(engine, prompts, schedule):
    """schedule: [[(name, count), ...], ...] -- each inner list is one engine step; a request starts at its first mention
    and ends (blocks and slot given back) when its prompt is used up.  'name#k' is prompt `name` run once more.
    Returns {name: float32 [len(prompt), vocab]}: the logits at every position."""
    from lmdeploy_b200.messages import GenerationConfig
    from lmdeploy_b200.turbomind.engine import TurboMindInstance
    inst = TurboMindInstance(engine)
    hold = GenerationConfig(max_new_tokens=0, ignore_eos=True)
    at, live, out = {}, {}, {}
    for step in schedule:
        plan = {}
        for name, count in step:
            toks = prompts[name.split("#")[0]]
            lo = at.get(name, 0)
            hi = at[name] = lo + count
            assert hi <= len(toks), (name, hi)
            if name not in live:
                live[name] = inst.open(engine.new_session_id(), toks[lo:hi], hold)
            else:
                live[name].prompt.extend(toks[lo:hi])
            live[name].logit_positions.extend(range(lo, hi))
            plan[live[name].session_id] = count
        engine.step(plan)
        for name, _ in step:
            seq = live[name]
            rows = out.setdefault(name, {})
            for p in list(seq.position_logits):
                rows[p] = seq.position_logits.pop(p).numpy()
            if at[name] == len(prompts[name.split("#")[0]]):
                engine.scheduler.finish(live.pop(name).session_id)
    return {k: np.stack([v[p] for p in range(len(v))]) for k, v in out.items()}


def oracle_logits(cfg, tensors, tokens):
    """The whole prompt through the plain implementation in float64 -> [n, vocab]."""
    t64 = {k: v.to(torch.float64) for k, v in tensors.items()}
    return G.forward(cfg, t64, list(tokens), G.Sequence(cfg, torch.float64)).numpy()


def prompts_for(cfg, lengths, seed=1):
    r = np.random.RandomState(seed)
    return {name: r.randint(0, cfg["vocab"], n).tolist() for name, n in lengths.items()}


def rel_error(got, want):
    """Per position: rms over the vocabulary of the difference (mean removed), relative to the rms of the wanted logits."""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt((w ** 2).mean())
