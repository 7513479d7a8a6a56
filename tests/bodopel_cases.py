"""Scaffolding of the Bodopel tests: small configurations with random weights, the engine built on them (on a GPU with the
CUDA library, or on the CPU with tests/hybrid_emulator.py standing in for it) and the same tokens through the plain oracle
(oracle/bodopel.py, float64).  Schedules are replayed with hybrid_cases.replay."""
import dataclasses

import torch

from hybrid_cases import BLOCK, _Shapes, prompts_for, rel_error, replay  # noqa: F401  (re-exported for the scenarios)
from oracle import bodopel as B


def attention(heads=6, kv_heads=3, dim=8, vdim=10, window=9, scale=0.4, softcap=5.0):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": scale,
                      "softcap": softcap}}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def config(layers=None, width=48, vocab=61, taps=3, scale=3.0, eps=1e-5, loop=(1, 3, 2), max_positions=320):
    """A Bodopel config.json as a dict.  The default stack has a layer before the loop, a looped pair of which one has no
    feed-forward, a layer after it, windows shorter and longer than a page fraction, and sizes that are neither equal to each
    other nor powers of two."""
    if layers is None:
        layers = [dict(attention(), mlp=dense()), dict(attention(heads=4, kv_heads=1, dim=12, vdim=6, window=70, softcap=2.0), mlp=None),
                  dict(attention(heads=2, kv_heads=2, dim=16, vdim=16, window=5, scale=0.2), mlp=dense(24)),
                  dict(attention(heads=3, kv_heads=1, dim=20, vdim=7, window=33, softcap=30.0), mlp=dense(56))]
    cfg = {"architecture": "Bodopel", "canon": {"taps": taps}, "embedding": {"scale": scale}, "layers": layers,
           "max_positions": max_positions, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def spec_of(cfg):
    from lmdeploy_b200.turbomind.specs import bodopel_spec
    return bodopel_spec(cfg)


def random_tensors(cfg, seed=0):
    """name -> float32 tensor with bf16-representable values (so bf16 and float32 engines and the float64 oracle share them)."""
    from lmdeploy_b200.turbomind.hybrid import HybridModel
    shapes = HybridModel.tensor_shapes(_Shapes(spec_of(cfg)))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in shapes.items():
        if name.endswith(("norm1", "norm2", "final.norm")):
            t = 0.3 * torch.randn(shape, generator=g)                       # deviation from one
        elif name.endswith(".norm"):
            t = 1.0 + 0.4 * torch.randn(shape, generator=g)
        elif name.endswith(("canon1", "canon2")):
            t = 0.5 * torch.randn(shape, generator=g)
        elif name.endswith(".r1"):
            t = 2.0 * torch.rand(shape, generator=g)
        elif name.endswith(".r2"):
            t = 0.5 * torch.rand(shape, generator=g)
        elif name.endswith(".talk"):
            t = torch.eye(shape[0]) + 0.4 * torch.randn(shape, generator=g)
        elif name.endswith(".b"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif name in ("pos", "loop.step"):
            t = 0.4 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = 0.3 * torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (1.5 / shape[-1] ** 0.5)
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def build_engine(cfg, tensors, *, device, dtype="f32", blocks=8, max_batch=4, emulate=False, prefill_tokens=None):
    """TurboMind over a HybridModel holding `tensors`.  emulate: the numpy stand-in replaces the CUDA library (CPU only)."""
    from lmdeploy_b200 import _hybrid_lib as H
    from lmdeploy_b200.messages import TurbomindEngineConfig
    from lmdeploy_b200.turbomind.engine import TurboMind
    from lmdeploy_b200.turbomind.hybrid import HybridModel
    spec = dataclasses.replace(spec_of(cfg), dtype=dtype)
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


def oracle_logits(cfg, tensors, tokens, trace=None):
    """The whole prompt through the plain implementation in float64 -> [n, vocab]."""
    t64 = {k: v.to(torch.float64) for k, v in tensors.items()}
    return B.forward(cfg, t64, list(tokens), B.Sequence(cfg, torch.float64), trace).numpy()
