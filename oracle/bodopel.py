"""Plain, slow restatement of the Bodopel layer equations in torch on the CPU -- TEST INFRASTRUCTURE ONLY.

One function per mechanism, written row by row and head by head (explicit loops over query position and head, every visible
key of a row at once; no paging, no batching, no tiling, no two-pass softmax, no key ranges): the opposite route from the product kernels in
lmdeploy_b200/csrc/hybrid/hybrid_ops.cu, with which it shares no code.  `dt` is the dtype everything runs in (float64 by
default).

Notation: n tokens of one sequence, W model width, weights stored [out, in] and applied as x @ W.T; a "run" is one
execution of a layer (a looped layer has one run per pass, each with a cache and conv history of its own)."""
import math

import torch


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight is the deviation from one: unit_rms(x) * (1 + w)."""
    return unit_rms(x, eps) * (1.0 + w)


def causal_taps(h, w, before):
    """h [n, W]; w [W, taps]; `before` [taps-1, W] = the inputs that precede h (zeros at a sequence's start).
    Returns (h + c, the last taps-1 inputs), c_t = sum_j w[:, j] * h_(t - taps + 1 + j)."""
    taps = w.shape[1]
    full = torch.cat([before, h], 0)                       # index t + taps - 1 is h_t
    out = h.clone()
    for t in range(h.shape[0]):
        for j in range(taps):
            out[t] = out[t] + w[:, j] * full[t + j]
    return out, full[full.shape[0] - (taps - 1):].clone()


def squared_relu_ff(h, p):
    """down(relu(up h)^2)."""
    a = torch.relu(h @ p["up"].T)
    return (a * a) @ p["down"].T


def window_scores(q, keys, i, first, m, r1, r2):
    """Attention weights of one query at position i over `keys` [L, H, dim] (key l sits at position first + l; the caller
    passes exactly the visible ones), per head: capped score minus a logarithmic distance penalty, then softmax.
    q [H, dim].  Returns [H, L]."""
    H = q.shape[0]
    L = keys.shape[0]
    cap = m.get("softcap")
    out = torch.zeros(H, L, dtype=q.dtype)
    dist = torch.tensor([float(i - (first + l)) for l in range(L)], dtype=q.dtype)
    for g in range(H):
        s = (keys[:, g] @ q[g]) * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s - r1[g] * torch.log(1.0 + r2[g] * dist)
        out[g] = torch.softmax(s, 0)
    return out


def attention_mixer(h, p, m, eps, positions, cache):
    """Windowed softmax attention with grouped key/value heads.  h [n, W]; p = the layer's 'mix.*' tensors; m = its
    'mixer' config; cache = dict(k [P, G, dim], v [P, G, vdim]) of the earlier positions, extended in place.
    Query and key are normed over their whole projection (all heads at once) with plain weights; after the softmax the
    heads' weight rows are recombined by the matrix `talk`; head h reads the values of key/value head h // (H / G); the
    concatenated heads are gated by sigmoid(g h) and projected by o."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q = unit_rms(h @ p["q"].T + p["q.b"], eps) * p["q.norm"]
    k = unit_rms(h @ p["k"].T + p["k.b"], eps) * p["k.norm"]
    v = h @ p["v"].T + p["v.b"]
    cache["k"] = torch.cat([cache["k"], k.reshape(n, G, D)], 0)
    cache["v"] = torch.cat([cache["v"], v.reshape(n, G, V)], 0)
    q = q.reshape(n, H, D)
    span = (m.get("mask") or {}).get("size")
    rep = H // G
    y = torch.zeros(n, H, V, dtype=h.dtype)
    for t in range(n):
        i = positions[t]
        first = max(0, i - span + 1) if span else 0
        keys = cache["k"][first:i + 1].repeat_interleave(rep, 1)          # [L, H, dim]: head g's keys are kv head g // rep
        wts = window_scores(q[t], keys, i, first, m, p["r1"], p["r2"])
        mixed = p["talk"] @ wts                                             # [H, L]: row h = sum_g talk[h, g] * wts[g]
        for hh in range(H):
            y[t, hh] = mixed[hh] @ cache["v"][first:i + 1, hh // rep]
    y = y.reshape(n, H * V) * torch.sigmoid(h @ p["g"].T)
    return y @ p["o"].T


def layer_runs(cfg):
    """[(layer index, pass index or None)] in execution order: layers start..stop-1 of `loop` are executed `times` times in
    a row (pass 0, 1, ...) where they stand, the others once."""
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(L)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return ([(i, None) for i in range(a)] + [(i, t) for t in range(times) for i in range(a, b)] + [(i, None) for i in range(b, L)])


class Sequence:
    """What one sequence carries from call to call: per run the conv histories of both sublayers and the key/value cache."""

    def __init__(self, cfg, dt=torch.float64):
        W, taps = cfg["width"], cfg["canon"]["taps"]
        self.length = 0
        self.runs = []
        for i, _ in layer_runs(cfg):
            m = cfg["layers"][i]["mixer"]
            self.runs.append(dict(taps1=torch.zeros(taps - 1, W, dtype=dt), taps2=torch.zeros(taps - 1, W, dtype=dt),
                                  cache=dict(k=torch.zeros(0, m["kv_heads"], m["dim"], dtype=dt),
                                             v=torch.zeros(0, m["kv_heads"], m["vdim"], dtype=dt))))


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, seq, trace=None):
    """Feed `tokens` (the next tokens of `seq`) -> logits [n, vocab].  `tensors`: name -> tensor of seq's dtype.
    trace: a list that receives the stream after every run."""
    eps = cfg["norm"]["eps"]
    n = len(tokens)
    positions = list(range(seq.length, seq.length + n))
    x = tensors["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"] + tensors["pos"][torch.tensor(positions)]
    loop = cfg.get("loop")
    for r, (i, t) in enumerate(layer_runs(cfg)):
        layer, st = cfg["layers"][i], seq.runs[r]
        if t is not None and i == loop["start"]:
            x = x + tensors["loop.step"][t]
        if layer["type"] != "attention":
            raise ValueError(layer["type"])
        h, st["taps1"] = causal_taps(offset_norm(x, tensors[f"l{i}.norm1"], eps), tensors[f"l{i}.canon1"], st["taps1"])
        x = x + attention_mixer(h, sub(tensors, f"l{i}.mix."), layer["mixer"], eps, positions, st["cache"])
        f = layer.get("mlp")
        if f is not None:
            if f.get("kind", "dense") != "dense":
                raise ValueError(f["kind"])
            h, st["taps2"] = causal_taps(offset_norm(x, tensors[f"l{i}.norm2"], eps), tensors[f"l{i}.canon2"], st["taps2"])
            x = x + squared_relu_ff(h, sub(tensors, f"l{i}.mlp."))
        if trace is not None:
            trace.append(x.clone())
    seq.length += n
    return offset_norm(x, tensors["final.norm"], eps) @ tensors["head"].T
