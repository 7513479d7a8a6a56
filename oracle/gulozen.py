"""Plain, slow restatement of the Gulozen layer equations in torch on the CPU -- TEST INFRASTRUCTURE ONLY.

One function per mechanism, written token by token where the mechanism is a recurrence, with explicit per-head keys and
values (no latent "absorption", no paging, no batching): the opposite route from the product kernels in
lmdeploy_b200/csrc/hybrid_ops.cu, with which it shares no code.  `dt` is the dtype everything runs in (float64 by default).

Notation: n tokens of one sequence, W model width, weights stored [out, in] and applied as x @ W.T."""
import math

import torch


def silu(z):
    return z * torch.sigmoid(z)


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def grouped_rms_norm(x, w, groups, eps):
    """Split the last axis into `groups` equal consecutive parts, bring each to unit rms by itself, scale by w."""
    shp = x.shape
    parts = x.reshape(*shp[:-1], groups, shp[-1] // groups)
    return rms_unit(parts, eps).reshape(shp) * w


def causal_taps(h, w, before):
    """h [n, W]; w [W, taps]; `before` [taps-1, W] = the inputs that precede h (zeros at a sequence's start).
    Returns (h + conv(h), the last taps-1 inputs) with conv(h)_t = sum_j w[:, j] * h_(t - taps + 1 + j)."""
    taps = w.shape[1]
    full = torch.cat([before, h], 0)                       # index t + taps - 1 is h_t
    out = h.clone()
    for t in range(h.shape[0]):
        for j in range(taps):
            out[t] = out[t] + w[:, j] * full[t + j]
    return out, full[full.shape[0] - (taps - 1):].clone()


def rotary_frequencies(dims, base, scaling=None):
    """Angle per position of pair i (i < dims/2), and the factor on cos and sin.  `scaling` = dict(factor, original, fast,
    slow) blends f_i with f_i / factor along a ramp over the pair index."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, freqs, magnitude):
    """x [n, ..., d]: dimension 2i pairs with 2i+1 for i < len(freqs); dimensions past 2 * len(freqs) pass unchanged."""
    out = x.clone()
    for t in range(x.shape[0]):
        for i, f in enumerate(freqs):
            a = float(positions[t]) * f
            c, s = math.cos(a) * magnitude, math.sin(a) * magnitude
            u, v = x[t, ..., 2 * i], x[t, ..., 2 * i + 1]
            out[t, ..., 2 * i] = u * c - v * s
            out[t, ..., 2 * i + 1] = v * c + u * s
    return out


def lightning_mixer(h, p, m, eps, state):
    """Decayed linear attention.  h [n, W]; p = the layer's 'mix.*' tensors; m = its 'mixer' config; state [H, dim, vdim]
    (updated in place): S <- decay_h * S + k v^T, o = S^T q, per token and head."""
    H, D, V = m["heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q = silu(h @ p["q"].T).reshape(n, H, D)
    k = silu(h @ p["k"].T).reshape(n, H, D)
    v = silu(h @ p["v"].T).reshape(n, H, V)
    o = torch.zeros(n, H, V, dtype=h.dtype)
    for t in range(n):
        for a in range(H):
            state[a] = float(m["decay"][a]) * state[a] + torch.outer(k[t, a], v[t, a])
            o[t, a] = state[a].T @ q[t, a]
    y = rms_unit(o.reshape(n, H * V), eps) * p["norm"]
    y = y * torch.sigmoid(h @ p["g"].T)
    return y @ p["o"].T


def latent_attention_mixer(h, p, m, eps, positions, past):
    """Attention whose keys and values are expanded from a cached latent.  `past` = dict(c [m, kv_rank], kr [m, rot_dim])
    of the earlier tokens (replaced by the extended one).  Keys and values are built per head for every cached token."""
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    n = h.shape[0]
    rot = m["rot"]
    freqs, mag = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    cq = rms_unit(h @ p["dq"].T, eps) * p["dq.norm"]
    q = (cq @ p["uq"].T).reshape(n, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], positions, freqs, mag)
    ckv = h @ p["dkv"].T
    c = rms_unit(ckv[:, :C], eps) * p["dkv.norm"]
    kr = rotate_pairs(ckv[:, C:], positions, freqs, mag)
    past["c"] = torch.cat([past["c"], c], 0)
    past["kr"] = torch.cat([past["kr"], kr], 0)
    keys = (past["c"] @ p["uk"].T).reshape(-1, H, D)
    vals = (past["c"] @ p["uv"].T).reshape(-1, H, V)
    first = past["c"].shape[0] - n                            # cache index of this call's first token
    o = torch.zeros(n, H, V, dtype=h.dtype)
    for t in range(n):
        seen = first + t + 1
        for a in range(H):
            s = (keys[:seen, a] @ q_plain[t, a] + past["kr"][:seen] @ q_rot[t, a]) * m["scale"]
            top = max(float(s.max()), float(p["sink"][a]))
            e = torch.exp(s - top)
            w = e / (e.sum() + math.exp(float(p["sink"][a]) - top))
            o[t, a] = w @ vals[:seen, a]
    y = o.reshape(n, H * V) * torch.sigmoid(h @ p["g"].T)
    return y @ p["o"].T


def routed_experts(h, p, f):
    """h [n, W]; p = the layer's 'mlp.*' tensors; f = its 'mlp' config.  softmax over all experts, the `top` largest,
    their scores as weights (not renormalised)."""
    E, top = f["router"]["experts"], f["router"]["top"]
    s = torch.softmax(h @ p["router"].T, -1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: -float(s[t, e]))[:top]
        for e in order:
            mid = silu(p[f"e{e}.gate"] @ h[t]) * (p[f"e{e}.up"] @ h[t])
            out[t] = out[t] + s[t, e] * (p[f"e{e}.down"] @ mid)
    return out


class Sequence:
    """What one sequence carries from call to call."""

    def __init__(self, cfg, dt=torch.float64):
        W, taps = cfg["width"], cfg["canon"]["taps"]
        self.length = 0
        self.taps = [torch.zeros(taps - 1, W, dtype=dt) for _ in cfg["layers"]]
        self.mix = []
        for layer in cfg["layers"]:
            m = layer["mixer"]
            if layer["type"] == "lightning":
                self.mix.append(torch.zeros(m["heads"], m["dim"], m["vdim"], dtype=dt))
            else:
                self.mix.append(dict(c=torch.zeros(0, m["kv_rank"], dtype=dt), kr=torch.zeros(0, m["rot_dim"], dtype=dt)))


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, seq, trace=None):
    """Feed `tokens` (the next tokens of `seq`) -> logits [n, vocab].  `tensors`: name -> tensor of seq's dtype.
    trace: a list that receives the stream after every layer."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    n = len(tokens)
    positions = list(range(seq.length, seq.length + n))
    x = tensors["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    history = [x]
    for i, layer in enumerate(cfg["layers"]):
        h, seq.taps[i] = causal_taps(x, tensors[f"l{i}.canon1"], seq.taps[i])
        p = sub(tensors, f"l{i}.mix.")
        if layer["type"] == "lightning":
            y = lightning_mixer(h, p, layer["mixer"], eps, seq.mix[i])
        elif layer["type"] == "latent_attention":
            y = latent_attention_mixer(h, p, layer["mixer"], eps, positions, seq.mix[i])
        else:
            raise ValueError(layer["type"])
        x = x + grouped_rms_norm(y, tensors[f"l{i}.norm1"], groups, eps)
        if layer.get("mlp") is not None:
            y = routed_experts(x, sub(tensors, f"l{i}.mlp."), layer["mlp"])
            x = x + grouped_rms_norm(y, tensors[f"l{i}.norm2"], groups, eps)
        history.append(x)
        d = tensors[f"l{i}.dwa"]
        x = sum(d[j] * history[j] for j in range(i + 2))
        if trace is not None:
            trace.append(x.clone())
    seq.length += n
    return grouped_rms_norm(x, tensors["final.norm"], groups, eps) @ tensors["head"].T
