"""Scenarios every engine serving a Bodopel decoder must pass, whatever runs its operators: `make(cfg, tensors, **kw)` builds
the engine (bodopel_cases.build_engine with a device, dtype and library chosen by the caller), `tol` bounds
hybrid_cases.rel_error against the float64 oracle.  Run on the CPU through the numpy stand-in (tests/test_bodopel_cpu.py: host
logic -- runs of looped layers, pages, slots, row addressing, scheduling) and on a GPU through the CUDA kernels
(tests/test_bodopel_gpu.py)."""
import numpy as np
import torch

import bodopel_cases as BC
from oracle import bodopel as B


def _check(got, want, tol, what):
    err = BC.rel_error(got, want)
    assert err.max() <= tol, f"{what}: relative error {err.max():.3g} at position {int(err.argmax())} (bound {tol})"


def whole_prompt(make, tol):
    """Whole prompts: longer than every window and than a page, a single token, a few tokens."""
    cfg = BC.config()
    w = BC.random_tensors(cfg)
    P = BC.prompts_for(cfg, {"a": 150, "b": 1, "c": 5})
    got = BC.replay(make(cfg, w), P, [[("a", 150)], [("b", 1)], [("c", 5)]])
    for k in P:
        _check(got[k], BC.oracle_logits(cfg, w, P[k]), tol, f"whole prompt {k}")


def layer_by_layer(make, tol):
    """The residual stream after every run (a looped layer counts once per pass) against the oracle's."""
    cfg = BC.config()
    w = BC.random_tensors(cfg, seed=2)
    P = BC.prompts_for(cfg, {"a": 80})
    eng = make(cfg, w)
    eng.layer_trace = []
    BC.replay(eng, P, [[("a", 80)]])
    want = []
    BC.oracle_logits(cfg, w, P["a"], trace=want)
    assert len(eng.layer_trace) == len(want) == 6                     # 1 + 2 x 2 + 1 runs
    for r, (g, x) in enumerate(zip(eng.layer_trace, want)):
        err = float((g.double().cpu() - x).abs().max() / x.abs().max())
        assert err <= tol, f"stream after run {r}: {err:.3g} of its largest value (bound {tol})"


def prefill_then_decode(make, tol, n=200, tail=120):
    """Most of a prompt in one step, the rest token by token: decoded tokens cross page borders (127 -> 128, 191 -> 192) and
    every window (5, 9, 33, 70) passes wholly over decoded tokens."""
    cfg = BC.config()
    w = BC.random_tensors(cfg, seed=3)
    P = BC.prompts_for(cfg, {"a": n})
    got = BC.replay(make(cfg, w), P, [[("a", n - tail)]] + [[("a", 1)]] * tail)
    _check(got["a"], BC.oracle_logits(cfg, w, P["a"]), tol, "prefill then decode")


def token_by_token(make, tol, n=76):
    """Every token alone from the first: the first tokens meet empty conv histories and windows that are not full yet."""
    cfg = BC.config()
    w = BC.random_tensors(cfg, seed=4)
    P = BC.prompts_for(cfg, {"a": n})
    got = BC.replay(make(cfg, w), P, [[("a", 1)]] * n)
    _check(got["a"], BC.oracle_logits(cfg, w, P["a"]), tol, "token by token")


def portions(make, tol):
    """Portions of several sizes down to one and two tokens (shorter than the convolution), cut inside pages, at their borders
    and inside windows."""
    cfg = BC.config(taps=4)
    w = BC.random_tensors(cfg, seed=5)
    cuts = [2, 3, 1, 2, 56, 2, 1, 61, 2, 64, 5, 9, 2, 33]
    P = BC.prompts_for(cfg, {"a": sum(cuts)})
    got = BC.replay(make(cfg, w), P, [[("a", c)] for c in cuts])
    _check(got["a"], BC.oracle_logits(cfg, w, P["a"]), tol, "portions")


def unequal_batch(make, tol):
    """Requests of unequal length in one batch -- portions beside single tokens -- against each alone."""
    cfg = BC.config()
    w = BC.random_tensors(cfg, seed=6)
    P = BC.prompts_for(cfg, {"a": 90, "b": 7, "c": 66, "d": 2})
    sched = [[("a", 30), ("b", 3)], [("b", 1), ("c", 64), ("a", 2)], [("a", 50), ("d", 2), ("c", 1), ("b", 1)],
             [("c", 1), ("a", 1), ("b", 2)], [("a", 7)]]
    got = BC.replay(make(cfg, w), P, sched)
    for k in P:
        _check(got[k], BC.oracle_logits(cfg, w, P[k]), tol, f"batched {k}")


def reuse_of_pages_and_slots(make, tol):
    """A pool of 3 pages and 2 state slots serves requests one after another and side by side: every page and slot is handed
    out again, and a request repeated in a used slot gives what it gave in a fresh one."""
    cfg = BC.config()
    w = BC.random_tensors(cfg, seed=7)
    P = BC.prompts_for(cfg, {"a": 100, "b": 20, "c": 64})
    eng = make(cfg, w, blocks=3, max_batch=2)
    sched = [[("a", 64), ("b", 20)], [("a", 36), ("c", 10)], [("c", 54), ("b#2", 5)], [("b#2", 15), ("a#2", 30)], [("a#2", 70)],
             [("c#2", 64), ("b#3", 20)]]
    got = BC.replay(eng, P, sched)
    assert eng.scheduler.alloc.num_free == 3 and sorted(eng.scheduler.slots) == [0, 1]
    for k, v in got.items():
        _check(v, BC.oracle_logits(cfg, w, P[k.split("#")[0]]), tol, f"reuse {k}")


def other_sizes(make, tol):
    """Sizes that a given model may make equal or 1: no loop, a loop of one pass, a loop over every layer, a loop that starts
    after the first layer and ends before the last, one head, as many key/value heads as heads, a window of one token, a window
    longer than the prompt, no feed-forward anywhere, no convolution history (taps 1), dim equal to vdim, a lone layer."""
    A = BC.attention
    stacks = [
        dict(layers=[dict(A(heads=1, kv_heads=1, dim=4, vdim=4, window=1), mlp=None)], width=16, taps=1, vocab=9, loop=None),
        dict(layers=[dict(A(heads=5, kv_heads=5, dim=8, vdim=3, window=500), mlp=BC.dense(8)),
                     dict(A(heads=8, kv_heads=2, dim=4, vdim=12, window=2, softcap=1.0), mlp=None)], width=40, taps=5, vocab=33, loop=(0, 2, 3)),
        dict(layers=[dict(A(), mlp=BC.dense(16)), dict(A(window=64), mlp=BC.dense(16)), dict(A(window=65), mlp=None)], width=24, taps=2,
             vocab=20, loop=(1, 2, 1)),
        dict(layers=[dict(A(heads=9, kv_heads=3, dim=36, vdim=40, window=63), mlp=BC.dense(100)), dict(A(heads=2, kv_heads=1), mlp=None)],
             width=72, taps=3, vocab=50, loop=(1, 2, 4)),
    ]
    for k, kw in enumerate(stacks):
        cfg = BC.config(**kw)
        w = BC.random_tensors(cfg, seed=10 + k)
        P = BC.prompts_for(cfg, {"a": 131, "b": 4})
        got = BC.replay(make(cfg, w), P, [[("a", 3)], [("a", 62), ("b", 2)], [("a", 1), ("b", 1)], [("a", 1)], [("a", 62), ("b", 1)], [("a", 1)],
                                          [("a", 1)]])
        for name in P:
            _check(got[name], BC.oracle_logits(cfg, w, P[name]), tol, f"sizes {k} {name}")


def wider_sizes(make, tol):
    """Sizes of the order of a real layer's heads: 16 query heads on 2 key/value heads (more heads per key/value head than one
    walk over a key takes), head dimensions of 64 and 128 (16-byte key reads) and an odd one (scalar reads), a window of 300 keys
    cut into key ranges when few rows are fed."""
    A = BC.attention
    stacks = [
        dict(layers=[dict(A(heads=16, kv_heads=2, dim=64, vdim=32, window=300, scale=0.05), mlp=BC.dense(96)),
                     dict(A(heads=20, kv_heads=2, dim=24, vdim=8, window=40, scale=0.1), mlp=None)], width=128, vocab=77, loop=(0, 1, 2), max_positions=400),
        dict(layers=[dict(A(heads=4, kv_heads=4, dim=128, vdim=128, window=129, scale=0.03), mlp=None),
                     dict(A(heads=3, kv_heads=1, dim=33, vdim=65, window=200, scale=0.1), mlp=BC.dense(64))], width=64, vocab=50, loop=None,
             max_positions=400),
    ]
    for k, kw in enumerate(stacks):
        cfg = BC.config(**kw)
        w = BC.random_tensors(cfg, seed=20 + k)
        P = BC.prompts_for(cfg, {"a": 380, "b": 5})
        got = BC.replay(make(cfg, w, blocks=8), P, [[("a", 310), ("b", 2)], [("a", 60), ("b", 1)], [("a", 1), ("b", 2)]] + [[("a", 1)]] * 9)
        for name in P:
            _check(got[name], BC.oracle_logits(cfg, w, P[name]), tol, f"wider sizes {k} {name}")


def greedy_generation(make, tol, new=10):
    """batched_generate (the scheduler's own admission, chunking and retirement, greedy sampling on the device) against the
    oracle generating greedily; a position whose two best oracle logits are closer than the tolerance may differ."""
    from lmdeploy_b200.messages import GenerationConfig
    from lmdeploy_b200.turbomind.engine import batched_generate
    cfg = BC.config()
    w = BC.random_tensors(cfg, seed=8)
    P = BC.prompts_for(cfg, {"a": 9, "b": 70, "c": 1})
    eng = make(cfg, w, blocks=4, max_batch=2, prefill_tokens=32)       # prompts longer than a step's token budget are chunked
    seqs = batched_generate(eng, [P[k] for k in "abc"], GenerationConfig(max_new_tokens=new, ignore_eos=True))
    assert eng.scheduler.alloc.num_free == 4 and sorted(eng.scheduler.slots) == [0, 1]
    for k, s in zip("abc", seqs):
        assert len(s.generated) == new and s.finish_reason == "length"
        toks = list(P[k])
        for i, t in enumerate(s.generated):
            lg = BC.oracle_logits(cfg, w, toks)[-1]
            if int(lg.argmax()) != t:
                assert lg.max() - lg[t] <= 4 * tol * np.abs(lg).max(), f"{k}: token {i} is {t}, oracle {int(lg.argmax())}"
            toks.append(t)


# ------------------------------------------------------------------------------------------------ one mechanism at a time
def _step_arrays(eng, start, n, pages, slot=1):
    """Step arrays of ONE sequence feeding rows [start, start + n), its pages in the given (shuffled) order."""
    from lmdeploy_b200.turbomind.hybrid import StepArrays
    dev = eng.model.device
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    ptrs = torch.tensor([eng.pool.base + b * eng.pool.block_bytes for b in pages], dtype=torch.int64, device=dev)
    return StepArrays(n=n, batch=1, tok_seq=i32([0] * n), tok_pos=i32(list(range(start, start + n))), cu_q=i32([0, n]), seq_slot=i32([slot]),
                      block_ptrs=ptrs, cu_blocks=i32([0, len(pages)]), state=eng.state, max_pos=start + n - 1)


def _close(got, want, tol, what):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
    assert err <= tol, f"{what}: {err:.3g} of the largest value (bound {tol})"


def marked_keys_at_window_and_page_edges(make, tol, cuts=((140,), (61, 3, 64, 1, 1, 2, 1, 1, 1, 1, 1, 1, 1, 1))):
    """The mixer alone, with weights and inputs made so that ONE score stands out: marked rows carry a large component along the
    first input channel, and the first columns of the query and key projections agree per head, so a marked query gives a marked
    key some twenty units of score more than any other.  Marked positions sit at the first token, at page borders (63, 64) and a
    window's length - 1 and a window's length behind other marked positions: a window one key too long or too short, a key lost at
    a page border or a wrong first token moves the output by its whole size.  Run as a prompt and with the tail token by token."""
    window = 70
    cfg = BC.config(layers=[dict(BC.attention(heads=4, kv_heads=2, dim=8, vdim=6, window=window, scale=3.0, softcap=60.0), mlp=None)], loop=None)
    w = BC.random_tensors(cfg, seed=31)
    m = cfg["layers"][0]["mixer"]
    g = torch.Generator().manual_seed(5)
    col = torch.randn(2, 8, generator=g).sign()                         # per key/value head: the direction marked rows share
    w["l0.mix.k"][:, 0] = col.reshape(-1) * 0.5
    w["l0.mix.q"][:, 0] = col.repeat_interleave(2, 0).reshape(-1) * 0.5
    for k in ("q", "k"):
        w[f"l0.mix.{k}.b"].zero_()
        w[f"l0.mix.{k}.norm"].fill_(1.0)
    w["l0.mix.r1"].fill_(0.25)
    marked = [0, 63, 64, 63 + window - 1, 63 + window, 64 + window]     # 132 sees 63 (just inside); 133 sees 64 but not 63; 134 neither
    n = 140
    h = 0.2 * torch.randn(n, cfg["width"], generator=g)
    h[:, 0] = 0.0
    h[marked, 0] = 40.0
    h = h.to(torch.bfloat16).to(torch.float32)
    p64 = {k[len("l0.mix."):]: v.double() for k, v in w.items() if k.startswith("l0.mix.")}
    want = B.attention_mixer(h.double(), p64, m, cfg["norm"]["eps"], list(range(n)),
                             dict(k=torch.zeros(0, 2, 8, dtype=torch.float64), v=torch.zeros(0, 2, 6, dtype=torch.float64)))
    # the marked keys decide the marked queries' outputs in the oracle itself: dropping the key just inside changes them
    for cut in cuts:
        eng = make(cfg, w)
        model, at, got = eng.model, 0, []
        for c in cut:
            c = min(c, n - at)
            x = h[at:at + c].to(model.device, model.T).contiguous()
            y = model.window_mixer(0, x, _step_arrays(eng, at, c, [2, 0, 1]))
            got.append(torch.mm(y.float(), model.w["l0.o"].float().t()).cpu())
            at += c
        assert at == n
        _close(torch.cat(got), want, tol, f"marked keys, portions {cut[:3]}...")
    seen = B.window_scores((p64["q"] @ h[132].double()).reshape(4, 8), torch.zeros(1, 4, 8, dtype=torch.float64), 132, 132, m, p64["r1"], p64["r2"])
    assert seen.shape == (4, 1)


def residual_norm_and_both_convolutions(make, tol):
    """Pre-norm input of both sublayers in portions shorter than the taps: the stream takes in the pending output and a vector
    for all rows, the norm multiplies by one plus the stored weight, the convolution of each sublayer keeps its own history."""
    cfg = BC.config(taps=4, loop=None)
    w = BC.random_tensors(cfg, seed=32)
    eng = make(cfg, w)
    model = eng.model
    W, n, eps = cfg["width"], 75, cfg["norm"]["eps"]
    g = torch.Generator().manual_seed(6)
    x0 = torch.randn(n, W, generator=g)
    add = torch.randn(n, W, generator=g).to(torch.bfloat16).float()
    vec = torch.randn(W, generator=g).to(torch.bfloat16).float()
    for sub in (1, 2):
        xs = (x0 + add + vec).double()
        want, _ = B.causal_taps(B.offset_norm(xs, w[f"l0.norm{sub}"].double(), eps), w[f"l0.canon{sub}"].double(),
                                torch.zeros(3, W, dtype=torch.float64))
        got, at = [], 0
        for c in [2, 1, 3, 1, 1, 60, 2, 5]:
            x = x0[at:at + c].to(model.device).contiguous()
            pend = add[at:at + c].to(model.device, model.T).contiguous()
            ev = vec.to(model.device, model.T).contiguous()
            got.append(model.norm_conv_input(0, 0, sub, x, pend, ev.data_ptr(), _step_arrays(eng, at, c, [0, 1])).float().cpu())
            _close(x.cpu(), xs[at:at + c], 1e-6, "stream after the add")
            at += c
        assert at == n
        _close(torch.cat(got), want, tol, f"input of sublayer {sub}")


def feed_forward_alone(make, tol):
    """down(relu(up h)^2) over rows with negative and positive pre-activations."""
    cfg = BC.config(loop=None)
    w = BC.random_tensors(cfg, seed=33)
    eng = make(cfg, w)
    model = eng.model
    h = torch.randn(37, cfg["width"], generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).float()
    want = B.squared_relu_ff(h.double(), {"up": w["l0.mlp.up"].double(), "down": w["l0.mlp.down"].double()})
    got = model.dense_mlp(0, h.to(model.device, model.T).contiguous()).float().cpu()
    _close(got, want, tol, "feed-forward")


def embedding_with_positions_and_pass_vectors(make, tol):
    """The stream after the first run depends on the scaled embedding, the position's vector (a request that starts at position
    0 against the same tokens fed later at other positions) and the vector of the first pass of a loop that starts at layer 0."""
    cfg = BC.config(layers=[dict(BC.attention(window=4), mlp=None)], loop=(0, 1, 3))
    w = BC.random_tensors(cfg, seed=34)
    toks = BC.prompts_for(cfg, {"a": 6})["a"]
    P = {"a": toks + toks}                                                   # the same six tokens at positions 0..5 and 6..11
    eng = make(cfg, w)
    eng.layer_trace = []
    got = BC.replay(eng, P, [[("a", 6)], [("a", 6)]])
    want = []
    _check(got["a"], BC.oracle_logits(cfg, w, P["a"], trace=want), tol, "repeated tokens")
    first, second = eng.layer_trace[0].double().cpu(), eng.layer_trace[3].double().cpu()       # run 0 of the first and of the second step
    for g, x in ((first, want[0][:6]), (second, want[0][6:])):
        assert float((g - x).abs().max() / x.abs().max()) <= tol
    assert float((first - second).abs().max()) > 0.1                         # positions matter


def score_scratch_in_row_chunks(make, tol):
    """The rows of a step pass through the attention in chunks when the scratch between its two passes is bounded: chunks of 4
    rows here, cut inside sequences and between them."""
    cfg = BC.config()
    w = BC.random_tensors(cfg, seed=35)
    P = BC.prompts_for(cfg, {"a": 93, "b": 21, "c": 3})
    eng = make(cfg, w)
    eng.model.window_scratch_bytes = 1
    got = BC.replay(eng, P, [[("a", 50), ("b", 21), ("c", 2)], [("a", 43), ("c", 1)]])
    for k in P:
        _check(got[k], BC.oracle_logits(cfg, w, P[k]), tol, f"row chunks {k}")


ALL = [feed_forward_alone, score_scratch_in_row_chunks, embedding_with_positions_and_pass_vectors, whole_prompt, layer_by_layer, prefill_then_decode, token_by_token, portions, unequal_batch, reuse_of_pages_and_slots, other_sizes,
       wider_sizes, greedy_generation, marked_keys_at_window_and_page_edges, residual_norm_and_both_convolutions]
