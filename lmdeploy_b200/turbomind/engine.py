"""TurboMind / TurboMindInstance: the host-side engine the Python API drives.

Mirrors lmdeploy/turbomind/turbomind.py (TurboMind :108-566, TurboMindInstance :568-813): an engine object owning
weights + KV pool, instances that stream tokens for a session.  The model forward is the native decode step
(libb200tm.so); scheduling is lmdeploy_b200.turbomind.scheduler."""
import asyncio
import os
import threading
from typing import List, Optional

import torch

from ..messages import DEFAULT_MAX_BATCH_SIZE, EngineOutput, GenerationConfig, ResponseType, TurbomindEngineConfig
from .runtime import DecodeModel, KvCachePool
from .scheduler import InputLengthError, Scheduler, Sequence
from .specs import SPECS, ModelSpec


def marshal_step(batch, block_ptr=None):
    """Argument arrays of one (mixed) step for `batch` = [Sequence]: sequence i feeds its `step_tokens` next tokens as
    rows [cu_q_len[i], cu_q_len[i+1]); cu_k_len counts cached history + the fed tokens (AttentionParams::cu_k_len
    includes the new tokens); block_ids is the concatenation of the sequences' block tables (pool indices -- what a TP
    leader broadcasts; every rank maps them to addresses of its own pool) and block_ptrs their addresses through
    `block_ptr` when one is given."""
    tokens, cu_q, cu_k, ids, cu_blocks = [], [0], [0], [], [0]
    q = k = max_k = 0
    for s in batch:
        n = s.step_tokens
        cached = s.cached
        prompt = s.prompt
        if n == 1 and cached < len(prompt) + len(s.generated):      # steady decode: one row, the token at position `cached`
            tokens.append(int(prompt[cached] if cached < len(prompt) else s.generated[cached - len(prompt)]))
        else:
            toks = s.next_inputs()
            if len(toks) != n:
                raise RuntimeError(f"session {s.session_id}: scheduled {n} tokens but {len(toks)} are available")
            tokens += [int(t) for t in toks]
        blocks = s.blocks
        if not blocks:
            raise RuntimeError(f"session {s.session_id} runs without KV blocks")
        q += n
        end = cached + n
        k += end
        if end > max_k:
            max_k = end
        cu_q.append(q)
        cu_k.append(k)
        ids += blocks
        cu_blocks.append(len(ids))
    st = dict(batch_size=len(batch), token_ids=tokens, token_num=len(tokens), cu_q_len=cu_q, cu_k_len=cu_k, block_ids=ids,
              cu_block_nums=cu_blocks, max_k_len=max_k)
    if block_ptr is not None:
        st["block_ptrs"] = [block_ptr(b) for b in ids]
    return st


class TurboMind:
    def __init__(self, spec: ModelSpec, engine_config: Optional[TurbomindEngineConfig] = None, *, model: DecodeModel = None,
                 eos_id: Optional[int] = None, num_blocks: Optional[int] = None, seed=0, channel=None):
        cfg = engine_config or TurbomindEngineConfig()
        if cfg.tp != 1 and (model is None or channel is None):
            raise NotImplementedError("tp > 1: launch one process per GPU (torchrun), give every rank its TP-sharded "
                                      "DecodeModel (lmdeploy_b200.turbomind.tp.TpGroup) and a StepChannel "
                                      "(lmdeploy_b200.turbomind.tp_engine); rank 0 drives step(), the others "
                                      "serve_follower()")
        self.channel = channel
        self.config = cfg
        self.spec = spec
        self.eos_id = eos_id
        self.max_batch = cfg.max_batch_size or DEFAULT_MAX_BATCH_SIZE
        self.hybrid = bool(getattr(spec, "hybrid", False))
        self._lock = threading.Lock()
        self._next_session = 0
        self.h2d_bytes = self.d2h_bytes = 0          # running totals of the step traffic (bench.py reports them per step)
        if self.hybrid:
            self._init_hybrid(cfg, model, num_blocks, seed)
            return
        # session_len left unset: what _get_and_verify_max_len derives from the HF config (converter.py get_tm_config step 4;
        # loader.default_session_len), 2048 when the config names no context length
        self.session_len = cfg.session_len or spec.session_len or spec.max_position_embeddings or 2048
        self.block_len = cfg.cache_block_seq_len
        self.model = model or DecodeModel(spec, quant_policy=cfg.quant_policy, block_len=self.block_len,
                                          max_batch=self.max_batch)
        if model is None:
            self.model.load_synthetic(seed)
        dev = self.model.device
        if num_blocks is None:
            if cfg.cache_max_entry_count >= 1:
                num_blocks = int(cfg.cache_max_entry_count)
            else:   # ratio of free memory, as CreateEngine does (turbomind.cc:293-311)
                free, _ = torch.cuda.mem_get_info(dev)
                num_blocks = int(free * cfg.cache_max_entry_count) // (self.model.layer_bytes * spec.layers)
        self.pool = KvCachePool(num_blocks, spec.layers, self.model.kv_heads, spec.head_dim, self.block_len,
                                cfg.quant_policy, device=dev)
        # Chunked prefill: a sequence still inside its prompt feeds up to B200_CHUNKED_PREFILL tokens (default 64) per step
        # through b200_model_chunk_step (tcgen05 prefill attention; parity-green on a B200 against the oracle, the
        # reference's own prefill kernels and token-by-token feeding: tests/test_prefill_attention_gpu.py,
        # tests/test_engine_gpu.py) as long as the step's row budget (max_batch rows) has room.  1 = one prompt token per
        # step through the decode kernel.
        chunk = int(os.environ.get("B200_CHUNKED_PREFILL", "64"))
        self.scheduler = Scheduler(max_batch=self.max_batch, block_len=self.block_len, num_blocks=num_blocks,
                                   session_len=self.session_len, prefix_caching=cfg.enable_prefix_caching,
                                   prefill_chunk=min(chunk, cfg.max_prefill_token_num), token_budget=self.max_batch)
        B = self.max_batch
        self._max_blocks = (self.session_len + self.block_len - 1) // self.block_len
        # Per-step control arrays live in ONE int32 device buffer [tokens B | cu_q B+1 | cu_k B+1 | cu_blocks B+1] fed by one
        # pinned staging buffer: a step costs a single ~1 KB H2D copy (plus the block table only when it changed) --
        # the counterpart of the pinned staging in UnifiedAttentionLayer::Setup (unified_attention_layer.cc:288-305).
        self._o_q, self._o_k, self._o_b, n_ctl = B, 2 * B + 1, 3 * B + 2, 4 * B + 3
        self.d_ctl = torch.zeros(n_ctl, dtype=torch.int32, device=dev)
        self.h_ctl = torch.zeros(n_ctl, dtype=torch.int32).pin_memory()
        self._h_ctl = self.h_ctl.numpy()
        self.d_tokens = self.d_ctl[:B]
        self.d_cu_q = self.d_ctl[self._o_q:self._o_q + B + 1]
        self.d_cu_k = self.d_ctl[self._o_k:self._o_k + B + 1]
        self.d_cu_blocks = self.d_ctl[self._o_b:self._o_b + B + 1]
        self.d_out = torch.zeros(B, dtype=torch.int32, device=dev)
        self.d_block_ptrs = torch.zeros(B * self._max_blocks, dtype=torch.int64, device=dev)
        self.h_out = torch.zeros(B, dtype=torch.int32).pin_memory()
        self._h_out = self.h_out.numpy()
        self.h_block_ptrs = torch.zeros(B * self._max_blocks, dtype=torch.int64).pin_memory()
        self._h_block_ptrs = self.h_block_ptrs.numpy()
        self._last_block_ids = None
        self._use_graphs = os.environ.get("B200_ENGINE_GRAPHS", "1") != "0"
        self._graphs, self._seen_sizes = {}, set()

    def _init_hybrid(self, cfg, model, num_blocks, seed):
        """Engine state for a hybrid decoder (specs.HybridSpec): the same scheduler and block pool, plus recurrent-state slots,
        one per batch slot.  A step may carry whole prompt portions (up to max_prefill_token_num rows), so the per-step
        arrays are packed on the host into one pinned buffer sized by the step and uploaded with one copy."""
        from .hybrid import HybridModel
        spec = self.spec
        if cfg.tp != 1 or self.channel is not None:
            raise NotImplementedError("hybrid decoders run on one GPU")
        if cfg.quant_policy != 0:
            raise NotImplementedError("hybrid decoders keep their latent cache in the projection type (quant_policy 0)")
        if cfg.enable_prefix_caching:
            raise NotImplementedError("prefix caching with recurrent state (the state at a block border is not kept)")
        self.session_len = cfg.session_len or spec.session_len or 2048
        if spec.max_positions:                      # learned positions: nothing is fed past the table (the token after it may be sampled)
            self.session_len = min(self.session_len, spec.max_positions + 1)
        self.block_len = cfg.cache_block_seq_len
        self.model = model or HybridModel(spec, block_len=self.block_len, max_batch=self.max_batch)
        if model is None:
            self.model.load_synthetic(seed)
        dev = self.model.device
        if num_blocks is None:
            if cfg.cache_max_entry_count >= 1:
                num_blocks = int(cfg.cache_max_entry_count)
            else:
                free, _ = torch.cuda.mem_get_info(dev)
                num_blocks = int(free * cfg.cache_max_entry_count) // self.model.block_bytes
        self.pool = self.model.make_cache(num_blocks)
        self.state = self.model.make_state(self.max_batch)
        budget = max(self.max_batch, cfg.max_prefill_token_num)
        self.scheduler = Scheduler(max_batch=self.max_batch, block_len=self.block_len, num_blocks=num_blocks,
                                   session_len=self.session_len, prefix_caching=False,
                                   prefill_chunk=max(1, cfg.max_prefill_token_num), token_budget=budget, state_slots=self.max_batch)
        self.last_logits = None          # float logits [rows, vocab] of the last step and the row each belongs to
        self.last_rows = {}
        self._max_blocks = (self.session_len + self.block_len - 1) // self.block_len
        self._use_graphs = os.environ.get("B200_ENGINE_GRAPHS", "1") != "0"
        self._hybrid_graphs, self._hybrid_seen = {}, set()

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path, engine_config=None, *, dtype=None, **kw):
        """`pretrained_model_name_or_path`: a key of SPECS (synthetic random weights of that geometry; no real
        checkpoints exist in this image) or a directory holding an HF-format checkpoint (config.json +
        *.safetensors, InternLM2 / Llama, fp16 or AWQ; or a hybrid decoder named by the config's `architecture`) read by
        lmdeploy_b200.turbomind.loader.  dtype: overrides engine_config.dtype for the loader; 'float32' (true 32-bit serving) is
        offered by hybrid decoders only and is not a value of TurbomindEngineConfig.dtype, whose rules are the reference's."""
        import os
        if pretrained_model_name_or_path in SPECS:
            return cls(SPECS[pretrained_model_name_or_path], engine_config, **kw)
        if os.path.isdir(pretrained_model_name_or_path):
            from .loader import load_hf_checkpoint
            cfg = engine_config or TurbomindEngineConfig()
            spec, model, eos = load_hf_checkpoint(pretrained_model_name_or_path, quant_policy=cfg.quant_policy,
                                                  block_len=cfg.cache_block_seq_len, hf_overrides=cfg.hf_overrides,
                                                  model_format=cfg.model_format,
                                                  max_batch=cfg.max_batch_size or DEFAULT_MAX_BATCH_SIZE, dtype=dtype or cfg.dtype)
            return cls(spec, cfg, model=model, eos_id=eos, **kw)
        raise FileNotFoundError(pretrained_model_name_or_path)

    def create_instance(self):
        return TurboMindInstance(self)

    # ------------------------------------------------------------------ one engine step
    def step(self, plan=None):
        """Schedule + run one step for the active batch; returns [(sequence, token|None)] events.  Under tensor
        parallelism only the leader (rank 0) calls this; it publishes the step's arrays to the followers first.
        plan: {session id: tokens to feed} runs exactly that batch instead of the scheduler's choice (Scheduler.schedule_planned)."""
        sched = self.scheduler
        batch = sched.schedule() if plan is None else sched.schedule_planned(plan)
        if not batch:
            # a tick may legitimately form no batch (it only retired or preempted); a long run of them with work pending
            # means the scheduler cannot make progress -- fail loudly instead of spinning in the callers' loops
            self._idle_ticks = getattr(self, "_idle_ticks", 0) + 1
            if sched.has_work and self._idle_ticks > 1000:
                raise RuntimeError(f"scheduler stalled: {sched.metrics()}")
            return []
        self._idle_ticks = 0
        st = marshal_step(batch)
        if self.channel is not None:
            self.channel.publish(st)
        cu_q = st["cu_q_len"]
        rows = [cu_q[i + 1] - 1 for i in range(len(batch))]                              # sample = last row of each sequence
        # rows whose logits a caller asked for by position (Sequence.logit_positions)
        asked = [(s, p, cu_q[i] + p - s.cached) for i, s in enumerate(batch) for p in s.logit_positions
                 if s.cached <= p < s.cached + s.step_tokens]
        if self.hybrid:
            out = self._execute_hybrid(st, batch, rows + [r for _, _, r in asked])
        else:
            out = self._execute(st)
        sampled = [out[r] for r in rows]
        if any(s.sampling is not None for s in batch):
            self._sample(batch, rows, sampled)
        if asked:
            lg = self._logits_of_rows([r for _, _, r in asked], st["token_num"])
            for (s, p, _), row in zip(asked, lg):
                s.position_logits[p] = row
                s.logit_positions.remove(p)
        events = sched.update(batch, sampled)
        if any(s.want_logits or s.want_logprobs for s in batch):
            self._collect_extras(batch, rows, events, st["token_num"])
        return events

    def _logits_of_rows(self, rows, token_num):
        """Float logits [len(rows), vocab] on the host for rows of the step that just ran."""
        if self.hybrid:
            idx = torch.tensor([self.last_rows[r] for r in rows], dtype=torch.long, device=self.last_logits.device)
            return self.last_logits.index_select(0, idx).cpu()
        lg = self.model.logits(token_num)[:, :self.spec.vocab]
        return lg[torch.tensor(rows, dtype=torch.long, device=lg.device)].float().cpu()

    def _execute_hybrid(self, st, batch, rows):
        """One step of a hybrid decoder: zero the state slot of every sequence that starts (position 0), pack the step's arrays
        [tokens n | tok_seq n | tok_pos n | cu_q B+1 | cu_blocks B+1 | seq_slot B | rows r] into one pinned buffer, upload,
        run HybridModel.step, arg-max the last row of every sequence.  Returns {row: greedy id}."""
        import numpy as np
        B, n = st["batch_size"], st["token_num"]
        dev = self.model.device
        for s in batch:
            if s.cached == 0:
                self.state.reset(s.slot)
        cu_q, cu_k = st["cu_q_len"], st["cu_k_len"]
        uniq = list(dict.fromkeys(rows))
        r = len(uniq)
        ctl = np.empty(3 * n + 2 * (B + 1) + B + r, np.int32)
        ctl[:n] = st["token_ids"]
        for i in range(B):
            lo, hi = cu_q[i], cu_q[i + 1]
            end = cu_k[i + 1] - cu_k[i]
            ctl[n + lo:n + hi] = i
            ctl[2 * n + lo:2 * n + hi] = np.arange(end - (hi - lo), end, dtype=np.int32)
        o = 3 * n
        ctl[o:o + B + 1] = cu_q
        ctl[o + B + 1:o + 2 * B + 2] = st["cu_block_nums"]
        ctl[o + 2 * B + 2:o + 3 * B + 2] = [s.slot for s in batch]
        ctl[o + 3 * B + 2:] = uniq
        ptrs = np.asarray(st["block_ids"], np.int64) * self.pool.block_bytes + self.pool.base
        pin = dev.type == "cuda"
        h_ctl = torch.from_numpy(ctl)
        h_ptrs = torch.from_numpy(ptrs)
        if pin:
            h_ctl, h_ptrs = h_ctl.pin_memory(), h_ptrs.pin_memory()
        self.h2d_bytes += ctl.nbytes + ptrs.nbytes
        max_pos = st["max_k_len"] - 1
        trace = getattr(self, "layer_trace", None)

        def run(d_ctl, d_ptrs):
            return self.model.step(n=n, batch=B, tokens=d_ctl[:n], tok_seq=d_ctl[n:2 * n], tok_pos=d_ctl[2 * n:3 * n],
                                   cu_q=d_ctl[o:o + B + 1], cu_blocks=d_ctl[o + B + 1:o + 2 * B + 2],
                                   seq_slot=d_ctl[o + 2 * B + 2:o + 3 * B + 2], block_ptrs=d_ptrs, state=self.state,
                                   rows=d_ctl[o + 3 * B + 2:], n_rows=r, max_pos=max_pos, trace=trace)

        # A step of single decoded tokens is shape-static given its batch size and the attention's key ranges: every array lives
        # in a fixed device buffer, so its launches are replayed from a CUDA graph, captured the second time the key is seen
        # (the engine does the same for dense models, per batch size).
        key = (B, self.model.decode_key(n, max_pos)) if n == B and uniq == list(range(B)) else None
        if key is not None and self._use_graphs and pin and trace is None and self.model.events is None:
            g = self._hybrid_graphs.get(key)
            if g is None and key in self._hybrid_seen:
                g = dict(ctl=torch.zeros(len(ctl), dtype=torch.int32, device=dev),
                         ptrs=torch.zeros(B * self._max_blocks, dtype=torch.int64, device=dev))
                g["ctl"].copy_(h_ctl)
                torch.cuda.synchronize(dev)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    g["logits"] = run(g["ctl"], g["ptrs"])
                    g["ids"] = self.model.argmax(g["logits"])
                g["graph"] = graph
                self._hybrid_graphs[key] = g
            self._hybrid_seen.add(key)
            if g is not None:
                g["ctl"].copy_(h_ctl, non_blocking=True)
                g["ptrs"][:len(ptrs)].copy_(h_ptrs, non_blocking=True)
                g["graph"].replay()
                self.last_logits, self.last_rows = g["logits"], {row: k for k, row in enumerate(uniq)}
                ids = g["ids"].cpu().tolist()
                self.d2h_bytes += 4 * r
                return {row: ids[k] for k, row in enumerate(uniq)}
        logits = run(h_ctl.to(dev, non_blocking=True), h_ptrs.to(dev, non_blocking=True))
        self.last_logits, self.last_rows = logits, {row: k for k, row in enumerate(uniq)}
        ids = self.model.argmax(logits).cpu().tolist()
        self.d2h_bytes += 4 * r
        return {row: ids[k] for k, row in enumerate(uniq)}

    def _sample(self, batch, rows, sampled):
        """do_sample sequences that produce a token in this step: the device sampling stage (b200_sample: repetition penalty,
        temperature, top-k, top-p, min-p, one XORWOW state per request seeded by GenerationConfig.random_seed -- what
        LogitsProcessor + Sampling do in the reference, generation/logits_processor.cc:66-125, generation/sampling.cc:92-183)
        replaces the step's arg-max for their rows, reading the same logits buffer."""
        import ctypes as C
        import numpy as np
        from .. import _lib as L
        lib, dev = L.load(), self.model.device
        items = [(i, s) for i, s in enumerate(batch) if s.sampling is not None and s.cached + s.step_tokens >= s.context_len]
        if not items:
            return
        if not hasattr(self, "_rng_states"):
            self._rng_bytes = lib.b200_sampling_rng_state_bytes()
            self._rng_states = torch.zeros(self.max_batch * self._rng_bytes, dtype=torch.uint8, device=dev)
            self._rng_free = list(range(self.max_batch - 1, -1, -1))
            self._samp_ws = torch.zeros(lib.b200_sampling_workspace_bytes(self.max_batch, self.spec.vocab), dtype=torch.uint8,
                                        device=dev)
            self._rng_owner = {}
        stream = torch.cuda.current_stream().cuda_stream
        # slots of finished requests return to the free list; new requests get a slot and their seed
        for slot, owner in list(self._rng_owner.items()):
            if owner.finished:
                del self._rng_owner[slot]
                self._rng_free.append(slot)
        fresh = [s for _, s in items if s.rng_slot < 0]
        if fresh:
            seeds = np.zeros(self.max_batch, np.uint64)
            mask = np.zeros(self.max_batch, np.uint8)
            for s in fresh:
                s.rng_slot = self._rng_free.pop()
                self._rng_owner[s.rng_slot] = s
                seeds[s.rng_slot], mask[s.rng_slot] = s.sampling["seed"] & 0xFFFFFFFFFFFFFFFF, 1
            d_seeds = torch.from_numpy(seeds.view(np.int64)).to(dev)
            d_mask = torch.from_numpy(mask).to(dev)
            L.check(lib.b200_sampling_init_rng(self._rng_states.data_ptr(), d_seeds.data_ptr(), d_mask.data_ptr(), self.max_batch,
                                               stream), "b200_sampling_init_rng")
        n = len(items)
        f32 = lambda key: torch.tensor([s.sampling[key] for _, s in items], dtype=torch.float32, device=dev)
        d_rows = torch.tensor([rows[i] for i, _ in items], dtype=torch.int32, device=dev)
        d_t, d_p, d_m, d_pen = f32("temperature"), f32("top_p"), f32("min_p"), f32("repetition_penalty")
        d_k = torch.tensor([s.sampling["top_k"] for _, s in items], dtype=torch.int32, device=dev)
        d_slot = torch.tensor([s.rng_slot for _, s in items], dtype=torch.int32, device=dev)
        d_out = torch.zeros(n, dtype=torch.int32, device=dev)
        p = L.SamplingParams()
        if self.hybrid:
            # the sampling stage reads T logits: the step's float logits as bf16, rows renumbered to that compact tensor
            lg16 = self.last_logits.to(torch.bfloat16).contiguous()
            d_rows = torch.tensor([self.last_rows[rows[i]] for i, _ in items], dtype=torch.int32, device=dev)
            p.logits, p.ld, p.dtype = lg16.data_ptr(), lg16.stride(0), 1
        else:
            p.logits, p.ld, p.dtype = lib.b200_model_buffer(self.model.handle, 0), self.model.vocab_local, self.model.cfg.dtype
        p.count, p.vocab = n, self.spec.vocab
        p.rows, p.temperature, p.top_k, p.top_p, p.min_p = (d_rows.data_ptr(), d_t.data_ptr(), d_k.data_ptr(), d_p.data_ptr(),
                                                            d_m.data_ptr())
        hist = None
        if any(s.sampling["repetition_penalty"] != 1.0 for _, s in items):
            # the ids seen so far (prompt + generated), uploaded for the requests that ask for the penalty
            hist = [torch.tensor((s.prompt + s.generated) if s.sampling["repetition_penalty"] != 1.0 else [0], dtype=torch.int32,
                                 device=dev) for _, s in items]
            d_hp = torch.tensor([h.data_ptr() for h in hist], dtype=torch.int64, device=dev)
            d_hl = torch.tensor([h.numel() if s.sampling["repetition_penalty"] != 1.0 else 0 for h, (_, s) in zip(hist, items)],
                                dtype=torch.int32, device=dev)
            p.repetition_penalty, p.history, p.history_len = d_pen.data_ptr(), d_hp.data_ptr(), d_hl.data_ptr()
        p.rng_states, p.rng_index, p.out_ids = self._rng_states.data_ptr(), d_slot.data_ptr(), d_out.data_ptr()
        p.workspace, p.workspace_bytes, p.stream = self._samp_ws.data_ptr(), self._samp_ws.numel(), stream
        L.check(lib.b200_sample(C.byref(p)), "b200_sample")
        ids = d_out.cpu().tolist()
        for (i, _), t in zip(items, ids):
            sampled[i] = int(t)

    def _collect_extras(self, batch, rows, events, token_num):
        """output_logits='generation' / logprobs=k: for every token accepted in this step, the fp32 logits of the row it was
        sampled from and/or {token id: log-probability} of the k most likely ids plus the sampled one -- what the
        reference returns (turbomind.py _get_logits / _get_logprobs).  Read from the step's logits buffer (T, one GPU)."""
        row_of = {id(s): r for s, r in zip(batch, rows)}
        lg = None
        for s, tok in events:
            if tok is None or not (s.want_logits or s.want_logprobs):
                continue
            if self.hybrid:
                row = self.last_logits[self.last_rows[row_of[id(s)]]]
            else:
                if lg is None:
                    lg = self.model.logits(token_num)[:, :self.spec.vocab].float()
                row = lg[row_of[id(s)]]
            if s.want_logits:
                s.logits.append(row.cpu())
            if s.want_logprobs:
                lp = torch.log_softmax(row, -1)
                top = torch.topk(lp, min(s.want_logprobs, lp.numel()))
                d = {int(i): float(v) for v, i in zip(top.values.tolist(), top.indices.tolist())}
                d[int(tok)] = float(lp[int(tok)])
                s.logprobs.append(d)

    def serve_follower(self):
        """Tensor-parallel rank > 0: execute the steps the leader publishes until it shuts the channel down.  Every rank
        owns a KV pool of the same geometry, so the leader's block ids are valid here; the sampled ids are the same on
        every rank (vocab-sharded argmax exchange) and are ignored by the followers."""
        while True:
            st = self.channel.receive()
            if st is None:
                return
            self._execute(st)

    def _execute(self, st):
        """Upload one step's arrays, run it on this rank's model shard, return the sampled id of every row."""
        B, T = st["batch_size"], st["token_num"]
        h = self._h_ctl
        h[:T] = st["token_ids"]
        h[self._o_q:self._o_q + B + 1] = st["cu_q_len"]
        h[self._o_k:self._o_k + B + 1] = st["cu_k_len"]
        h[self._o_b:self._o_b + B + 1] = st["cu_block_nums"]
        self.d_ctl.copy_(self.h_ctl, non_blocking=True)
        self.h2d_bytes += self.h_ctl.numel() * 4
        ids = st["block_ids"]
        if ids != self._last_block_ids:          # the block table changes only when a sequence crosses a block boundary
            n = len(ids)
            hp = self._h_block_ptrs[:n]
            hp[:] = ids
            hp *= self.pool.block_bytes
            hp += self.pool.base
            self.d_block_ptrs[:n].copy_(self.h_block_ptrs[:n], non_blocking=True)
            self.h2d_bytes += n * 8
            self._last_block_ids = ids

        def launch():
            self.model.decode_step(batch=B, token_ids=self.d_tokens, cu_q_len=self.d_cu_q, cu_k_len=self.d_cu_k,
                                   block_ptrs=self.d_block_ptrs, cu_block_nums=self.d_cu_blocks, out_tokens=self.d_out,
                                   max_k_len=st["max_k_len"], token_num=T)

        # A pure decode step is shape-static given the batch size (every argument lives in a fixed device buffer, the
        # attention work partition is computed on the device), so its ~300 launches are replayed from a CUDA graph per
        # batch size -- captured the second time that size is seen (the first run doubles as the warm-up).
        if T == B and self._use_graphs:
            g = self._graphs.get(B)
            if g is None and B in self._seen_sizes:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    launch()
                self._graphs[B] = g
            if g is not None:
                g.replay()
            else:
                launch()
                self._seen_sizes.add(B)
        else:
            launch()
        self.h_out.copy_(self.d_out, non_blocking=True)
        self.d2h_bytes += self.h_out.numel() * 4
        torch.cuda.current_stream().synchronize()
        return self._h_out[:T].tolist()

    def close(self):
        """Release tensor-parallel followers (if any) and the communicator."""
        if self.channel is not None and self.channel.is_leader:
            self.channel.shutdown()
        tp = getattr(self, "_tp", None)
        if tp is not None:
            tp.close()
            self._tp = None

    def get_schedule_metrics(self, index=0):
        """ScheduleMetrics of this rank (TurboMind.get_schedule_metrics, lmdeploy/turbomind/turbomind.py)."""
        from ..messages import ScheduleMetrics
        return ScheduleMetrics(**self.scheduler.metrics())

    def new_session_id(self):
        with self._lock:
            self._next_session += 1
            return self._next_session


class TurboMindInstance:
    """Stream tokens for one session.  Same call shape as the reference's
    TurboMindInstance.async_stream_infer(session_id, input_ids, gen_config=...) (turbomind.py:687-813)."""

    def __init__(self, engine: TurboMind):
        self.engine = engine

    def _submit(self, session_id, input_ids, gen_config):
        g = gen_config or GenerationConfig()
        # max_new_tokens = None: until the session is full (the scheduler clamps to session_len), as the reference does
        rope = getattr(getattr(self.engine, "spec", None), "rope", None)
        if rope is not None and rope.dynamic_ntk_base(len(input_ids)) != rope.base:
            raise NotImplementedError(f"a {len(input_ids)}-token prompt exceeds the model's trained context "
                                      f"({rope.max_position_embeddings}); dynamic-NTK rescaling of the rope base per "
                                      "request is not implemented on this path")
        budget = g.max_new_tokens if g.max_new_tokens is not None else 1 << 30
        seq = Sequence(session_id=session_id, prompt=list(map(int, input_ids)), max_new_tokens=budget,
                       stop_token_ids=list(g.stop_token_ids or []), ignore_eos=g.ignore_eos, eos_id=self.engine.eos_id)
        seq.want_logits, seq.want_logprobs = g.output_logits == "generation", int(g.logprobs or 0)
        if g.do_sample and not (g.top_k == 1 and g.repetition_penalty == 1.0):     # top_k == 1 without a penalty IS greedy
            if getattr(self.engine, "channel", None) is not None or self.engine.model.tp_size != 1:
                raise NotImplementedError("do_sample under tensor parallelism (the logits are vocabulary-sharded)")
            seed = g.random_seed if g.random_seed is not None else int.from_bytes(os.urandom(8), "little")
            seq.sampling = dict(temperature=float(g.temperature), top_k=int(g.top_k), top_p=float(g.top_p),
                                min_p=float(g.min_p), repetition_penalty=float(g.repetition_penalty), seed=int(seed))
        if (seq.want_logits or seq.want_logprobs) and getattr(self.engine, "channel", None) is not None:
            raise NotImplementedError("logits / logprobs outputs under tensor parallelism (the logits are vocabulary-sharded)")
        self.engine.scheduler.add(seq)
        return seq

    def open(self, session_id, input_ids, gen_config: GenerationConfig = None):
        """An open-ended request: its input continues (append to the returned Sequence's `prompt` between steps), nothing is
        sampled for it, and it lives until Scheduler.finish(session_id).  Runs through TurboMind.step(plan) like any other."""
        seq = self._submit(session_id, input_ids, gen_config)
        seq.hold = True
        return seq

    def stream_infer(self, session_id, input_ids, gen_config: GenerationConfig = None, **kw):
        try:
            seq = self._submit(session_id, input_ids, gen_config)
        except InputLengthError:
            yield EngineOutput(ResponseType.INPUT_LENGTH_ERROR, [], 0)
            return
        except KeyError:
            yield EngineOutput(ResponseType.SESSION_REPEAT, [], 0)
            return
        # EngineOutput.token_ids = "the newly generated token ids in each iteration" (lmdeploy/messages.py:721-743,
        # turbomind.py async_stream_infer: output_ids_buf[prev_len:seq_len]); a stop token is part of them.  num_token is
        # the running total.
        sent = 0
        while not seq.finished:
            self.engine.step()
            if len(seq.generated) > sent and not seq.finished:
                new, lo, sent = seq.generated[sent:], sent, len(seq.generated)
                yield EngineOutput(ResponseType.SUCCESS, list(new), sent, **self._extras(seq, lo, sent))
        yield EngineOutput(ResponseType.FINISH if seq.finish_reason != "cancel" else ResponseType.CANCEL,
                           list(seq.generated[sent:]), len(seq.generated), **self._extras(seq, sent, len(seq.generated)))

    @staticmethod
    def _extras(seq, lo, hi):
        out = {}
        if seq.want_logprobs:
            out["logprobs"] = seq.logprobs[lo:hi]
        if seq.want_logits and hi > lo:
            out["logits"] = torch.stack(seq.logits[lo:hi])
        return out

    async def async_stream_infer(self, session_id, input_ids, gen_config: GenerationConfig = None, **kw):
        for out in self.stream_infer(session_id, input_ids, gen_config):
            yield out
            await asyncio.sleep(0)

    def cancel(self, session_id):
        self.engine.scheduler.cancel(session_id)


def _per_prompt(gen_config, n):
    if isinstance(gen_config, (list, tuple)):
        if len(gen_config) != n:
            raise ValueError(f"{len(gen_config)} generation configs for {n} prompts")
        return list(gen_config)
    return [gen_config] * n


def _submit_or_reject(inst, engine, prompt, gen_config):
    """A prompt that cannot be admitted becomes a finished Sequence with finish_reason 'error' (the others still run)."""
    try:
        return inst._submit(engine.new_session_id(), prompt, gen_config)
    except InputLengthError as e:
        seq = Sequence(session_id=-1, prompt=list(map(int, prompt)), max_new_tokens=0, stop_token_ids=[], ignore_eos=True,
                       eos_id=None)
        seq.finished, seq.finish_reason, seq.error = True, "error", str(e)
        return seq


def batched_generate(engine, prompts: List[List[int]], gen_config=None):
    """Run a list of token-id prompts to completion with continuous batching; returns the Sequence of every prompt.
    gen_config: one GenerationConfig for all prompts or one per prompt."""
    inst = TurboMindInstance(engine)
    cfgs = _per_prompt(gen_config, len(prompts))
    seqs = [_submit_or_reject(inst, engine, p, g) for p, g in zip(prompts, cfgs)]
    while engine.scheduler.has_work:
        engine.step()
    return seqs


def stream_generate(engine, prompts: List[List[int]], gen_config=None):
    """Continuous batching with per-token delivery: yields (prompt index, Sequence, new token ids) after every engine step
    in which that prompt produced tokens; the last yield of a prompt has Sequence.finished set (it carries the final tokens,
    or an empty list when the prompt ended without producing any in that step -- cancelled, out of KV memory)."""
    inst = TurboMindInstance(engine)
    cfgs = _per_prompt(gen_config, len(prompts))
    seqs = [_submit_or_reject(inst, engine, p, g) for p, g in zip(prompts, cfgs)]
    sent = [0] * len(seqs)
    done = [False] * len(seqs)
    while not all(done):
        if engine.scheduler.has_work:
            engine.step()
        for i, s in enumerate(seqs):
            if done[i]:
                continue
            if len(s.generated) > sent[i]:
                new = s.generated[sent[i]:]
                sent[i] = len(s.generated)
                done[i] = s.finished                 # the chunk that carries the last token is the final one
                yield i, s, list(new)
            elif s.finished:
                done[i] = True
                yield i, s, []
