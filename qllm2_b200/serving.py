"""Continuous-batching decode (greedy or sampled) on a pool of per-sequence PAM state slots.

The reference decodes one batch with a single `step_offset` for all rows (v11/model.py:785,
1206-1245), so sequences of different lengths cannot share a step.  Here every live sequence owns
a slot of a preallocated state pool `[n_slots, L, K, H, d, d, 2]`; a decode step gathers nothing
and reallocates nothing -- `qpam_decode_step` updates the slots named by `slot_ids` in place, with
per-sequence RoPE positions.  New sequences are prefetched in one packed ragged prefill
(`cu_seqlens`), their final states are written into free slots, and they join the next step.

`SlotScheduler` is pure host logic (no GPU) and is unit-tested on CPU.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

import torch

from . import _lib, ops
from .fused_forward import FusedForward
from .model import V11LM


# ------------------------------------------------------------------------------------ scheduler
@dataclass
class Request:
    rid: int
    prompt: List[int]
    max_new_tokens: int
    generated: List[int] = field(default_factory=list)
    slot: int = -1
    prefilled: int = 0          # prompt tokens already absorbed into the slot's state

    @property
    def prefilling(self) -> bool:
        return self.prefilled < len(self.prompt)

    @property
    def position(self) -> int:
        """Absolute position of the next token to be fed (prompt length + tokens generated so far - 1)."""
        return len(self.prompt) + len(self.generated) - 1

    @property
    def done(self) -> bool:
        return len(self.generated) >= self.max_new_tokens


class SlotScheduler:
    """Admission and retirement of sequences over a fixed number of state slots."""

    def __init__(self, n_slots: int, max_prefill_tokens: int = 1 << 17, chunked_prefill: bool = False):
        """chunked_prefill=True lets a prompt be absorbed in pieces of at most `max_prefill_tokens` per engine
        step (the next piece starts from the state the previous one left in the slot), so one long prompt
        cannot stall the decode steps of the other sequences; False admits whole prompts only."""
        if n_slots <= 0:
            raise ValueError("n_slots must be positive")
        if max_prefill_tokens <= 0:
            raise ValueError("max_prefill_tokens must be positive")
        self.n_slots = n_slots
        self.max_prefill_tokens = max_prefill_tokens
        self.chunked_prefill = chunked_prefill
        self.free: Deque[int] = deque(range(n_slots))
        self.waiting: Deque[Request] = deque()
        self.live: Dict[int, Request] = {}       # slot -> request
        self.finished: List[Request] = []
        self._next_id = 0

    def submit(self, prompt: Sequence[int], max_new_tokens: int) -> int:
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        rid = self._next_id
        self._next_id += 1
        self.waiting.append(Request(rid, list(prompt), max_new_tokens))
        return rid

    def admit(self) -> List[Request]:
        """Move waiting requests into free slots (FIFO), bounded by slots and a prefill token budget."""
        batch, tokens = [], 0
        while self.waiting and self.free:
            nxt = self.waiting[0]
            if batch and tokens + len(nxt.prompt) > self.max_prefill_tokens:
                break
            self.waiting.popleft()
            nxt.slot = self.free.popleft()
            self.live[nxt.slot] = nxt
            batch.append(nxt)
            tokens += len(nxt.prompt)
        return batch

    def plan_prefill(self):
        """Prefill work of one engine step as (request, first prompt token, token count) items.  Whole prompts
        when `chunked_prefill` is off; otherwise sequences already in a slot continue first, then waiting ones
        are admitted, all within the token budget (a piece may end mid-prompt)."""
        if not self.chunked_prefill:
            return [(r, 0, len(r.prompt)) for r in self.admit()]
        items, budget = [], self.max_prefill_tokens
        for r in self.live_requests():
            if r.prefilling and budget > 0:
                take = min(len(r.prompt) - r.prefilled, budget)
                items.append((r, r.prefilled, take))
                budget -= take
        while self.waiting and self.free and budget > 0:
            r = self.waiting.popleft()
            r.slot = self.free.popleft()
            self.live[r.slot] = r
            take = min(len(r.prompt), budget)
            items.append((r, 0, take))
            budget -= take
        return items

    def retire_finished(self) -> List[Request]:
        out = [r for r in self.live.values() if r.done]
        for r in out:
            del self.live[r.slot]
            self.free.append(r.slot)
            self.finished.append(r)
        return out

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.live

    def live_requests(self) -> List[Request]:
        return [self.live[s] for s in sorted(self.live)]


# ------------------------------------------------------------------------------------ engine
class _PrefillMix:
    """Sequence mixing at prefill: the packed ragged scan; final states go to the sequences' slots."""
    q_scale = 1.0     # the scan applies head_dim^-0.5 itself

    def __init__(self, eng, cu, slots, s0_of=None):
        self.eng, self.cu, self.slots, self.s0_of = eng, cu, slots, s0_of

    def __call__(self, layer, q, k, v, gamma, coef):
        y, s = ops.pam_scan_tokens(q, k, v, gamma, coef=coef, cu_seqlens=self.cu, head_dim=q.shape[3],
                                   s0=None if self.s0_of is None else self.s0_of(layer))
        ops.pam_pool_store(self.eng.pool, self.slots, s, layer=layer)
        return y.view(q.shape[2], -1)


class _DecodeMix:
    """Sequence mixing at decode: one recurrent step in place on the slots of the live sequences."""

    def __init__(self, eng, slots):
        self.eng, self.slots = eng, slots
        self.q_scale = eng.model.config.head_dim ** -0.5

    def __call__(self, layer, q, k, v, gamma, coef):
        n, H, _, d, _ = q.shape
        K = gamma.shape[0]
        y = ops.pam_decode_step(self.eng.pool, self.slots, q.view(n, H, d, 2), k.view(n, H, d, 2), v.view(n, H, d, 2),
                                gamma.view(K, n, H), None if coef is None else coef.view(K, n, H, 2), layer=layer)
        return y.view(n, -1)


class ContinuousBatcher:
    """Greedy decode of many sequences through a V11LM with continuous batching."""

    def __init__(self, model: V11LM, n_slots: int, state_dtype: Optional[torch.dtype] = None,
                 max_prefill_tokens: int = 1 << 17, cuda_graph: bool = False, max_position: int = 8192,
                 fused: bool = True, chunked_prefill: bool = False, sampling: Optional[dict] = None):
        """cuda_graph=True captures the decode step once for a full batch of n_slots rows (idle rows carry
        slot id -1, which the step kernel skips) and replays it every step: the per-token cost is then the
        kernels', not the launches' of the Python layer loop.  fused=True runs the blocks through
        `FusedForward` (packed weights, ~10 launches per layer) when the configuration allows it;
        fused=False keeps the module path (`V11Block` operators).  chunked_prefill=True absorbs prompts in
        pieces of at most max_prefill_tokens per step, each piece scanned from the state its predecessor left in
        the slot (the streaming use of the reference's stateful forward, v11/duplex/infer_stream.py:101-102).
        sampling=dict(temperature=, top_k=, top_p=, repetition_penalty=) draws every token with the reference's
        sampling block (v11/model.py:1221-1244) as one kernel inside the step -- the token history of every slot
        lives on the device and the kernel appends to it, so a captured step needs no host data; None (or a
        temperature <= 0) decodes greedily."""
        self.model = model.eval()
        cfg = model.config
        p = next(model.parameters())
        self.device, self.dtype = p.device, p.dtype
        self.state_dtype = state_dtype or (torch.float32 if p.dtype == torch.float32 else torch.bfloat16)
        self.pool = torch.zeros(n_slots, cfg.n_layers, cfg.n_states, cfg.n_heads, cfg.head_dim, cfg.head_dim, 2,
                                dtype=self.state_dtype, device=self.device)
        self.sched = SlotScheduler(n_slots, max_prefill_tokens, chunked_prefill=chunked_prefill)
        self.steps = 0
        self.decoded_tokens = 0
        self.n_slots = n_slots
        self.cuda_graph = cuda_graph
        self._graph = None
        self.max_position = max_position
        self.ff = FusedForward(model, max_position) if fused and FusedForward.unsupported_reason(model) is None else None
        self._ensure_rope(max_position)    # tables must not grow while a captured graph reads them
        self.sampling = None
        if sampling is not None and float(sampling.get("temperature", 1.0)) > 0:
            self.sampling = dict(temperature=float(sampling.get("temperature", 1.0)), top_k=int(sampling.get("top_k", 0)),
                                 top_p=float(sampling.get("top_p", 0.0)),
                                 repetition_penalty=float(sampling.get("repetition_penalty", 1.0)))
            self._hist = torch.zeros(n_slots, max_position + 1, dtype=torch.long, device=self.device)
            self._hist_len = torch.zeros(n_slots, dtype=torch.int32, device=self.device)
        if cuda_graph:
            self._g_ids = torch.zeros(n_slots, 1, dtype=torch.long, device=self.device)
            self._g_pos = torch.zeros(n_slots, 1, dtype=torch.long, device=self.device)
            self._g_slots = torch.full((n_slots,), -1, dtype=torch.int32, device=self.device)
            self._g_out = None

    def submit(self, prompt, max_new_tokens):
        return self.sched.submit([int(t) for t in prompt], max_new_tokens)

    def _ensure_rope(self, need: int):
        """Rotary tables must cover every position before a step that cannot look at its positions on the host."""
        if self.ff is not None:
            if need > self.max_position:
                raise RuntimeError(f"position {need - 1} is beyond max_position={self.max_position} of this batcher")
            return
        from .model import build_rope_cache
        for blk in self.model.blocks:
            if blk.pam.use_rope and blk.pam.rope_cache.shape[0] < need:
                if self._graph is not None:
                    raise RuntimeError(f"position {need - 1} is beyond max_position of the captured decode step")
                blk.pam.register_buffer("rope_cache", build_rope_cache(max(need, 2 * blk.pam.rope_cache.shape[0]), blk.pam.head_dim).to(self.device),
                                        persistent=False)

    def _pick(self, lm_rows, slots):
        """Next token of every row from its head hidden state lm_rows [n, D, 2]: arg-max of the tied head, or one
        draw of the sampling kernel (which also appends the token to the slot's history)."""
        if self.sampling is None:
            return self.ff.greedy_next(lm_rows) if self.ff is not None else self.model.greedy_next(lm_rows)
        if self.ff is not None:
            # logits in the model's dtype, as the reference forms them before its .float(); the kernel widens them
            Hm = torch.cat([lm_rows[..., 0], lm_rows[..., 1]], dim=-1)
            logits = (ops.head_logits(Hm, self.ff.w_vocab) if Hm.dtype == torch.bfloat16
                      else torch.nn.functional.linear(Hm, self.ff.w_vocab))
        else:
            Hm, W = self.model.tied_head_matrices(lm_rows.unsqueeze(1))
            logits = (Hm @ W.to(Hm.dtype).T).float()
        return ops.sample_logits(logits, history=self._hist, hist_len=self._hist_len, slot_ids=slots, append=True,
                                 **self.sampling)

    @torch.no_grad()
    def _prefill(self, items):
        """items: (request, first prompt token, token count).  A piece that starts mid-prompt is scanned from the
        state its predecessor left in the slot; a request emits its first token when its last piece is done."""
        lens = [take for _, _, take in items]
        self._ensure_rope(max(st + take for _, st, take in items))
        # token ids and positions are assembled on the host and copied once each
        ids = torch.cat([torch.as_tensor(r.prompt[st:st + take], dtype=torch.long) for r, st, take in items]).to(self.device)[None]
        positions = torch.cat([torch.arange(st, st + take) for _, st, take in items]).to(self.device)[None]
        cu = torch.zeros(len(items) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(lens).cumsum(0).int()
        cu = cu.to(self.device)
        slots = torch.tensor([r.slot for r, _, _ in items], dtype=torch.int32, device=self.device)
        s0_of = None
        if any(st > 0 for _, st, _ in items):
            resumed = torch.tensor([1.0 if st > 0 else 0.0 for _, st, _ in items], device=self.device)

            def s0_of(layer):      # [K,S,H,d,d,2] float32; fresh sequences start from zero whatever the slot held
                s = self.pool[slots.long(), layer].float() * resumed[:, None, None, None, None, None]
                return s.permute(1, 0, 2, 3, 4, 5).contiguous()
        if self.sampling is not None:      # the penalty looks at the whole prompt: load the slots' histories
            for r, st, take in items:
                self._hist[r.slot, st:st + take] = torch.as_tensor(r.prompt[st:st + take], dtype=torch.long).to(self.device)
            self._hist_len[slots.long()] = torch.tensor([st + take for _, st, take in items], dtype=torch.int32, device=self.device)
            # a piece that ends mid-prompt draws nothing: its row is padded out (slot -1)
            pick_slots = torch.tensor([r.slot if st + take == len(r.prompt) else -1 for r, st, take in items],
                                      dtype=torch.int32, device=self.device)
        else:
            pick_slots = slots
        if self.ff is not None:
            xn = self.ff.hidden(ids, _PrefillMix(self, cu, slots, s0_of), positions=positions)
            nxt = self._pick(self.ff.head_hidden(xn[(cu[1:] - 1).long()]), pick_slots)
        else:
            nxt = self._prefill_modules(ids, positions, cu, slots, s0_of, pick_slots)
        for (r, st, take), t in zip(items, nxt.tolist()):
            r.prefilled = st + take
            if not r.prefilling:
                r.generated.append(int(t))

    def _prefill_modules(self, ids, positions, cu, slots, s0_of=None, pick_slots=None):
        m = self.model
        z = m.embed_norm(m.embed(ids))
        for li, blk in enumerate(m.blocks):
            z = z + blk.cgu(blk.norm1(z)) * blk.cgu_scale
            xn = blk.norm2(z)
            pam = blk.pam
            q, k, vprime, gamma, coef = pam.project_gated(xn, positions=positions)
            y, s = ops.pam_scan(q, k, vprime, gamma, coef=coef, cu_seqlens=cu, head_dim=pam.head_dim,
                                s0=None if s0_of is None else s0_of(li))
            ops.pam_pool_store(self.pool, slots, s, layer=li)
            out = pam.o_proj(y.transpose(1, 2).contiguous().view(1, ids.shape[1], pam.inner_dim, 2))
            z = z + out * blk.pam_scale
        last = (cu[1:] - 1).long()
        lm = m._head_hidden(z[:, last])                                     # [1, n, D, 2]
        return self._pick(lm[0], slots if pick_slots is None else pick_slots)

    @torch.no_grad()
    def warmup(self):
        """Capture the decode step now (cuda_graph=True) instead of at the first decode step: a warm-up run on
        idle rows only (slot id -1, no state changes), then the capture, which records and does not execute."""
        if not self.cuda_graph or self._graph is not None:
            return
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._decode_tensors(self._g_ids, self._g_pos, torch.full_like(self._g_slots, -1))
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._g_out = self._decode_tensors(self._g_ids, self._g_pos, self._g_slots)
        self._graph = graph

    @torch.no_grad()
    def _decode(self, live: List[Request]):
        n = len(live)
        self._ensure_rope(max(r.position for r in live) + 1)
        ids = torch.tensor([r.generated[-1] for r in live], dtype=torch.long)
        positions = torch.tensor([r.position for r in live], dtype=torch.long)
        slots = torch.tensor([r.slot for r in live], dtype=torch.int32)
        if self.cuda_graph:
            self._g_ids.zero_()
            self._g_pos.zero_()
            self._g_slots.fill_(-1)
            self._g_ids[:n, 0] = ids.to(self.device)
            self._g_pos[:n, 0] = positions.to(self.device)
            self._g_slots[:n] = slots.to(self.device)
            self.warmup()
            self._graph.replay()
            nxt = self._g_out[:n]
        else:
            nxt = self._decode_tensors(ids.to(self.device)[:, None], positions.to(self.device)[:, None],
                                       slots.to(self.device))
        for r, t in zip(live, nxt.tolist()):
            r.generated.append(int(t))
        self.decoded_tokens += n

    @torch.no_grad()
    def _decode_tensors(self, ids, positions, slots):
        """One decode step for rows (ids [n,1], positions [n,1], slots [n]); returns next ids [n]."""
        if self.ff is not None:
            xn = self.ff.hidden(ids, _DecodeMix(self, slots), positions=positions)
            return self._pick(self.ff.head_hidden(xn), slots)
        m = self.model
        n = ids.shape[0]
        z = m.embed_norm(m.embed(ids))                                      # [n,1,D,2]
        for li, blk in enumerate(m.blocks):
            z = z + blk.cgu(blk.norm1(z)) * blk.cgu_scale
            xn = blk.norm2(z)
            pam = blk.pam
            q, k, vprime, gamma, coef = pam.project_gated(xn, positions=positions)   # gamma [K,n,H,1]
            y = ops.pam_decode_step(self.pool, slots, (q[:, :, 0] * pam.head_dim ** -0.5).contiguous(),
                                    k[:, :, 0].contiguous(), vprime[:, :, 0].contiguous(),
                                    gamma[..., 0].contiguous(), None if coef is None else coef[:, :, :, 0].contiguous(),
                                    layer=li)
            out = pam.o_proj(y.reshape(n, 1, pam.inner_dim, 2))
            z = z + out * blk.pam_scale
        return self._pick(m._head_hidden(z)[:, 0], slots)

    # ---------------------------------------------------------------- live sessions
    def export_session(self, rid: int, remove: bool = True) -> dict:
        """Everything needed to continue request `rid` later or elsewhere: its prompt and generated tokens, its
        budget and its recurrent state, the slot's [L, K, H, d, d, 2] block of the pool, as host tensors (the
        state is what the reference carries between `forward(..., states=)` calls, v11/model.py:785-841).  Only
        a sequence that has finished its prefill and is not done can be exported; `remove=True` frees the slot."""
        req = next((r for r in self.sched.live.values() if r.rid == rid), None)
        if req is None or req.prefilling or req.done:
            raise KeyError(f"request {rid} is not a live, prefilled, unfinished sequence")
        torch.cuda.current_stream().synchronize()
        blob = {"prompt": list(req.prompt), "generated": list(req.generated), "max_new_tokens": req.max_new_tokens,
                "state": self.pool[req.slot].cpu(), "state_dtype": str(self.state_dtype).replace("torch.", ""),
                "shape": tuple(self.pool.shape[1:])}
        if remove:
            del self.sched.live[req.slot]
            self.sched.free.append(req.slot)
        return blob

    def import_session(self, blob: dict, max_new_tokens: Optional[int] = None) -> int:
        """Continue an exported sequence in a free slot of this engine (same model shape); returns its new request
        id.  The state is copied into the pool (converted to the pool's dtype), the token history into the
        sampler's, and the sequence joins the next decode step."""
        if tuple(blob["shape"]) != tuple(self.pool.shape[1:]):
            raise ValueError(f"session state {tuple(blob['shape'])} does not fit this pool {tuple(self.pool.shape[1:])}")
        if not self.sched.free:
            raise RuntimeError("no free slot for the imported session")
        slot = self.sched.free.popleft()
        rid = self.sched._next_id
        self.sched._next_id += 1
        req = Request(rid, list(blob["prompt"]), int(max_new_tokens or blob["max_new_tokens"]), list(blob["generated"]), slot,
                      len(blob["prompt"]))
        self._ensure_rope(req.position + 1)
        self.pool[slot].copy_(blob["state"].to(self.device, self.pool.dtype))
        if self.sampling is not None:
            toks = torch.as_tensor(req.prompt + req.generated, dtype=torch.long)
            self._hist[slot, :toks.numel()] = toks.to(self.device)
            self._hist_len[slot] = toks.numel()
        self.sched.live[slot] = req
        return rid

    def step(self) -> int:
        """Admit + prefill waiting sequences, then advance every live sequence by one token."""
        self.sched.retire_finished()
        live_before = [r for r in self.sched.live_requests() if not r.done and not r.prefilling]
        batch = self.sched.plan_prefill()
        if batch:
            self._prefill(batch)
        if live_before:
            self._decode(live_before)
        self.sched.retire_finished()
        self.steps += 1
        if self.steps % 64 == 0:
            # the host has just read this step's tokens, so the device is idle: a cheap point to learn of a kernel that
            # gave up on a wait (its outputs, and every token since, would be invalid)
            _lib.raise_on_device_error("ContinuousBatcher.step")
        return len(live_before) + len(batch)

    def run(self) -> Dict[int, List[int]]:
        while not self.sched.idle:
            self.step()
        _lib.raise_on_device_error("ContinuousBatcher.run")
        return {r.rid: r.generated for r in self.sched.finished}


# ------------------------------------------------------------------------------------ V11LM.generate
class _BatchPrefillMix:
    """Sequence mixing at the prefill of `generate`: B equal-length rows, final states into slots 0..B-1."""
    q_scale = 1.0

    def __init__(self, pool, slots):
        self.pool, self.slots = pool, slots

    def __call__(self, layer, q, k, v, gamma, coef):
        y, s = ops.pam_scan_tokens(q, k, v, gamma, coef=coef, head_dim=q.shape[3])
        ops.pam_pool_store(self.pool, self.slots, s, layer=layer)
        return y.view(q.shape[0] * q.shape[2], -1)


class _PoolDecodeMix:
    def __init__(self, pool, slots, head_dim):
        self.pool, self.slots, self.q_scale = pool, slots, head_dim ** -0.5

    def __call__(self, layer, q, k, v, gamma, coef):
        n, H, _, d, _ = q.shape
        K = gamma.shape[0]
        y = ops.pam_decode_step(self.pool, self.slots, q.view(n, H, d, 2), k.view(n, H, d, 2), v.view(n, H, d, 2),
                                gamma.view(K, n, H), None if coef is None else coef.view(K, n, H, 2), layer=layer)
        return y.view(n, -1)


def _fused_forward_of(model: V11LM, need_positions: int) -> FusedForward:
    """The model's packed forward, rebuilt when a parameter changed or longer positions are needed."""
    key = (tuple(p._version for p in model.parameters()), next(model.parameters()).dtype, next(model.parameters()).device)
    cached = getattr(model, "_fused_forward_cache", None)
    if cached is not None and cached[0] == key and (cached[1].rope is None or cached[1].rope.shape[0] >= need_positions):
        return cached[1]
    ff = FusedForward(model, max_position=max(need_positions, 2 * model.config.max_seq_len))
    model._fused_forward_cache = (key, ff)
    return ff


@torch.no_grad()
def generate_fused(model: V11LM, input_ids, max_new_tokens, sample, eos_token_id=None):
    """`V11LM.generate` on the packed forward: one parallel prefill, then per token one decode step replayed
    from a CUDA graph (layer loop of v11/model.py:1206-1245).  `sample(logits [B,V] float32 or None, out) -> next
    ids [B,1]` picks the tokens; it gets None when it declared `sample.greedy` (arg-max without logits)."""
    cfg = model.config
    B, T0 = input_ids.shape
    ff = _fused_forward_of(model, T0 + max_new_tokens + 1)
    dev = input_ids.device
    state_dtype = torch.float32 if ff.dtype == torch.float32 else torch.bfloat16
    pool = torch.zeros(B, cfg.n_layers, cfg.n_states, cfg.n_heads, cfg.head_dim, cfg.head_dim, 2, dtype=state_dtype, device=dev)
    slots = torch.arange(B, dtype=torch.int32, device=dev)
    greedy = getattr(sample, "greedy", False)

    def head(xn_rows):
        lm = ff.head_hidden(xn_rows)
        return ff.greedy_next(lm)[:, None] if greedy else ff.logits(lm)

    out = input_ids.clone()
    xn = ff.hidden(out, _BatchPrefillMix(pool, slots))
    res = head(xn.view(B, T0, cfg.dim, 2)[:, -1])
    ids_buf = torch.zeros(B, 1, dtype=torch.long, device=dev)
    pos_buf = torch.zeros(B, 1, dtype=torch.long, device=dev)
    mix = _PoolDecodeMix(pool, slots, cfg.head_dim)
    graph, g_res = None, None
    done = torch.zeros(B, dtype=torch.bool, device=dev)
    for i in range(max_new_tokens):
        nxt = res if greedy else sample(res, out)
        out = torch.cat([out, nxt], dim=1)
        if eos_token_id is not None:
            done |= nxt.squeeze(1) == eos_token_id
            if bool(done.all()):
                break
        if i + 1 == max_new_tokens:
            break
        ids_buf.copy_(nxt)
        pos_buf.fill_(T0 + i)
        if graph is None and i == 0:
            res = head(ff.hidden(ids_buf, mix, positions=pos_buf))          # first step eagerly (warms every kernel up)
        elif graph is None:
            graph = torch.cuda.CUDAGraph()                                  # capture records the step, it does not run it
            with torch.cuda.graph(graph):
                g_res = head(ff.hidden(ids_buf, mix, positions=pos_buf))
            graph.replay()
            res = g_res.clone()
        else:
            graph.replay()
            res = g_res.clone()
    return out
