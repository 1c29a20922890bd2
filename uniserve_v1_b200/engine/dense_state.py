"""An engine for decoders that keep a dense per-sequence state (the hybrid
Qwen3.5 family: key / value rows for its attention layers, convolution window and
delta-rule matrix for its linear layers) instead of KV pages.

Same calls as ``LLMEngine`` - ``add_request`` / ``step`` / ``abort`` / ``has_work`` /
``stats`` - so the HTTP service, the chat layer and the tools run on it unchanged.
One step admits waiting requests up to ``max_num_seqs``, runs the next prompt chunk of
every request still reading its prompt, and one decode position for every other one.
Sampling follows the request's parameters with draws addressed by (seed, position), so
a request produces the same tokens whatever else is running.  Requests that have read
their prompt advance together when the model offers ``decode_batch`` (projections, experts,
the delta rule and the convolution run on all rows at once, attention per sequence);
prompt chunks run one sequence at a time.  Prompts share work through snapshots of the whole
state at interval boundaries (``state_interval``), the recurrent counterpart of prefix pages.

Reference behaviour: crates/engine/src/runner/causal_lm (state slots and
``state_interval`` checkpoints of recurrent layers) - reference project path.
"""
from __future__ import annotations

import copy
import hashlib
import itertools
import time
from collections import OrderedDict
from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import functional as F
from .types import FinishReason, Request, RequestState, SamplingParams, StepOutput


@dataclass
class DenseStateConfig:
    max_num_seqs: int = 8
    max_model_len: int = 4096
    prefill_chunk: int = 512


class _NoPages:
    """The face of a block manager for the admin routes: the prefix cache here holds state
    snapshots, not pages."""

    def __init__(self, engine):
        self._e = engine

    @property
    def enable_prefix_cache(self) -> bool:
        return self._e.enable_prefix_cache

    @enable_prefix_cache.setter
    def enable_prefix_cache(self, on: bool) -> None:
        self._e.enable_prefix_cache = bool(on)

    def flush(self) -> int:
        n = len(self._e.state_cache)
        self._e.state_cache.clear()
        return n


class DenseStateEngine:
    def __init__(self, model, max_num_seqs: int = 8, max_model_len: int = 4096,
                 prefill_chunk: int = 512, tower=None, state_interval: int = 64,
                 state_cache_entries: int = 32):
        self.model = model
        # Prefix cache of recurrent decoders: a snapshot of the whole per-sequence state at
        # every ``state_interval`` tokens of a prompt, keyed by the chained hash of the tokens
        # before it (and the isolation salt).  A later request with the same prefix starts from
        # the longest snapshot instead of reading those tokens again.
        self.state_interval = max(1, int(state_interval))
        self.state_cache_entries = int(state_cache_entries)
        self.state_cache: "OrderedDict[bytes, tuple]" = OrderedDict()
        self.enable_prefix_cache = state_cache_entries > 0
        # with a vision tower requests may carry images: (patch rows, grids) in ``media``
        self.mm = None
        if tower is not None:
            from ..models.qwen3_5 import Qwen35Multimodal
            self.mm = Qwen35Multimodal(model, tower)
        self.config = DenseStateConfig(max_num_seqs, max_model_len, prefill_chunk)
        self.blocks = _NoPages(self)
        self.failed: Optional[str] = None
        self.waiting: list = []
        self.running: list = []
        self.requests: dict = {}
        self.states: dict = {}
        self._ids = itertools.count(1)
        self._stats = {"prefill_tokens": 0, "decode_tokens": 0, "finished": 0, "steps": 0,
                       "preemptions": 0, "cached_tokens": 0}
        self.spec_stats = {"steps": 0, "proposed": 0, "accepted": 0}

    # ------------------------------------------------------------- requests --
    def add_request(self, prompt_ids, params: Optional[SamplingParams] = None,
                    request_id: Optional[str] = None, priority: int = 0,
                    cache_salt: Optional[str] = None, output_ids: Optional[list] = None,
                    media=None) -> str:
        rid = request_id or f"req-{next(self._ids)}"
        V = self.model.cfg.vocab_size
        if not prompt_ids:
            raise ValueError("empty prompt")
        if any((t < 0 or t >= V) for t in prompt_ids):
            raise ValueError("input_error: token id outside the vocabulary")
        if len(prompt_ids) + 1 > self.config.max_model_len:
            raise ValueError(f"prompt of {len(prompt_ids)} tokens exceeds max_model_len "
                             f"{self.config.max_model_len}")
        req = Request(rid, list(prompt_ids), params or SamplingParams(), priority=priority,
                      cache_salt=cache_salt)
        if output_ids:                      # a resumed request recomputes its state
            req.output_ids = list(output_ids)
        if media is not None:
            if self.mm is None:
                raise ValueError("input_error: this deployment does not take images")
            pixels, grids = media
            m = self.mm.tower.cfg.spatial_merge_size
            want = sum(t * (h // m) * (w // m) for t, h, w in grids)
            have = sum(1 for t in prompt_ids if t == self.model.cfg.image_token_id)
            if want != have or pixels.shape[0] != sum(t * h * w for t, h, w in grids):
                raise ValueError("input_error: image placeholders do not match the images")
            req.media = (pixels, [tuple(g) for g in grids])
        self.requests[rid] = req
        self.waiting.append(req)
        return rid

    def abort(self, request_id: str) -> bool:
        req = self.requests.get(request_id)
        if req is None or req.finished:
            return False
        self._finish(req, FinishReason.ABORT)
        return True

    def has_work(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    def _finish(self, req: Request, reason: FinishReason) -> None:
        req.state, req.finish_reason, req.finish_time = RequestState.FINISHED, reason, \
            time.monotonic()
        self.states.pop(req.request_id, None)
        for q in (self.waiting, self.running):
            if req in q:
                q.remove(req)
        self._stats["finished"] += 1

    # ----------------------------------------------------------------- step --
    def _sample(self, req: Request, logits_row: torch.Tensor) -> int:
        p = req.params
        if p.needs_shaping or p.logprobs:
            # penalties, bias, bans, minimum length and log-probabilities: the paged
            # runner's shaping code on this one row (same order, same draw addressing)
            from .runner import CausalLmRunner as ModelRunner

            class _Row:
                eos_token_id = getattr(self.model.cfg, "eos_token_id", None)
                d2h_bytes = 0
            toks, info = ModelRunner._shape_and_sample(_Row(), logits_row.float()[None].contiguous(),
                                                       [req])
            if info and req.request_id in info:
                req.logprobs.append(info[req.request_id])
            return int(toks[0])
        if p.temperature <= 0.0:
            return int(logits_row.argmax())
        dev = logits_row.device
        logits = (logits_row.float() / p.temperature)[None].contiguous()
        tok = F.sample_from_logits(
            logits, torch.tensor([p.top_k if p.top_k and p.top_k > 0 else 0], dtype=torch.int32,
                                 device=dev),
            torch.tensor([p.top_p], dtype=torch.float32, device=dev),
            torch.tensor([getattr(p, "min_p", 0.0) or 0.0], dtype=torch.float32, device=dev),
            torch.tensor([req.seed - (1 << 64) if req.seed >= (1 << 63) else req.seed],
                         dtype=torch.int64, device=dev),
            torch.tensor([req.num_tokens], dtype=torch.int64, device=dev))
        return int(tok[0])

    # ------------------------------------------------------------ prefix states --
    def _prefix_keys(self, req: Request) -> list:
        """Chained keys of the prompt at every multiple of the interval (the last token is
        always read, so its logits exist)."""
        import numpy as np
        iv, ids = self.state_interval, req.prompt_ids
        h = hashlib.sha256(("state\0" + (req.cache_salt or "")).encode()).digest()
        keys = []
        for hi in range(iv, len(ids), iv):
            h = hashlib.sha256(h + np.asarray(ids[hi - iv:hi], dtype="<i4").tobytes()).digest()
            keys.append((hi, h))
        return keys

    def _restore_prefix(self, req: Request) -> None:
        if not self.enable_prefix_cache or getattr(req, "media", None) is not None or \
                req.output_ids:
            return
        req._keys = self._prefix_keys(req)
        for hi, key in reversed(req._keys):
            snap = self.state_cache.get(key)
            if snap is not None:
                self.state_cache.move_to_end(key)
                self.states[req.request_id] = copy.deepcopy(snap)
                req.num_computed = req.num_cached = hi
                self._stats["cached_tokens"] += hi
                return

    def _snapshot(self, req: Request) -> None:
        keys = getattr(req, "_keys", None)
        if not keys or req.num_computed % self.state_interval or \
                req.num_computed > len(req.prompt_ids):
            return
        key = next((k for hi, k in keys if hi == req.num_computed), None)
        if key is None or key in self.state_cache:
            return
        self.state_cache[key] = copy.deepcopy(self.states[req.request_id])
        while len(self.state_cache) > self.state_cache_entries:
            self.state_cache.popitem(last=False)

    def _forward_media(self, req: Request, chunk: torch.Tensor, st: list, n: int):
        """A chunk of a request with images: vision rows stand at the placeholder tokens and
        positions are the three-axis ones; tokens after the prompt continue on all axes."""
        from ..models.qwen3_5 import mrope_positions
        from ..models.qwen3_vl_vision import splice
        cfg = self.model.cfg
        if not hasattr(req, "_mm"):
            pixels, grids = req.media
            ids = torch.tensor(req.prompt_ids, device=self.model.device)
            rows, deep = self.mm.tower.forward(pixels, grids)
            emb = splice(self.model.w["embed"][ids.long()], ids, cfg.image_token_id, rows)
            pos3, nxt = mrope_positions(req.prompt_ids, cfg.image_token_id, grids,
                                        self.mm.tower.cfg.spatial_merge_size)
            at = (ids == cfg.image_token_id).nonzero(as_tuple=True)[0]
            req._mm = (emb, pos3, nxt - len(req.prompt_ids), at, deep)
        emb, pos3, delta, at, deep = req._mm
        lo, hi, P = req.num_computed, req.num_computed + n, len(req.prompt_ids)
        e = self.model.w["embed"][chunk.long()]
        p = (torch.arange(lo, hi) + delta)[None].expand(3, -1).clone()
        if lo < P:
            k = min(hi, P) - lo
            e = torch.cat([emb[lo:lo + k], e[k:]], 0)
            p[:, :k] = pos3[:, lo:lo + k]
        ds = None
        if deep:                                  # deep-stack rows of the image positions in [lo, hi)
            sel = ((at >= lo) & (at < hi)).nonzero(as_tuple=True)[0]
            ds = (at[sel] - lo, [d[sel] for d in deep])
        return self.model.forward(chunk, st, lo, embeds=e, positions3=p, deepstack=ds)

    def _stop(self, req: Request, tok: int) -> Optional[FinishReason]:
        p = req.params
        if not p.ignore_eos and tok == getattr(self.model.cfg, "eos_token_id", -1):
            return FinishReason.STOP
        if tok in (getattr(p, "stop_token_ids", None) or ()):
            return FinishReason.STOP
        if len(req.output_ids) >= p.max_tokens or req.num_tokens >= self.config.max_model_len:
            return FinishReason.LENGTH
        return None

    def step(self) -> list:
        while self.waiting and len(self.running) < self.config.max_num_seqs:
            req = self.waiting.pop(0)
            req.state = RequestState.RUNNING
            self.states[req.request_id] = self.model.new_state()
            self._restore_prefix(req)
            self.running.append(req)
        outs = []
        self._stats["steps"] += 1
        dev = self.model.device
        # requests that have read their prompt advance together: one batched decode step
        batched = {}
        if hasattr(self.model, "decode_batch"):
            rows = [r for r in self.running if r.output_ids and
                    r.num_computed == r.num_tokens - 1]
            if len(rows) >= 2:
                toks = torch.tensor([r.output_ids[-1] for r in rows], device=dev)
                pos = torch.tensor([r.num_computed + (r._mm[2] if hasattr(r, "_mm") else 0)
                                    for r in rows])
                logits = self.model.decode_batch(toks, [self.states[r.request_id] for r in rows],
                                                 pos[None].expand(3, -1))
                for i, r in enumerate(rows):
                    batched[r.request_id] = logits[i:i + 1]
        for req in list(self.running):
            st = self.states[req.request_id]
            ids = req.all_ids
            todo = len(ids) - req.num_computed
            n = min(todo, self.config.prefill_chunk)
            if n > 1 and getattr(req, "_keys", None):
                # chunks end on snapshot boundaries while the prompt is being read
                iv = self.state_interval
                edge = (req.num_computed // iv + 1) * iv
                span = max(iv, (self.config.prefill_chunk // iv) * iv)
                n = min(n, edge - req.num_computed + span - iv)
            chunk = torch.tensor(ids[req.num_computed:req.num_computed + n], device=dev)
            if req.request_id in batched:
                logits = batched[req.request_id]
            elif getattr(req, "media", None) is not None:
                logits = self._forward_media(req, chunk, st, n)
            else:
                logits = self.model.forward(chunk, st, req.num_computed)
            req.num_computed += n
            self._snapshot(req)
            self._stats["decode_tokens" if (n == 1 and req.output_ids) else "prefill_tokens"] += n
            if req.num_computed < len(ids):
                continue                    # still reading its prompt
            p_lp = bool(req.params.logprobs)
            tok = self._sample(req, logits[-1])
            if req.first_token_time is None:
                req.first_token_time = time.monotonic()
            req.output_ids.append(tok)
            reason = self._stop(req, tok)
            if reason is not None:
                self._finish(req, reason)
            outs.append(StepOutput(req.request_id, [tok], reason is not None, reason,
                                   num_cached_tokens=req.num_cached,
                                   logprobs=[req.logprobs[-1]] if (p_lp and req.logprobs) else None))
        return outs

    # ------------------------------------------------------------ speculation --
    def speculative_step(self, drafter) -> list:
        """A step with speculation for recurrent decoders: when every running request decodes
        greedily (no images), each gets the drafter's proposal verified in one call over its
        last token plus the drafts.  Keys and values of rejected positions could simply be cut,
        but the recurrent layers cannot step back: the state is snapshotted before the call and,
        on a rejection, restored and advanced again over the accepted tokens only."""
        from .speculation import accept
        rows = [r for r in self.running if r.output_ids and r.num_computed == r.num_tokens - 1]
        if not rows or len(rows) != len(self.running) or self.waiting or \
                any(r.params.temperature > 0.0 or r.params.needs_shaping or r.params.logprobs or
                    getattr(r, "media", None) is not None for r in rows):
            return self.step()
        self._stats["steps"] += 1
        outs, dev = [], self.model.device
        for req in rows:
            room = min(self.config.max_model_len - req.num_tokens - 1,
                       req.params.max_tokens - len(req.output_ids) - 1)
            st = self.states[req.request_id]
            # a drafter that keeps its own cache in the request's state reads it from there
            d = drafter.propose_from_state(req.all_ids, st) \
                if hasattr(drafter, "propose_from_state") else drafter.propose(req.all_ids)
            d = [int(t) for t in d][:max(0, min(drafter.k, room))]
            keep = copy.deepcopy(st) if d else None
            toks = [req.output_ids[-1]] + d
            logits = self.model.forward(torch.tensor(toks, device=dev), st, req.num_computed)
            emit = accept(d, logits.argmax(-1).tolist())
            self.spec_stats["steps"] += 1
            self.spec_stats["proposed"] += len(d)
            self.spec_stats["accepted"] += len(emit) - 1
            if len(emit) - 1 < len(d):             # a draft was refused: replay the accepted part
                st = self.states[req.request_id] = keep
                self.model.forward(torch.tensor(toks[:len(emit)], device=dev), st, req.num_computed)
            self._stats["decode_tokens"] += len(emit)
            new = []
            for tok in emit:
                req.num_computed += 1
                req.output_ids.append(tok)
                new.append(tok)
                reason = self._stop(req, tok)
                if reason is not None:
                    break
            if reason is not None:
                self._finish(req, reason)
            outs.append(StepOutput(req.request_id, new, reason is not None, reason,
                                   num_cached_tokens=req.num_cached))
        return outs

    def generate(self, prompts: list, params=None) -> list:
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        rids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while self.has_work():
            self.step()
        return [self.requests[r].output_ids for r in rids]

    def stats(self) -> dict:
        s = dict(self._stats)
        held = sum(1 for _ in self.states)
        s.update({"kv": {"pages": self.config.max_num_seqs, "free": self.config.max_num_seqs - held,
                         "cached": 0, "hits": 0, "lookups": 0, "evictions": 0},
                  "running": len(self.running), "waiting": len(self.waiting)})
        return s
