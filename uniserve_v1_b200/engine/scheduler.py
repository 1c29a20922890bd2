"""Continuous-batching scheduler with chunked prefill, prefix reuse and recompute
preemption, driven by a pluggable policy.

The mechanism mirrors the reference's ``schedule()`` / ``update()`` pair
(crates/engine/src/scheduler/schedule.rs:223, update.rs:130, reference project
paths): requests wait, are admitted in the order the policy dispatches, get
pages from the block manager, run as prefill chunks or one-token decode rows,
commit full pages under chained keys after each call, and are preempted by
recompute when the pool runs dry.  A policy makes the same six decisions as the
reference's ``trait Policy`` (crates/scheduling/src/policy.rs:33-60): ``init``,
``observe``, ``dispatch``, ``preempt``, ``place``, ``limits``; it is a Python
object rather than a wasm program.
"""
from __future__ import annotations

import hashlib

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Optional

from .block_manager import BlockManager
from .types import FinishReason, Request, RequestState, StepOutput


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 128                 # decode rows
    max_num_batched_tokens: int = 8192      # prefill tokens per call
    chunked_prefill_size: int = 8192
    max_prefill_seqs: int = 31
    max_model_len: int = 40960
    page_size: int = 16
    eos_token_id: Optional[int] = None
    decode_lookahead: int = 1               # pages are ensured this many tokens ahead


class Policy:
    """Default ``arrival`` policy: admit by (priority, arrival), preempt the
    latest arrival, place on the only group (reference:
    crates/scheduling/policies/arrival/src/arrival.rs:34-46)."""

    name = "arrival"

    def init(self, config: SchedulerConfig) -> None:
        self.config = config

    def observe(self, event: str, request: Optional[Request] = None, **facts) -> None:
        pass

    def dispatch(self, waiting: list, room: dict) -> list:
        return sorted(waiting, key=lambda r: (-r.priority, r.arrival))

    def preempt(self, running: list) -> Optional[Request]:
        cands = [r for r in running]
        return max(cands, key=lambda r: (-r.priority, r.arrival)) if cands else None

    def place(self, request: Request, groups: list) -> int:
        return 0

    def limits(self) -> dict:
        return {}


@dataclass
class Chunk:
    request: Request
    start: int          # first token index computed in this call
    length: int
    sample: bool        # the call reaches the request's last token


@dataclass
class Batch:
    kind: str                    # "prefill" | "decode"
    chunks: list
    step_id: int = 0

    @property
    def num_tokens(self) -> int:
        return sum(c.length for c in self.chunks)

    def validate(self, page_size: int) -> None:
        """Plain-data checks before any launch (crates/engine/src/batch.rs
        ``Batch::validate``, reference path)."""
        for c in self.chunks:
            need = (c.start + c.length + page_size - 1) // page_size
            if len(c.request.pages) < need:
                raise AssertionError(f"{c.request.request_id}: {len(c.request.pages)} pages < {need}")
            if c.length <= 0 or c.start + c.length > c.request.num_tokens:
                raise AssertionError(f"{c.request.request_id}: bad chunk {c.start}+{c.length}")


class Scheduler:
    def __init__(self, blocks: BlockManager, config: SchedulerConfig,
                 policy: Optional[Policy] = None):
        self.blocks = blocks
        self.config = config
        self.policy = policy or Policy()
        self.policy.init(config)
        self.waiting: deque = deque()
        self.running: list = []
        self.requests: dict = {}
        self.step_id = 0
        self.free_slots = list(range(config.max_num_seqs - 1, -1, -1))
        self.stats = {"preemptions": 0, "prefill_tokens": 0, "decode_tokens": 0,
                      "cached_tokens": 0, "finished": 0, "steps": 0}

    # ------------------------------------------------------------- requests --
    def add_request(self, req: Request) -> None:
        if len(req.prompt_ids) == 0:
            raise ValueError("empty prompt")
        if len(req.prompt_ids) + 1 > self.config.max_model_len:
            raise ValueError(f"prompt of {len(req.prompt_ids)} tokens exceeds max_model_len "
                             f"{self.config.max_model_len}")
        self.requests[req.request_id] = req
        self.waiting.append(req)
        self.policy.observe("arrived", req)

    def abort(self, request_id: str) -> Optional[Request]:
        req = self.requests.get(request_id)
        if req is None or req.finished:
            return None
        self._finish(req, FinishReason.ABORT)
        return req

    def has_work(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    # ------------------------------------------------------------- schedule --
    def _pages_needed(self, req: Request, upto_tokens: int) -> int:
        need = (upto_tokens + self.config.page_size - 1) // self.config.page_size
        return max(0, need - len(req.pages))

    def _admit(self, req: Request) -> bool:
        """Attach: pin the cached prefix, take a slot."""
        if not self.free_slots:
            return False
        if req.num_computed == 0 and not req.pages:
            keys = self.blocks.page_keys(req.all_ids, req.cache_salt)
            # The last token is always computed so its logits exist.
            max_pages = (req.num_tokens - 1) // self.config.page_size
            hit = self.blocks.match_prefix(keys[:max_pages])
            if hasattr(self.blocks, "fetch_prefix"):     # continue in the host tier
                hit = list(hit) + self.blocks.fetch_prefix(keys, len(hit), max_pages)
            req.pages = list(hit)
            req.num_computed = len(hit) * self.config.page_size
            req.committed_pages = len(hit)
            if not req.output_ids:
                req.num_cached = req.num_computed
            self.stats["cached_tokens"] += req.num_computed
        req.slot = self.free_slots.pop()
        req.state = RequestState.RUNNING
        return True

    def _preempt_one(self, protect: Optional[Request] = None) -> bool:
        cands = [r for r in self.running if r is not protect]
        victim = self.policy.preempt(cands)
        if victim is None:
            return False
        self.running.remove(victim)
        self.blocks.release(victim.pages)
        victim.pages = []
        victim.num_computed = 0
        victim.committed_pages = 0
        victim.state = RequestState.PREEMPTED
        victim.preemptions += 1
        if victim.slot >= 0:
            self.free_slots.append(victim.slot)
            victim.slot = -1
        self.waiting.appendleft(victim)
        self.stats["preemptions"] += 1
        self.policy.observe("preempted", victim)
        return True

    def schedule(self) -> Optional[Batch]:
        cfg = self.config
        self.step_id += 1
        # 1. requests still prefilling (chunked) or newly admitted
        budget = min(cfg.max_num_batched_tokens, cfg.chunked_prefill_size)
        chunks: list = []
        prefilling = [r for r in self.running if r.num_computed < r.num_tokens - 1
                      or (not r.output_ids and r.num_computed < r.num_tokens)]
        order = self.policy.dispatch(list(self.waiting),
                                     {"free_pages": self.blocks.num_free, "budget": budget}) \
            if self.waiting else []
        for req in prefilling + order:
            if budget <= 0 or len(chunks) >= cfg.max_prefill_seqs:
                break
            newly = req.state != RequestState.RUNNING
            if newly:
                if len(self.running) >= cfg.max_num_seqs or not self._admit(req):
                    break
            remaining = req.num_tokens - req.num_computed
            take = min(remaining, budget)
            need = self._pages_needed(req, req.num_computed + take)
            pages = self.blocks.allocate(need)
            if pages is None:
                # shrink the chunk to what fits, else give up on admitting more
                free_tok = self.blocks.num_free * cfg.page_size
                room = len(req.pages) * cfg.page_size - req.num_computed + free_tok
                take = min(take, room)
                if take <= 0:
                    if newly:
                        self.free_slots.append(req.slot)
                        req.slot = -1
                        self.blocks.release(req.pages)
                        req.pages, req.num_computed, req.committed_pages = [], 0, 0
                        req.state = RequestState.WAITING
                    break
                pages = self.blocks.allocate(self._pages_needed(req, req.num_computed + take))
                if pages is None:
                    break
            req.pages.extend(pages)
            if newly:
                self.waiting.remove(req)
                self.running.append(req)
                self.policy.observe("admitted", req)
            chunks.append(Chunk(req, req.num_computed, take,
                                req.num_computed + take == req.num_tokens))
            budget -= take
        if chunks:
            self.stats["prefill_tokens"] += sum(c.length for c in chunks)
            b = Batch("prefill", chunks, self.step_id)
            b.validate(cfg.page_size)
            return b
        # 2. decode: one row per running request
        if not self.running:
            return None
        rows = []
        decoding = [r for r in self.running
                    if r.output_ids and r.num_computed == r.num_tokens - 1]
        if not decoding:
            # Only stalled prefills are left: free room by preempting one of them.
            if len(self.running) > 1 and self._preempt_one(protect=self.running[0]):
                return self.schedule()
            raise RuntimeError("KV pool too small for a single request")
        preempted = False
        for req in decoding:
            if preempted and req not in self.running:
                continue          # preempted while making room for an earlier row
            while True:
                need = self._pages_needed(req, req.num_tokens + cfg.decode_lookahead - 1)
                if need == 0:
                    break
                pages = self.blocks.allocate(need)
                if pages is not None:
                    req.pages.extend(pages)
                    break
                preempted = True
                if not self._preempt_one(protect=req):
                    raise RuntimeError("KV pool too small for a single request")
            rows.append(req)
        if preempted:
            rows = [r for r in rows if r in self.running]
        chunks = [Chunk(r, r.num_tokens - 1, 1, True) for r in rows]
        self.stats["decode_tokens"] += len(chunks)
        b = Batch("decode", chunks, self.step_id)
        b.validate(cfg.page_size)
        return b

    # --------------------------------------------------------------- update --
    def _commit_pages(self, req: Request) -> None:
        ps = self.config.page_size
        full = req.num_computed // ps
        if full <= req.committed_pages or not self.blocks.enable_prefix_cache:
            return
        # the request's key chain grows by the pages it filled (tokens only append, so the
        # links computed so far stay valid across preemption and recompute)
        chain = getattr(req, "_chain", None)
        if chain is None:
            chain = req._chain = [self.blocks.chain_seed(req.cache_salt), []]
        keys = chain[1]
        while len(keys) < full:
            i = len(keys)
            chain[0], k = self.blocks.chain_next(chain[0], req.token_slice(i * ps, (i + 1) * ps))
            keys.append(k)
        for i in range(req.committed_pages, full):
            self.blocks.commit(req.pages[i], keys[i])
        ev = self.blocks.kv_events
        if ev is not None:                  # the same pages as KV events for outside routers
            from ..server.export import block_digest
            dig = getattr(req, "_ev_digests", None)
            if dig is None:
                salt = req.cache_salt.encode() if req.cache_salt else None
                dig = req._ev_digests = [hashlib.sha256(salt).digest() if salt else None]
            while len(dig) - 1 < full:
                i = len(dig) - 1
                dig.append(block_digest(dig[-1], req.token_slice(i * ps, (i + 1) * ps)))
            lo = req.committed_pages
            ev.stored(req.pages[lo:full], dig[lo + 1:full + 1], dig[lo],
                      req.token_slice(lo * ps, full * ps))
        req.committed_pages = full

    def _finish(self, req: Request, reason: FinishReason, error: Optional[str] = None) -> None:
        if req in self.running:
            self.running.remove(req)
        if req in self.waiting:
            self.waiting.remove(req)
        self.blocks.release(req.pages)
        req.pages = []
        if req.slot >= 0:
            self.free_slots.append(req.slot)
            req.slot = -1
        req.state = RequestState.FINISHED
        req.finish_reason = reason
        req.error = error
        req.finish_time = time.monotonic()
        self.stats["finished"] += 1
        self.policy.observe("finished", req, reason=reason.value)

    def _stop_reason(self, req: Request, tok: int) -> Optional[FinishReason]:
        p = req.params
        n_out = len(req.output_ids)
        if n_out >= p.min_tokens:
            if not p.ignore_eos and self.config.eos_token_id is not None \
                    and tok == self.config.eos_token_id:
                return FinishReason.STOP
            if tok in p.stop_token_ids:
                return FinishReason.STOP
        if n_out >= p.max_tokens:
            return FinishReason.LENGTH
        if req.num_tokens >= self.config.max_model_len:
            return FinishReason.LENGTH
        return None

    def update(self, batch: Batch, sampled: dict, logprobs: Optional[dict] = None,
               errors: Optional[dict] = None) -> list:
        """Applies one call's output.  ``sampled[request_id]`` is the token drawn
        for chunks with ``sample``; ``errors[request_id]`` fails a row
        (numerical fault) without touching the others."""
        outs = []
        self.stats["steps"] += 1
        for c in batch.chunks:
            req = c.request
            if req.finished:
                continue
            if errors and req.request_id in errors:
                self._finish(req, FinishReason.ERROR, errors[req.request_id])
                outs.append(StepOutput(req.request_id, [], True, FinishReason.ERROR,
                                       error=errors[req.request_id]))
                continue
            req.num_computed = c.start + c.length
            new = []
            reason = None
            if c.sample:
                tok = int(sampled[req.request_id])
                req.output_ids.append(tok)
                if req.first_token_time is None:
                    req.first_token_time = time.monotonic()
                if logprobs and req.request_id in logprobs:
                    req.logprobs.append(logprobs[req.request_id])
                new = [tok]
                reason = self._stop_reason(req, tok)
            self._commit_pages(req)
            if reason is not None:
                self._finish(req, reason)
            outs.append(StepOutput(req.request_id, new, reason is not None, reason,
                                   logprobs=[req.logprobs[-1]] if (new and req.logprobs) else None,
                                   num_cached_tokens=req.num_cached))
        return outs
