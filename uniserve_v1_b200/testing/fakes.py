"""Deterministic fakes of the execution side.

``FakeRunner`` stands in for ``CausalLmRunner``: the token it "samples" for a
request is a pure function of the request's tokens so far, which makes
preemption-by-recompute, migration and chunked prefill checkable exactly: any
path that loses or duplicates a token changes every later token.
"""
from __future__ import annotations

import zlib
from typing import Optional

from ..engine.block_manager import BlockManager
from ..engine.scheduler import Batch, Policy, Scheduler, SchedulerConfig
from ..engine.types import ErrorClass, Request, SamplingParams


def fake_token(ids, vocab: int = 1000) -> int:
    data = b"".join(int(t).to_bytes(4, "little") for t in ids[-64:]) + len(ids).to_bytes(4, "little")
    return zlib.crc32(data) % vocab


class FakeRunner:
    def __init__(self, vocab: int = 1000, fail_on: Optional[set] = None, nan_on: Optional[set] = None):
        self.vocab = vocab
        self.fail_on = fail_on or set()       # step ids that raise (fatal worker failure)
        self.nan_on = nan_on or set()         # request ids whose rows produce an invalid token
        self.calls = []
        self.h2d_bytes = self.d2h_bytes = 0

    def execute(self, batch: Batch):
        self.calls.append((batch.kind, [(c.request.request_id, c.start, c.length) for c in batch.chunks]))
        if batch.step_id in self.fail_on:
            raise RuntimeError("injected worker failure")
        sampled = {}
        for c in batch.chunks:
            if c.sample:
                r = c.request
                assert c.start + c.length == r.num_tokens
                sampled[r.request_id] = -1 if r.request_id in self.nan_on else \
                    fake_token(r.all_ids, self.vocab)
        return sampled, {}


class FakeEngine:
    """Scheduler + block manager + FakeRunner behind the LLMEngine interface."""

    def __init__(self, num_pages=64, page_size=16, max_num_seqs=8, max_model_len=512,
                 max_num_batched_tokens=64, policy: Optional[Policy] = None, vocab=1000,
                 enable_prefix_cache=True, eos_token_id=None, **runner_kw):
        self.blocks = BlockManager(num_pages, page_size, "fake", enable_prefix_cache)
        self.config = SchedulerConfig(max_num_seqs=max_num_seqs,
                                      max_num_batched_tokens=max_num_batched_tokens,
                                      chunked_prefill_size=max_num_batched_tokens,
                                      max_model_len=max_model_len, page_size=page_size,
                                      eos_token_id=eos_token_id)
        self.scheduler = Scheduler(self.blocks, self.config, policy)
        self.runner = FakeRunner(vocab, **runner_kw)
        self.vocab = vocab
        self.failed = None
        self._n = 0

    def add_request(self, prompt_ids, params=None, request_id=None, priority=0, cache_salt=None,
                    output_ids=None):
        rid = request_id or f"r{self._n}"
        self._n += 1
        req = Request(rid, list(prompt_ids), params or SamplingParams(), priority=priority,
                      cache_salt=cache_salt)
        if output_ids:
            req.output_ids = list(output_ids)
        self.scheduler.add_request(req)
        return rid

    def abort(self, rid):
        return self.scheduler.abort(rid) is not None

    def has_work(self):
        return self.scheduler.has_work()

    def step(self):
        batch = self.scheduler.schedule()
        if batch is None:
            return []
        try:
            sampled, lps = self.runner.execute(batch)
        except Exception as e:
            self.failed = f"{ErrorClass.FATAL_WORKER_FAILURE.value}: {e}"
            raise
        errors = {rid: f"{ErrorClass.NUMERICAL_FAULT.value}: sampled token {t}"
                  for rid, t in sampled.items() if t < 0 or t >= self.vocab}
        return self.scheduler.update(batch, sampled, lps, errors)

    def run(self, max_steps=100000):
        outs = []
        for _ in range(max_steps):
            if not self.has_work():
                break
            outs.extend(self.step())
        return outs

    def stats(self):
        s = dict(self.scheduler.stats)
        s.update({"kv": self.blocks.stats(), "running": len(self.scheduler.running),
                  "waiting": len(self.scheduler.waiting)})
        return s


def expected_output(prompt, n, vocab=1000, stop=None):
    ids = list(prompt)
    out = []
    for _ in range(n):
        t = fake_token(ids, vocab)
        ids.append(t)
        out.append(t)
        if stop is not None and t == stop:
            break
    return out
