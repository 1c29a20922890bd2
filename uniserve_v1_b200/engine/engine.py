"""The token engine: scheduler + block manager + runner behind one object.

``LLMEngine.generate`` is the public batch API (what ``bench.py`` times end to
end); the HTTP layer drives ``add_request`` / ``step`` from its engine loop.
One engine drives the GPU(s) of one replica; with a tensor/expert group every
rank runs the same engine in lock step (rank 0's schedule is the schedule:
all ranks see the same requests in the same order, so their schedulers agree).

Reference behaviour: crates/engine/src/scheduler/mod.rs:796-1065 (run/step),
crates/engine/src/worker.rs:1587 (worker loop), docs/architecture.md:128
(two-turn steps) — reference project paths.
"""
from __future__ import annotations

import os

import itertools
import time
import weakref
from typing import Optional

import torch

from ..models.qwen3_moe import Qwen3MoeModel
from .block_manager import BlockManager
from .quota import QuotaExceeded, quota_of
from .runner import CausalLmRunner
from .scheduler import Policy, Scheduler, SchedulerConfig
from .types import ErrorClass, FinishReason, Request, SamplingParams, StepOutput


GRAPH_POOL_BYTES = 2 << 30      # captured graphs and their workspaces, per engine on a GPU
_HOLDERS = itertools.count()


class Watchdog:
    """Reports a job in flight longer than ``timeout`` seconds
    (crates/engine/src/worker/watchdog.rs:1-17, reference path).  Host-side only:
    device waits are bounded inside the kernels and surface as a status word."""

    def __init__(self, timeout: float = 150.0):
        self.timeout = timeout
        self.started: Optional[float] = None
        self.what = ""

    def begin(self, what: str) -> None:
        self.started, self.what = time.monotonic(), what

    def end(self) -> None:
        self.started = None

    def overdue(self) -> Optional[str]:
        if self.started is not None and time.monotonic() - self.started > self.timeout:
            return f"{self.what} in flight for more than {self.timeout:.0f}s"
        return None


def _weight_tensors(model):
    """(holder, attribute or key, tensor) of every weight tensor a model object owns: its own
    tensor attributes and those of its per-layer weight records."""
    def walk(holder):
        items = holder.items() if isinstance(holder, dict) else vars(holder).items()
        for name, v in list(items):
            if torch.is_tensor(v) and v.dim() > 0:
                yield holder, name, v
    yield from walk(model)
    for lw in getattr(model, "layers", None) or []:
        if lw is not None:
            yield from walk(lw)
            fp8 = getattr(lw, "fp8", None)
            if fp8 is not None:
                yield from walk(fp8)


def _weights_on(model, device) -> int:
    """Bytes of a model's weight tensors that live on ``device``'s kind of memory (tied
    tensors once)."""
    seen, total = set(), 0
    for _, name, t in _weight_tensors(model):
        if str(name).startswith("_"):               # step scratch kept on the model object
            continue
        if t.device.type == device.type and id(t) not in seen:
            seen.add(id(t))
            total += t.numel() * t.element_size()
    return total


def _host_available() -> float:
    """Bytes of host memory that can still be taken without swapping."""
    try:
        import psutil
        return float(psutil.virtual_memory().available)
    except Exception:                                   # pragma: no cover - psutil is present
        return float("inf")


def _set_tensor(holder, name, value) -> None:
    if isinstance(holder, dict):
        holder[name] = value
    else:
        setattr(holder, name, value)


class LLMEngine:
    def __init__(self, model: Qwen3MoeModel, num_pages: Optional[int] = None, page_size: int = 16,
                 max_num_seqs: int = 128, max_model_len: int = 4096,
                 max_num_batched_tokens: int = 8192, mem_fraction_static: float = 0.9,
                 enable_prefix_cache: bool = True, use_graphs: bool = True,
                 policy: Optional[Policy] = None, weights_identity: str = "random-init",
                 watchdog_timeout: float = 150.0, host_kv_pages: int = 0,
                 host_kv_ratio: float = 0.0, host_kv_gib: Optional[float] = None,
                 kv_dtype: Optional[str] = None, pipeline_decode: Optional[bool] = None,
                 quota=None, quota_strict: bool = False,
                 host_reserve_gib: Optional[float] = None):
        self.model = model
        self.device = model.device
        if kv_dtype in ("fp8", "fp8_e4m3", "e4m3"):
            model.kv_dtype = "fp8"       # E4M3 pages, one FP32 scale per page and plane
        elif kv_dtype not in (None, "auto", "bf16", "bfloat16"):
            raise ValueError(f"kv cache dtype {kv_dtype!r} is not served (bf16 or fp8)")
        max_model_len = min(max_model_len, model.cfg.max_position_embeddings)
        if num_pages is None:
            num_pages = self._divide_memory(mem_fraction_static, page_size, max_num_seqs,
                                            max_model_len)
        # the device's ledger: this engine's weights, graph pool and KV cache against the
        # fraction of the device its deployment may use (engine/quota.py)
        self.quota = quota if quota is not None else quota_of(self.device)
        self.quota_holder = f"engine-{os.getpid()}-{next(_HOLDERS)}"
        self.quota_strict = bool(quota_strict)
        self.quota_over: Optional[str] = None
        self._quota_items = {
            "weights": _weights_on(model, self.device),
            "graph_pool": GRAPH_POOL_BYTES if (self.device.type == "cuda" and use_graphs) else 0,
            "cache_segment": int(num_pages) * int(model.kv_bytes_per_page(page_size))}
        self.quota.state_fraction(self.quota_holder, min(1.0, max(1e-6, mem_fraction_static)))
        weakref.finalize(self, self.quota.release, self.quota_holder)
        self._reserve_quota(("weights", "graph_pool", "cache_segment"))
        self.blocks = BlockManager(num_pages, page_size, weights_identity, enable_prefix_cache)
        self.config = SchedulerConfig(max_num_seqs=max_num_seqs,
                                      max_num_batched_tokens=max_num_batched_tokens,
                                      chunked_prefill_size=max_num_batched_tokens,
                                      max_model_len=max_model_len, page_size=page_size,
                                      eos_token_id=model.cfg.eos_token_id)
        self.scheduler = Scheduler(self.blocks, self.config, policy)
        self.runner = CausalLmRunner(model, num_pages, page_size, max_num_seqs, max_model_len,
                                     use_graphs)
        self.runner.eos_token_id = model.cfg.eos_token_id
        if host_kv_pages == 0 and host_kv_ratio > 0:
            # sized as a multiple of the device pool, within a host-memory budget
            budget = (host_kv_gib if host_kv_gib is not None else 16.0) * (1 << 30)
            if host_reserve_gib is not None:
                # the node keeps this much host memory free of KV pages
                # (storage_config.host_reserve_gib of the reference's policy package)
                budget = min(budget, max(0.0, _host_available() - host_reserve_gib * (1 << 30)))
            per_page = max(1, model.kv_bytes_per_page(page_size))
            host_kv_pages = int(min(host_kv_ratio * num_pages, budget // per_page))
        if host_kv_pages > 0 and enable_prefix_cache:
            # Second KV tier: prefix pages evicted from the device pool move to host memory
            # and come back on a later hit (offload / prefetch decisions of the arrival
            # policy, crates/scheduling/policies/arrival/src/arrival.rs:34-46, reference path).
            self.blocks.enable_host_tier(host_kv_pages)
            self.runner.enable_host_tier(host_kv_pages)
        self.watchdog = Watchdog(watchdog_timeout)
        self._ids = itertools.count()
        self.failed: Optional[str] = None
        self.health = None        # parallel.health.Heartbeat of a multi-rank deployment
        # decode steps in flight (two turns): US_PIPELINE_DECODE=0 reads every step before the
        # next is issued
        self.pipeline_decode = pipeline_decode if pipeline_decode is not None else \
            (self.device.type == "cuda" and os.environ.get("US_PIPELINE_DECODE", "1") == "1")
        self.stream_steps = 32    # steps per upload of the step state
        self._stream = None
        self.asleep = 0           # sleep level (0 = awake)
        self._parked: list = []   # weights held in host memory while asleep at level 2
        self._parked_hosts: dict = {}
        self.profiler = None      # engine.profiling.StepProfiler when profiling is on
        self.spec_stats = {"steps": 0, "proposed": 0, "accepted": 0}

    def _reserve_quota(self, items) -> None:
        """Reserves ``items`` of this engine against the device's ledger.  A strict engine is
        refused past the limit (``QuotaExceeded``; what it reserved in this call is given
        back); otherwise the reservation is recorded all the same and ``quota_over`` says
        what did not fit."""
        done = []
        for item in items:
            n = self._quota_items.get(item, 0)
            key = f"weights-{id(self.model)}" if item == "weights" else None
            try:
                self.quota.reserve(self.quota_holder, item, n, key=key)
            except QuotaExceeded as e:
                if self.quota_strict:
                    for it in done:
                        self.quota.release(self.quota_holder, it)
                    raise
                self.quota.reserve(self.quota_holder, item, n, key=key, force=True)
                self.quota_over = str(e)
            done.append(item)

    def retire(self) -> int:
        """Ends this engine's reservations on the device's ledger (an engine that an update
        committed away from, a rolled-back target, an engine replaced after a failure).
        Returns the bytes released."""
        return self.quota.release(self.quota_holder)

    def _divide_memory(self, fraction, page_size, max_num_seqs, max_model_len) -> int:
        """Quota division: what is left of ``fraction`` of the device after the
        weights goes to KV pages (crates/engine/src/memory/division.rs, reference)."""
        per_page = self.model.kv_bytes_per_page(page_size)
        want = max_num_seqs * ((max_model_len + page_size - 1) // page_size) + 1
        if self.device.type != "cuda":
            return min(want, 4096)
        free, total = torch.cuda.mem_get_info(self.device)
        used_by_us = total - free
        budget = int(total * fraction) - used_by_us - GRAPH_POOL_BYTES   # graphs + workspaces
        pages = max(64, budget // per_page)
        return int(min(pages, want))

    # -------------------------------------------------------------- requests --
    def add_request(self, prompt_ids, params: Optional[SamplingParams] = None,
                    request_id: Optional[str] = None, priority: int = 0,
                    cache_salt: Optional[str] = None, output_ids: Optional[list] = None) -> str:
        if self.failed:
            raise RuntimeError(f"engine stopped: {self.failed}")
        rid = request_id or f"req-{next(self._ids)}"
        V = self.model.cfg.vocab_size
        if any((t < 0 or t >= V) for t in prompt_ids):
            raise ValueError("input_error: token id outside the vocabulary")
        req = Request(rid, list(prompt_ids), params or SamplingParams(), priority=priority,
                      cache_salt=cache_salt)
        if output_ids:                     # a migrated request resumes with its tokens
            req.output_ids = list(output_ids)
        self.scheduler.add_request(req)
        return rid

    def abort(self, request_id: str) -> bool:
        return self.scheduler.abort(request_id) is not None

    def has_work(self) -> bool:
        return not self.asleep and self.scheduler.has_work()

    # ---------------------------------------------------------- sleep / wake --
    def sleep(self, level: int = 1) -> dict:
        """Gives the GPU back while the process, its scheduler and its queue stay.
        Level 1 frees the KV cache and the captured graphs (the prefix cache is dropped);
        level 2 also moves the weights to pinned host memory.  Requests in flight are
        preempted (they recompute after ``wake``); new ones queue.  Returns the bytes freed.
        Reference behaviour: crates/engine/src/process (sleep / wake of a deployment)."""
        if self.asleep:
            return {"level": self.asleep, "freed_bytes": 0}
        sch = self.scheduler
        while sch.running:                      # recompute-style preemption of everything
            if not sch._preempt_one():
                break
        self.blocks.flush()
        freed = 0
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self._stream = None                     # steps in flight have completed
        self.runner.release_graphs()
        for pair in self.runner.kv_caches:
            for t in pair:
                if t is not None:
                    freed += t.numel() * t.element_size()
        self.runner.kv_caches = None
        self._parked = []
        if level >= 2:
            hosts = {}                          # one host copy per tensor (tied weights alias)
            for holder, name, t in _weight_tensors(self.model):
                if t.is_cuda:
                    if id(t) not in hosts:
                        host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                        host.copy_(t)
                        hosts[id(t)] = (host, t)        # keeps t alive until every alias is cut
                        freed += t.numel() * t.element_size()
                    self._parked.append((holder, name, id(t), t.device))
                    _set_tensor(holder, name, None)
            self._parked_hosts = {k: h for k, (h, _) in hosts.items()}
            del hosts
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            torch.cuda.empty_cache()
        self.asleep = level
        for item in ("cache_segment", "graph_pool") + (("weights",) if level >= 2 else ()):
            self.quota.release(self.quota_holder, item)
        return {"level": level, "freed_bytes": freed}

    def wake(self) -> dict:
        """Undoes ``sleep``: weights back on the device, a fresh (empty) KV cache of the same
        size; graphs are captured again on first use."""
        if not self.asleep:
            return {"level": 0}
        # the quota first: a strict engine that no longer fits stays asleep, untouched
        self._reserve_quota(("cache_segment", "graph_pool") +
                            (("weights",) if self.asleep >= 2 else ()))
        back = {}
        for holder, name, key, dev in self._parked:
            if key not in back:
                back[key] = self._parked_hosts[key].to(dev, non_blocking=True)
            _set_tensor(holder, name, back[key])
        self._parked, self._parked_hosts = [], {}
        self.runner.kv_caches = self.model.new_kv_caches(self.blocks.num_pages, self.config.page_size)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        level, self.asleep = self.asleep, 0
        return {"level": 0, "was": level}

    # ------------------------------------------------------------------ step --
    # ------------------------------------------------- decode steps in flight --
    def _stream_start(self):
        """Starts a stream of decode steps when every running request is decoding and
        nothing waits: pages for the next steps are taken now, the step state is uploaded
        once, and two steps are issued before the first is read."""
        sch = self.scheduler
        rows = [r for r in sch.running if r.output_ids and r.num_computed == r.num_tokens - 1]
        if not rows or len(rows) != len(sch.running) or sch.waiting or self.profiler is not None:
            return None
        if self.runner.variant_for(rows) == "logits":
            return None
        limit = min(self.runner.history_steps, self.stream_steps,
                    min(self.config.max_model_len - r.num_tokens for r in rows),
                    max(r.params.max_tokens - len(r.output_ids) for r in rows))
        if limit < 2:
            return None
        for r in rows:
            pages = self.blocks.allocate(sch._pages_needed(r, r.num_tokens + limit))
            if pages is None:
                return None
            r.pages.extend(pages)
        if getattr(self.blocks, "host_slots", 0):
            self.runner.apply_kv_moves(*self.blocks.take_moves())
        st = self.runner.decode_begin(rows)
        st.limit = limit
        return st

    def _stream_step(self) -> list:
        """One call = one step's tokens.  The next step is already on the device when this
        one is read (two turns in flight), so the host's share of a step - reading, stop
        rules, page commits, streaming - overlaps the device's."""
        from .scheduler import Batch, Chunk
        st, sch = self._stream, self.scheduler
        self.watchdog.begin(f"decode stream step {st.collected}")
        try:
            while not st.draining and st.launched < st.limit and st.launched - st.collected < 2:
                self.runner.decode_launch(st)
            toks = self.runner.decode_collect(st, st.collected)
        except Exception as e:
            self._stream = None
            self.failed = f"{ErrorClass.FATAL_WORKER_FAILURE.value}: {e}"
            if self.health is not None:
                self.health.report_failure(self.failed)
            raise
        finally:
            self.watchdog.end()
        st.collected += 1
        live = [(i, r) for i, r in enumerate(st.rows)
                if not r.finished and r.request_id in sch.requests]
        outs = []
        if live:
            V = self.model.cfg.vocab_size
            errors = {r.request_id: f"{ErrorClass.NUMERICAL_FAULT.value}: sampled token {toks[i]}"
                      for i, r in live if toks[i] < 0 or toks[i] >= V}
            batch = Batch("decode", [Chunk(r, r.num_tokens - 1, 1, True) for _, r in live])
            sch.stats["decode_tokens"] += len(live)
            outs = sch.update(batch, {r.request_id: int(toks[i]) for i, r in live}, None, errors)
        # the set of rows changed, or somebody waits: read what is in flight, then re-plan
        if len(sch.running) != len(st.rows) or sch.waiting or \
                any(r.finished for r in st.rows):
            st.draining = True
        if st.collected >= st.launched and (st.draining or st.launched >= st.limit):
            self._stream = None
        elif st.draining and not any(not r.finished and r.request_id in sch.requests
                                     for r in st.rows):
            self._stream = None             # nobody is left to read the steps in flight for
        return outs

    def step(self) -> list:
        if self.asleep:
            return []
        if self._stream is None and self.pipeline_decode:
            self._stream = self._stream_start()
        if self._stream is not None:
            outs = self._stream_step()
            if self.blocks.kv_events is not None:
                self.blocks.kv_events.flush()
            return outs
        batch = self.scheduler.schedule()
        if batch is None:
            return []
        outs = self.run_batch(batch)
        if self.blocks.kv_events is not None:
            self.blocks.kv_events.flush()       # a step's KV events are one batch
        return outs

    def run_batch(self, batch, capacity: Optional[int] = None) -> list:
        """Executes a scheduled batch and applies its results.  ``capacity``: the row count
        the members of an expert union agreed on for this step (``engine/union.py``)."""
        if getattr(self.blocks, "host_slots", 0):
            self.runner.apply_kv_moves(*self.blocks.take_moves())
        self.watchdog.begin(f"{batch.kind} step {batch.step_id}")
        try:
            if self.profiler is not None:
                with self.profiler.step(batch.kind, batch.step_id):
                    sampled, lps = self.runner.execute(batch, capacity)
            elif capacity is not None:
                sampled, lps = self.runner.execute(batch, capacity)
            else:
                sampled, lps = self.runner.execute(batch)
        except Exception as e:     # fatal_worker_failure: stop the engine, fail every request
            self.failed = f"{ErrorClass.FATAL_WORKER_FAILURE.value}: {e}"
            if self.health is not None:     # the peers learn of it before their next launch
                self.health.report_failure(self.failed)
            raise
        finally:
            self.watchdog.end()
        errors = {}
        V = self.model.cfg.vocab_size
        for rid, tok in sampled.items():
            if tok < 0 or tok >= V:
                errors[rid] = f"{ErrorClass.NUMERICAL_FAULT.value}: sampled token {tok}"
        return self.scheduler.update(batch, sampled, lps, errors)

    def decode_burst(self, steps: int) -> list:
        """Multi-step decode: when every running request is decoding, ensures
        pages for ``steps`` more tokens, replays the decode graph ``steps`` times
        with the device advancing its own step state, then applies the tokens.
        Requests that stop inside the burst drop their surplus tokens."""
        sch = self.scheduler
        rows = [r for r in sch.running if r.output_ids and r.num_computed == r.num_tokens - 1]
        if not rows or len(rows) != len(sch.running) or sch.waiting:
            return self.step()
        steps = min(steps, self.runner.history_steps,
                    min(self.config.max_model_len - r.num_tokens for r in rows))
        if steps <= 1 or self.runner.variant_for(rows) == "logits":
            return self.step()
        for r in rows:
            pages = self.blocks.allocate(sch._pages_needed(r, r.num_tokens + steps))
            if pages is None:
                return self.step()
            r.pages.extend(pages)
        if getattr(self.blocks, "host_slots", 0):
            self.runner.apply_kv_moves(*self.blocks.take_moves())
        toks, _ = self.runner.decode(rows, steps)
        outs = []
        from .scheduler import Batch, Chunk
        for s_ in range(steps):
            live = [(i, r) for i, r in enumerate(rows) if not r.finished]
            if not live:
                break
            batch = Batch("decode", [Chunk(r, r.num_tokens - 1, 1, True) for _, r in live])
            sch.stats["decode_tokens"] += len(live)
            outs.extend(sch.update(batch, {r.request_id: int(toks[s_, i]) for i, r in live}))
        return outs

    def speculative_step(self, drafter) -> list:
        """One step with speculation: when every running request is decoding greedily, each
        gets up to ``drafter.k`` proposed tokens verified in one call and advances by the
        agreed prefix plus one token; otherwise an ordinary step runs."""
        from .scheduler import Batch, Chunk
        from .speculation import accept
        sch = self.scheduler
        stateful = getattr(drafter, "needs_hidden", False)
        if stateful and getattr(self.runner, "hidden_tap", None) is None and hasattr(drafter, "tap"):
            self.runner.hidden_tap = drafter.tap       # prompt rows reach the drafter at prefill
        rows = [r for r in sch.running if r.output_ids and r.num_computed == r.num_tokens - 1]
        if not rows or len(rows) != len(sch.running) or sch.waiting or \
                self.runner.variant_for(rows) != "greedy":
            return self.step()
        drafts = []
        if stateful:
            drafter.forget({r.request_id for r in self.scheduler.requests.values()
                            if not r.finished})
        for r in rows:
            room = min(self.config.max_model_len - r.num_tokens - 1,
                       r.params.max_tokens - len(r.output_ids) - 1)
            d = drafter.propose_for(r) if stateful else drafter.propose(r.all_ids)
            d = d[:max(0, min(drafter.k, room))]
            pages = self.blocks.allocate(sch._pages_needed(r, r.num_tokens + len(d)))
            if pages is None:
                d, pages = [], []
            r.pages.extend(pages)
            drafts.append(d)
        # a drafter that feeds on the target's hidden states gets its first ones from a
        # verification of the last token alone
        if not any(drafts) and not (stateful and
                                    any(not drafter.ready(r.request_id) for r in rows)):
            return self.step()
        if getattr(self.blocks, "host_slots", 0):
            self.runner.apply_kv_moves(*self.blocks.take_moves())
        self.watchdog.begin("verify step")
        try:
            if stateful:
                targets, hiddens = self.runner.verify(rows, drafts, want_hidden=True)
            else:
                targets, hiddens = self.runner.verify(rows, drafts), None
        finally:
            self.watchdog.end()
        outs = []
        self.spec_stats["steps"] += 1
        for r, d, t in zip(rows, drafts, targets):
            emit = accept(d, t)
            if stateful:
                i = rows.index(r)
                drafter.observe(r.request_id, r.num_tokens - 1, hiddens[i][:len(emit)], emit)
            self.spec_stats["proposed"] += len(d)
            self.spec_stats["accepted"] += len(emit) - 1
            for tok in emit:
                if r.finished:
                    break
                batch = Batch("decode", [Chunk(r, r.num_tokens - 1, 1, True)])
                sch.stats["decode_tokens"] += 1
                outs.extend(sch.update(batch, {r.request_id: tok}))
        return outs

    # -------------------------------------------------------------- generate --
    def generate(self, prompts: list, params=None, on_output=None) -> list:
        """Runs the prompts to completion; returns the output token lists in
        prompt order.  ``params`` is one SamplingParams or a list."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while self.scheduler.has_work():
            outs = self.step()
            if on_output:
                for o in outs:
                    on_output(o)
        return [self.scheduler.requests[i].output_ids for i in ids]

    def stats(self) -> dict:
        s = dict(self.scheduler.stats)
        s.update({"kv": self.blocks.stats(), "running": len(self.scheduler.running),
                  "waiting": len(self.scheduler.waiting), "h2d_bytes": self.runner.h2d_bytes,
                  "d2h_bytes": self.runner.d2h_bytes,
                  "blocking_calls": dict(self.runner.blocking),
                  "blocking_seconds": self.runner.blocking_s,
                  "quota": {"holder": self.quota_holder, "device": self.quota.name,
                            "bytes": self.quota.usage(self.quota_holder),
                            "limit": self.quota.limit(), "over": self.quota_over}})
        return s
