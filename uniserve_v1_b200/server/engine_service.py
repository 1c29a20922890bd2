"""The engine loop of a serving process and the request-side adapter around it.

One thread owns the engine (one issuer per device); HTTP handlers hand it
requests through a queue and receive step outputs on per-request asyncio queues.
A finished, failed or aborted request always ends its stream.  Requests are kept
as migratable facts (prompt, generated tokens, seed) so a restarted engine can
resume them (crates/daemon/src/migration.rs:12-25, leader.rs:1559, engine/hold.rs,
reference project paths).
"""
from __future__ import annotations

import asyncio
import queue
import threading
import time
import uuid
from typing import Optional

from ..engine.types import FinishReason, SamplingParams, StepOutput


class Overloaded(RuntimeError):
    pass


class EngineService:
    def __init__(self, engine, observation=None, max_queued: Optional[int] = None,
                 max_migrations: int = 3, engine_factory=None, drafter=None):
        self.engine = engine
        # speculative decoding: every step goes through the drafter when it applies
        # (all running requests decoding greedily), an ordinary step otherwise
        self.drafter = drafter
        self.obs = observation
        self.max_queued = max_queued
        self.max_migrations = max_migrations
        self.engine_factory = engine_factory      # rebuilds the engine after a fatal failure
        self.inbox: queue.Queue = queue.Queue()
        self.streams: dict = {}                   # request_id -> (loop, asyncio.Queue)
        self.meta: dict = {}
        self.lock = threading.Lock()
        self.wake = threading.Event()
        self.stopping = False
        self.paused = False
        self.thread = threading.Thread(target=self._run, name="engine-loop", daemon=True)
        self.started = False
        self.last_snapshot = 0.0
        self.steps = 0
        from .updates import StepClock
        self.step_clock = StepClock()
        self.update = None                        # server.updates.EpochUpdate in progress
        self.draining = None                      # the previous engine while it drains

    def call(self, fn, timeout: float = 300.0):
        """Runs ``fn(engine)`` on the engine's own thread, between two steps, and returns its
        value (sleep, wake and other actions that must not race a step)."""
        if not self.started or not self.thread.is_alive():
            return fn(self.engine)
        box, done = {}, threading.Event()
        self.inbox.put(("call", fn, box, done))
        self.wake.set()
        if not done.wait(timeout):
            raise TimeoutError("the engine loop did not take the action in time")
        if "error" in box:
            raise box["error"]
        return box.get("value")

    def start(self):
        if not self.started:
            self.started = True
            self.thread.start()

    def stop(self, timeout: float = 30.0):
        self.stopping = True
        self.wake.set()
        if self.started:
            self.thread.join(timeout)

    # ------------------------------------------------------------ submission --
    def submit(self, prompt_ids, params: SamplingParams, request_id: Optional[str] = None,
               priority: int = 0, cache_salt: Optional[str] = None, lend: bool = False,
               handoff=None, media=None):
        """Returns (request_id, asyncio.Queue of StepOutput); call from an event loop.
        ``lend``: the request leaves after its first token - its stream ends with an output
        that carries the framed state (prefill role).  ``handoff``: continue a request that
        another engine lent (decode role); ``prompt_ids`` are then only kept for accounting."""
        if self.max_queued is not None and self.inbox.qsize() + len(self.streams) >= self.max_queued:
            raise Overloaded("too many queued requests")
        rid = request_id or "chatcmpl-" + uuid.uuid4().hex
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        with self.lock:
            self.streams[rid] = (loop, q)
            self.meta[rid] = {"arrival": time.monotonic(), "first": None, "tokens": 0,
                              "prompt": list(prompt_ids), "params": params, "outputs": [],
                              "migrations": 0, "priority": priority, "salt": cache_salt,
                              "lend": lend, "media": media}
        if handoff is not None:
            # one hand-off, or (the frames of every exporting rank, the body they came in)
            hs, body = handoff if isinstance(handoff, tuple) else ([handoff], None)
            for h in hs:
                h.request_id = rid
            self.meta[rid]["outputs"] = list(hs[0].output_ids)
            self.inbox.put(("import", rid, hs, body))
        else:
            self.inbox.put(("add", rid, list(prompt_ids), params, priority, cache_salt, None,
                            media))
        self.wake.set()
        return rid, q

    def abort(self, request_id: str):
        self.inbox.put(("abort", request_id))
        self.wake.set()

    # ------------------------------------------------------------------ loop --
    def _deliver(self, out: StepOutput):
        with self.lock:
            ent = self.streams.get(out.request_id)
            meta = self.meta.get(out.request_id)
        if meta is not None and out.new_token_ids:
            now = time.monotonic()
            if meta["first"] is None:
                meta["first"] = now
                if self.obs:
                    self.obs.observe("uniserve_ttft_seconds", now - meta["arrival"])
            meta["tokens"] += len(out.new_token_ids)
            meta["outputs"].extend(out.new_token_ids)
        if ent is not None:
            loop, q = ent
            loop.call_soon_threadsafe(q.put_nowait, out)
        if out.finished:
            with self.lock:
                self.streams.pop(out.request_id, None)
                meta = self.meta.pop(out.request_id, None)
            if self.obs and meta:
                dur = time.monotonic() - meta["arrival"]
                outcome = out.finish_reason.value if out.finish_reason else "unknown"
                self.obs.inc("uniserve_requests_total", {"outcome": outcome})
                if meta["tokens"] > 1 and meta["first"]:
                    self.obs.observe("uniserve_tpot_seconds",
                                     (time.monotonic() - meta["first"]) / (meta["tokens"] - 1))
                self.obs.event("request", out.request_id, outcome=outcome, seconds=dur,
                               output_tokens=meta["tokens"], prompt_tokens=len(meta["prompt"]),
                               cached_tokens=out.num_cached_tokens)

    def _recover(self, error: Exception):
        """Fatal worker failure: rebuild the engine and resubmit every live request
        with the tokens it already generated (bounded by ``max_migrations``)."""
        if self.engine_factory is None:
            with self.lock:
                live = list(self.streams.keys())
            for rid in live:
                self._deliver(StepOutput(rid, [], True, FinishReason.ERROR, error=str(error)))
            return
        retire = getattr(self.engine, "retire", None)
        if retire is not None:                # the failed engine's quota goes to its successor
            retire()
        self.engine = self.engine_factory()
        with self.lock:
            live = list(self.meta.items())
        for rid, m in live:
            m["migrations"] += 1
            if m["migrations"] > self.max_migrations:
                self._deliver(StepOutput(rid, [], True, FinishReason.ERROR,
                                         error=f"migrated more than {self.max_migrations} times"))
                continue
            self.inbox.put(("add", rid, m["prompt"], m["params"], m["priority"], m["salt"],
                            list(m["outputs"]), m.get("media")))
        if self.obs:
            self.obs.inc("uniserve_engine_restarts_total")

    # ---------------------------------------------------------------- updates --
    def begin_update(self, update) -> None:
        """Starts an epoch update (``server.updates.EpochUpdate``); the loop advances it."""
        if self.update is not None and not self.update.done:
            raise RuntimeError("an update is already in progress")
        self.update = update
        self.wake.set()

    def migrate_all(self, source, target) -> int:
        """Every live request of ``source`` continues on ``target`` from its migratable facts
        (prompt, generated tokens, sampling parameters); returns how many moved."""
        moved = 0
        for req in list(source.scheduler.running) + list(source.scheduler.waiting):
            rid = req.request_id
            with self.lock:
                m = self.meta.get(rid)
            source.abort(rid)
            if m is None:
                continue
            m["migrations"] += 1
            if m["migrations"] > self.max_migrations:
                self._deliver(StepOutput(rid, [], True, FinishReason.ERROR,
                                         error=f"migrated more than {self.max_migrations} times"))
                continue
            try:
                target.add_request(m["prompt"], m["params"], request_id=rid,
                                   priority=m["priority"], cache_salt=m["salt"],
                                   output_ids=list(m["outputs"]))
                moved += 1
            except Exception as e:
                self._deliver(StepOutput(rid, [], True, FinishReason.ERROR, error=str(e)))
        return moved

    def _run(self):
        while not self.stopping:
            if self.update is not None and not self.update.done:
                try:
                    self.update.advance(self)
                except Exception as e:
                    self.update.phase, self.update.reason = "abandoned", str(e)
            if self.draining is not None and self.draining.has_work():
                try:                            # the previous engine steps what it still holds
                    for o in self.draining.step():
                        self._deliver(o)
                except Exception:
                    self.migrate_all(self.draining, self.engine)
            try:
                while True:
                    msg = self.inbox.get_nowait()
                    if msg[0] == "add":
                        _, rid, ids, params, prio, salt, outputs, media = msg
                        try:
                            extra = {"media": media} if media is not None else {}
                            self.engine.add_request(ids, params, request_id=rid, priority=prio,
                                                    cache_salt=salt, output_ids=outputs, **extra)
                        except Exception as e:      # input_error rejects the request
                            self._deliver(StepOutput(rid, [], True, FinishReason.ERROR, error=str(e)))
                    elif msg[0] == "import":
                        try:
                            from ..engine.handoff import import_request, pack_frames
                            whole = getattr(self.engine, "import_request", None)
                            if whole is not None:     # every rank of a replicated engine
                                body = msg[3] if len(msg) > 3 and msg[3] is not None else \
                                    pack_frames([h.to_bytes() for h in msg[2]])
                                whole(msg[1], body)
                            else:
                                import_request(self.engine, msg[2])
                        except Exception as e:
                            self._deliver(StepOutput(msg[1], [], True, FinishReason.ERROR,
                                                     error=f"hand-off refused: {e}"))
                    elif msg[0] == "call":          # an operator action on the engine's thread
                        _, fn, box, done = msg
                        try:
                            box["value"] = fn(self.engine)
                        except Exception as e:
                            box["error"] = e
                        done.set()
                    elif msg[0] == "abort":
                        if self.engine.abort(msg[1]) or \
                                (self.draining is not None and self.draining.abort(msg[1])):
                            self._deliver(StepOutput(msg[1], [], True, FinishReason.ABORT))
            except queue.Empty:
                pass
            if self.paused or not self.engine.has_work():
                busy = self.draining is not None and self.draining.has_work()
                if not busy:
                    self.wake.wait(0.05 if self.update is None or self.update.done else 0.005)
                    self.wake.clear()
                continue
            t_step = time.monotonic()
            try:
                if self.drafter is not None and hasattr(self.engine, "speculative_step"):
                    outs = self.engine.speculative_step(self.drafter)
                else:
                    outs = self.engine.step()
            except Exception as e:
                if self.update is not None and self.update.phase == "trial":
                    self.update.rollback(self, f"target failed: {e}")     # back to the previous
                    continue
                self._recover(e)
                continue
            self.steps += 1
            self.step_clock.record(time.monotonic() - t_step,
                                   sum(len(o.new_token_ids) for o in outs))
            for o in outs:
                if o.finished:
                    if o.finish_reason == FinishReason.ERROR:
                        self.step_clock.failed += 1
                    else:
                        self.step_clock.finished += 1
            for o in outs:
                meta = self.meta.get(o.request_id)
                if meta and meta.get("lend") and o.new_token_ids and not o.finished:
                    from ..engine.handoff import export_request
                    whole = getattr(self.engine, "export_request", None)
                    blob = whole(o.request_id) if whole is not None else \
                        export_request(self.engine, o.request_id).to_bytes()
                    o = StepOutput(o.request_id, o.new_token_ids, True, None,
                                   num_cached_tokens=o.num_cached_tokens, handoff=blob)
                self._deliver(o)
            now = time.monotonic()
            if self.obs and now - self.last_snapshot > 1.0:
                self.last_snapshot = now
                st = self.engine.stats()
                self.obs.set("uniserve_kv_cache_used_pages", st["kv"]["pages"] - st["kv"]["free"],
                             {"tier": "device"})
                self.obs.set("uniserve_running_requests", st["running"])
                self.obs.set("uniserve_waiting_requests", st["waiting"])
                self.obs.set("uniserve_preemptions_total", st["preemptions"])
                for site, n in (st.get("blocking_calls") or {}).items():
                    self.obs.set("uniserve_blocking_calls_total", n, {"site": site})
                self.obs.set("uniserve_blocking_seconds_total", st.get("blocking_seconds", 0.0))
                snap = getattr(getattr(self.engine, "model", None), "expert_load_snapshot", None)
                if snap is not None and now - getattr(self, "_last_load", 0.0) > 5.0:
                    self._last_load = now          # what the expert-order program balances
                    for layer, row in snap().items():
                        for e, n in enumerate(row):
                            self.obs.set("uniserve_expert_tokens_total", n,
                                         {"layer": str(layer), "expert": str(e)})
                self.obs.snapshot()
