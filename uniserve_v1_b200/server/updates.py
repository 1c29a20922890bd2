"""Epoch updates: a configuration change that needs a new engine is applied while serving.

Phases (the reference's update machine, docs/architecture.md:45-48 and
crates/daemon/src/updates/update.rs, reference project paths), folded into one process:

1. **Preparing.**  The target engine is built (weights, KV cache, graphs) on a helper
   thread while the serving engine goes on stepping.  A target that fails here is dropped
   and the update is *abandoned* with nothing changed.
2. **Switching.**  New requests go to the target from now on; the previous engine admits
   nothing and steps the requests it holds until each ends by itself.  At the deadline
   ``update_config.drain_s`` the rest leave as migratable facts (prompt + generated tokens)
   and are resubmitted to the target (their prefix pages are recomputed or found in the
   target's cache; sampling is addressed by (seed, position), so the continuation is the
   same).
3. **Trial.**  The target serves on trial for ``update_config.trial`` with the previous
   engine kept parked.  A fatal failure of the target, or a threshold of
   ``update_config.rollback`` (failure rate, step-time regression, throughput regression
   against the previous engine's baseline) runs the switch the other way: *rolled back*.
4. **Committed.**  The decision is recorded, then the previous engine is released.

``EngineService`` owns the machine: it calls ``advance`` once per loop turn from the one
thread that touches engines.
"""
from __future__ import annotations

import threading
import time
from collections import deque
from typing import Callable, Optional


def _retire(engine) -> None:
    """Ends an engine's reservations on its device's quota ledger (engine/quota.py)."""
    for e in (engine, getattr(engine, "engine", None)):
        retire = getattr(e, "retire", None) if e is not None else None
        if callable(retire):
            try:
                retire()
            except Exception:
                pass
            return


class StepClock:
    """Moving record of an engine's step times and output tokens (for the trial)."""

    def __init__(self, keep: int = 512):
        self.steps = deque(maxlen=keep)      # (seconds, tokens)
        self.failed = 0
        self.finished = 0

    def record(self, seconds: float, tokens: int) -> None:
        self.steps.append((seconds, tokens))

    def mean_step(self) -> Optional[float]:
        return sum(s for s, _ in self.steps) / len(self.steps) if self.steps else None

    def throughput(self) -> Optional[float]:
        t = sum(s for s, _ in self.steps)
        return sum(n for _, n in self.steps) / t if t > 0 else None


class EpochUpdate:
    def __init__(self, build: Callable[[], object], trial_s: float = 30.0, drain_s: float = 5.0,
                 failure_rate: Optional[float] = None,
                 step_time_regression: Optional[float] = None,
                 throughput_regression: Optional[float] = None,
                 min_steps: int = 8, on_phase: Optional[Callable[[str, str], None]] = None,
                 clock: Callable[[], float] = time.monotonic):
        self.build = build
        self.trial_s, self.drain_s = float(trial_s), float(drain_s)
        self.failure_rate = failure_rate
        self.step_time_regression = step_time_regression
        self.throughput_regression = throughput_regression
        self.min_steps = min_steps
        self.on_phase = on_phase or (lambda phase, why: None)
        self.clock = clock
        self.phase = "preparing"
        self.reason = ""
        self.target = None
        self.previous = None
        self.error: Optional[str] = None
        self.baseline = None                 # StepClock of the previous engine at the switch
        self.trial_clock = StepClock()
        self.deadline = 0.0
        self.trial_end = 0.0
        self.history = ["preparing"]
        self._thread = threading.Thread(target=self._prepare, name="epoch-prepare", daemon=True)
        self._thread.start()

    # ------------------------------------------------------------------ phases --
    def _prepare(self) -> None:
        try:
            self.target = self.build()
        except Exception as e:               # nothing changed: the update is abandoned
            self.error = f"{type(e).__name__}: {e}"

    def _enter(self, phase: str, why: str = "") -> None:
        self.phase, self.reason = phase, why
        self.history.append(phase)
        self.on_phase(phase, why)

    @property
    def done(self) -> bool:
        return self.phase in ("committed", "rolled_back", "abandoned")

    def advance(self, svc) -> None:
        """One turn of the machine; ``svc`` is the EngineService (engine thread only)."""
        now = self.clock()
        if self.phase == "preparing":
            if self._thread.is_alive():
                return
            if self.error is not None or self.target is None:
                self._enter("abandoned", self.error or "no target")
                return
            # switching: new requests go to the target, the previous engine drains
            self.previous, svc.engine = svc.engine, self.target
            self.baseline = svc.step_clock
            svc.step_clock = self.trial_clock
            svc.draining = self.previous
            self.deadline = now + self.drain_s
            self._enter("switching")
        elif self.phase == "switching":
            if self.previous.has_work() and now < self.deadline:
                return
            moved = svc.migrate_all(self.previous, svc.engine) if self.previous.has_work() else 0
            svc.draining = None
            self.trial_end = now + self.trial_s
            self._enter("trial", f"{moved} requests migrated at the drain deadline")
        elif self.phase == "trial":
            why = self._threshold()
            if why or getattr(svc.engine, "failed", None):
                self.rollback(svc, why or f"target failed: {svc.engine.failed}")
            elif now >= self.trial_end:
                self._enter("committed")                 # the decision first, then the release
                prev, self.previous = self.previous, None
                release = getattr(getattr(prev, "runner", None), "release_graphs", None)
                if release:
                    release()
                _retire(prev)                            # its quota ends with it

    def _threshold(self) -> Optional[str]:
        t, b = self.trial_clock, self.baseline
        if self.failure_rate is not None and t.finished + t.failed >= 4:
            rate = t.failed / (t.finished + t.failed)
            if rate > self.failure_rate:
                return f"failure rate {rate:.2f} over {self.failure_rate}"
        if len(t.steps) < self.min_steps or b is None or len(b.steps) < self.min_steps:
            return None
        if self.step_time_regression is not None and \
                t.mean_step() > b.mean_step() * (1 + self.step_time_regression):
            return (f"step time {t.mean_step() * 1e3:.2f} ms against "
                    f"{b.mean_step() * 1e3:.2f} ms before")
        if self.throughput_regression is not None and b.throughput() and \
                t.throughput() < b.throughput() * (1 - self.throughput_regression):
            return f"throughput {t.throughput():.0f} tok/s against {b.throughput():.0f} before"
        return None

    def rollback(self, svc, why: str) -> None:
        """The switch the other way: the previous engine serves again, the target's
        requests continue there."""
        target, svc.engine = svc.engine, self.previous
        svc.step_clock = self.baseline or StepClock()
        svc.draining = None
        try:
            svc.migrate_all(target, svc.engine)
        except Exception:
            pass
        self.previous = None
        _retire(target)
        self._enter("rolled_back", why)
