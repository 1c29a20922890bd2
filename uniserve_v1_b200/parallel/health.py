"""Peer liveness between steps: heartbeats over the rendezvous store.

Ranks that step in lock step (tensor / expert / sequence groups) must learn of
a dead peer on the host *before* their next launch: a collective or a peer-flag
wait issued towards a rank that is gone would otherwise run into its device-side
time limit.  Every rank publishes a counter under ``hb/<rank>`` from a background
thread and, when it fails in a way it can report, a reason under
``failed/<rank>``.  ``check()`` (called between steps, with nothing in flight)
raises ``PeerFailure`` when a peer reported a failure or its counter stopped
for longer than ``timeout_s``; the caller then fails its requests with
``fatal_worker_failure`` and the serving layer migrates them.

Reference behaviour: crates/engine/src/worker/watchdog.rs:1-17,
crates/daemon/src/migration.rs:1-40 (reference project paths).
"""
from __future__ import annotations

import threading
import time
from typing import Optional


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank}: {reason}")
        self.rank, self.reason = rank, reason


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 0.2,
                 timeout_s: float = 2.0, prefix: str = "health"):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s, self.prefix = interval_s, timeout_s, prefix
        self._stop = threading.Event()
        self._count = 0
        self._seen = {r: (None, time.monotonic()) for r in range(world) if r != rank}
        self._beat()
        self._thread = threading.Thread(target=self._run, name="heartbeat", daemon=True)
        self._thread.start()

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def _beat(self) -> None:
        self._count += 1
        self.store.set(self._key("hb", self.rank), str(self._count))

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                self._beat()
            except Exception:      # the store is gone: the job is ending
                return

    def report_failure(self, reason: str) -> None:
        """Tell the peers why this rank is leaving (best effort)."""
        try:
            self.store.set(self._key("failed", self.rank), reason[:500])
        except Exception:
            pass

    def check(self) -> None:
        """Raises PeerFailure for the first peer that reported a failure or went silent."""
        now = time.monotonic()
        for r in self._seen:
            fk = self._key("failed", r)
            if self.store.check([fk]):
                raise PeerFailure(r, self.store.get(fk).decode())
            hk = self._key("hb", r)
            value = self.store.get(hk).decode() if self.store.check([hk]) else None
            last, since = self._seen[r]
            if value != last:
                self._seen[r] = (value, now)
            elif now - since > self.timeout_s:
                raise PeerFailure(r, f"no heartbeat for {now - since:.1f} s")

    def close(self) -> None:
        self._stop.set()
        self._thread.join(timeout=2 * self.interval_s + 1)
