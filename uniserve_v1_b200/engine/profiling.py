"""Always-on step counters, fence probes and profile sessions.

* **Fence probes** stamp the GPU's nanosecond timer into pinned host memory at
  chosen points of the stream (``ProbeRing.mark``); reading them back needs no
  synchronisation beyond the step's own read-back.  On a CPU device a probe is
  a host monotonic timestamp, so the same code paths run in CPU tests.
* **Host spans** record (name, start, end) on the calling thread.
* A **session** collects both into one SQLite file per rank (tables ``spans``,
  ``probes``, ``counters``, ``meta``) which ``tools/profile.py`` turns into a
  Perfetto / Chrome trace.

Reference: crates/engine/src/profiling/{markers,session,artifact,collectors}.rs,
docs/profiling.md (reference project paths).  The reference also wraps CUPTI
(activity records, PM/PC sampling, range profiler); those need the profiling
libraries' own interfaces and are not part of this package.
"""
from __future__ import annotations

import sqlite3
import threading
import time
from contextlib import contextmanager
from typing import Optional

import torch

from ..ops import native as N

N.register_signatures({"us_range_marker": (N.I, [N.P, N.I, N.c_ulonglong, N.P])})


class ProbeRing:
    """``capacity`` probe slots in pinned host memory, reused in a ring."""

    def __init__(self, capacity: int = 4096, device="cpu"):
        self.capacity = capacity
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.slots = torch.zeros(capacity, 4, dtype=torch.int64)
        if self.cuda:
            self.slots = self.slots.pin_memory()
        self.names: list = [None] * capacity
        self.cursor = 0
        self.pending: list = []          # slot indices marked and not yet collected

    def mark(self, name: str, tag: int = 0) -> int:
        i = self.cursor % self.capacity
        self.cursor += 1
        self.names[i] = name
        self.slots[i, 0] = 0
        if self.cuda:
            N.call("us_range_marker", self.slots.data_ptr(), i, tag, N.stream())
        else:
            self.slots[i, 0] = time.monotonic_ns()
            self.slots[i, 2] = tag
        self.pending.append(i)
        return i

    def collect(self, wait: bool = True) -> list:
        """(name, timer_ns, sm_clock, tag) of every probe that has fired, in order."""
        if self.cuda and wait:
            torch.cuda.current_stream(self.device).synchronize()
        out, still = [], []
        for i in self.pending:
            t = int(self.slots[i, 0])
            if t == 0:
                still.append(i)
                continue
            out.append((self.names[i], t, int(self.slots[i, 1]), int(self.slots[i, 2])))
        self.pending = still
        return out


class Session:
    """One profile session of one rank: an SQLite artifact."""

    def __init__(self, path: str, rank: int = 0, meta: Optional[dict] = None):
        self.path, self.rank = path, rank
        self.db = sqlite3.connect(path, check_same_thread=False)
        self.lock = threading.Lock()
        self.db.executescript(
            "CREATE TABLE IF NOT EXISTS spans(rank INT, thread TEXT, name TEXT, start_ns INT,"
            " end_ns INT, step INT);"
            "CREATE TABLE IF NOT EXISTS probes(rank INT, name TEXT, timer_ns INT, sm_clock INT,"
            " tag INT);"
            "CREATE TABLE IF NOT EXISTS counters(rank INT, name TEXT, step INT, value REAL);"
            "CREATE TABLE IF NOT EXISTS meta(key TEXT, value TEXT);")
        for k, v in (meta or {}).items():
            self.db.execute("INSERT INTO meta VALUES (?, ?)", (k, str(v)))
        # offset between the host's realtime clock and its monotonic clock, for alignment
        self.db.execute("INSERT INTO meta VALUES (?, ?)",
                        ("realtime_minus_monotonic_ns", str(time.time_ns() - time.monotonic_ns())))
        self.db.commit()

    def span(self, name: str, start_ns: int, end_ns: int, step: int = -1):
        with self.lock:
            self.db.execute("INSERT INTO spans VALUES (?,?,?,?,?,?)",
                            (self.rank, threading.current_thread().name, name, start_ns, end_ns,
                             step))

    def probes(self, rows):
        with self.lock:
            self.db.executemany("INSERT INTO probes VALUES (?,?,?,?,?)",
                                [(self.rank, n, t, c, g) for n, t, c, g in rows])

    def counter(self, name: str, step: int, value: float):
        with self.lock:
            self.db.execute("INSERT INTO counters VALUES (?,?,?,?)", (self.rank, name, step, value))

    def close(self):
        with self.lock:
            self.db.commit()
            self.db.close()


class StepProfiler:
    """Attached to an engine (``engine.profiler = StepProfiler(...)``): two fence
    probes and one host span per step while a session is open; the always-on
    counters (steps, device nanoseconds between the probes) run regardless."""

    def __init__(self, device="cpu", rank: int = 0, probes_per_step: int = 2):
        self.ring = ProbeRing(4096, device)
        self.rank = rank
        self.session: Optional[Session] = None
        self.steps = 0
        self.device_ns = 0
        self.host_ns = 0
        self.probes_per_step = probes_per_step

    def open(self, path: str, meta: Optional[dict] = None) -> Session:
        self.session = Session(path, self.rank, meta)
        return self.session

    def close(self):
        if self.session:
            self.flush()
            self.session.close()
            self.session = None

    @contextmanager
    def step(self, kind: str, step_id: int):
        t0 = time.monotonic_ns()
        if self.probes_per_step:
            self.ring.mark(f"{kind}.begin", step_id)
        try:
            yield
        finally:
            if self.probes_per_step:
                self.ring.mark(f"{kind}.end", step_id)
            t1 = time.monotonic_ns()
            self.steps += 1
            self.host_ns += t1 - t0
            if self.session:
                self.session.span(f"{kind} step", t0, t1, step_id)
            if len(self.ring.pending) >= 64:
                self.flush(wait=False)

    @contextmanager
    def span(self, name: str, step_id: int = -1):
        t0 = time.monotonic_ns()
        try:
            yield
        finally:
            if self.session:
                self.session.span(name, t0, time.monotonic_ns(), step_id)

    def flush(self, wait: bool = True):
        rows = self.ring.collect(wait)
        begin = {}
        for name, t, _, tag in rows:
            if name.endswith(".begin"):
                begin[tag] = t
            elif name.endswith(".end") and tag in begin:
                self.device_ns += t - begin.pop(tag)
        if self.session and rows:
            self.session.probes(rows)

    def counters(self) -> dict:
        return {"steps": self.steps, "device_seconds": self.device_ns / 1e9,
                "host_seconds": self.host_ns / 1e9}
