"""Always-on step counters, fence probes and profile sessions.

* **Fence probes** stamp the GPU's nanosecond timer into pinned host memory at
  chosen points of the stream (``ProbeRing.mark``); reading them back needs no
  synchronisation beyond the step's own read-back.  On a CPU device a probe is
  a host monotonic timestamp, so the same code paths run in CPU tests.
* **Host spans** record (name, start, end) on the calling thread.
* A **session** collects both into one SQLite file per rank (tables ``spans``,
  ``probes``, ``kernels``, ``counters``, ``meta``) which ``tools/profile.py`` turns
  into a Perfetto / Chrome trace.  A session names its collectors:
  ``fence_timeline`` (the probes) and ``timeline``, the activity records of every
  kernel and copy the process launches while the session is open (``KernelTimeline``:
  the CUPTI activity interface through ``torch.profiler``, which also sees the
  launches this package makes through its own library).  A session ends by
  ``close``, after a number of steps or after a duration.

Reference: crates/engine/src/profiling/{markers,session,artifact,collectors}.rs,
docs/profiling.md (reference project paths).  The reference's sampling collectors
(PM / PC sampling, range metrics) need the profiling library's own interfaces and are
not part of this package; asking a session for them is refused by name.
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
            "CREATE TABLE IF NOT EXISTS kernels(rank INT, name TEXT, kind TEXT, stream INT,"
            " start_ns INT, dur_ns INT);"
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

    def kernels(self, rows):
        """rows of (name, kind, stream, start_ns, dur_ns)."""
        with self.lock:
            self.db.executemany("INSERT INTO kernels VALUES (?,?,?,?,?,?)",
                                [(self.rank,) + tuple(r) for r in rows])

    def counter(self, name: str, step: int, value: float):
        with self.lock:
            self.db.execute("INSERT INTO counters VALUES (?,?,?,?)", (self.rank, name, step, value))

    def close(self):
        with self.lock:
            self.db.commit()
            self.db.close()


COLLECTORS = ("fence_timeline", "timeline")
SAMPLING_COLLECTORS = ("pm_sampling", "pc_sampling", "range_metrics")


class KernelTimeline:
    """The ``timeline`` collector: one record per kernel, copy and memset the process runs
    between ``start`` and ``stop`` (name, kind, stream, start, duration).  On a CUDA device
    the records come from the CUPTI activity interface behind ``torch.profiler``; on CPU
    ranks the operator records of the host stand in, so sessions are testable without a GPU.
    Tracing costs launch latency while it runs: sessions are for windows of steps."""

    def __init__(self, device="cpu"):
        self.cuda = torch.device(device).type == "cuda"
        self.prof = None

    def start(self) -> None:
        from torch.profiler import ProfilerActivity, profile
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if self.cuda else [])
        self.prof = profile(activities=acts, record_shapes=False, with_stack=False)
        self.prof.__enter__()

    def stop(self) -> list:
        if self.prof is None:
            return []
        if self.cuda:
            torch.cuda.synchronize()
        self.prof.__exit__(None, None, None)
        from torch.autograd import DeviceType
        want = DeviceType.CUDA if self.cuda else DeviceType.CPU
        rows = []
        if self.cuda:
            try:    # the activity records themselves carry the stream
                for ev in self.prof.profiler.kineto_results.events():
                    if ev.device_type() != want:
                        continue
                    name = ev.name()
                    kind = ("copy" if name.startswith("Memcpy") else
                            "memset" if name.startswith("Memset") else "kernel")
                    rows.append((name, kind, int(ev.device_resource_id()), int(ev.start_ns()),
                                 int(ev.duration_ns())))
                self.prof = None
                return rows
            except AttributeError:
                rows = []
        for e in self.prof.events():
            if e.device_type != want:
                continue
            t0, t1 = e.time_range.start, e.time_range.end          # microseconds
            name = e.name
            kind = ("copy" if name.startswith("Memcpy") else "memset" if name.startswith("Memset")
                    else "kernel") if self.cuda else "host_op"
            rows.append((name, kind, int(getattr(e, "device_index", 0) or 0),
                         int(t0 * 1000), int(max(0.0, t1 - t0) * 1000)))
        self.prof = None
        return rows


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

    def open(self, path: str, meta: Optional[dict] = None, collectors=("fence_timeline",),
             max_steps: Optional[int] = None, max_seconds: Optional[float] = None) -> Session:
        """Starts a session with the named collectors; it closes itself after ``max_steps``
        engine steps or ``max_seconds`` (checked at step ends), whichever comes first."""
        collectors = tuple(collectors or ("fence_timeline",))
        for c in collectors:
            if c in SAMPLING_COLLECTORS:
                raise ValueError(f"collector {c!r} needs the profiling library's sampling "
                                 "interfaces, which this package does not wrap")
            if c not in COLLECTORS:
                raise ValueError(f"unknown collector {c!r}; known: {', '.join(COLLECTORS)}")
        if self.session:
            self.close()
        meta = dict(meta or {}, collectors=",".join(collectors))
        self.session = Session(path, self.rank, meta)
        self.collectors = collectors
        self._left = max_steps
        self._deadline = time.monotonic() + max_seconds if max_seconds else None
        self.timeline = None
        if "timeline" in collectors:
            self.timeline = KernelTimeline(self.ring.device)
            self.timeline.start()
        return self.session

    def close(self):
        if self.session:
            self.flush()
            tl = getattr(self, "timeline", None)
            if tl is not None:
                self.session.kernels(tl.stop())
                self.timeline = None
            self.session.close()
            self.session = None
            self.last_closed = time.time()

    def state(self) -> dict:
        return {"open": self.session is not None,
                "path": self.session.path if self.session else None,
                "collectors": list(getattr(self, "collectors", ())) if self.session else [],
                "steps_left": getattr(self, "_left", None) if self.session else None,
                **self.counters()}

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
            if self.session:
                if getattr(self, "_left", None) is not None:
                    self._left -= 1
                done = (getattr(self, "_left", None) is not None and self._left <= 0) or \
                       (getattr(self, "_deadline", None) is not None
                        and time.monotonic() >= self._deadline)
                if done:
                    self.close()

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


def start_session(engine, collectors, output: Optional[str] = None, steps: Optional[int] = None,
                  seconds: Optional[float] = None, rank: int = 0) -> dict:
    """Opens a session on ``engine`` (attaching a ``StepProfiler`` when it has none): the
    form behind ``[profiling_config.session]`` of a package and ``POST /admin/profile``.
    Without ``output`` the artifact goes to the temporary directory."""
    import os
    import tempfile
    prof = getattr(engine, "profiler", None)
    if prof is None:
        device = getattr(getattr(engine, "model", None), "device", "cpu")
        prof = StepProfiler(device, rank=rank)
        engine.profiler = prof
    if output is None:
        output = os.path.join(tempfile.gettempdir(),
                              f"uniserve-profile-{os.getpid()}-{int(time.time())}-rank{rank}.sqlite")
    elif os.path.isdir(output):
        output = os.path.join(output, f"rank{rank}.sqlite")
    if "timeline" in collectors and not steps and not seconds:
        seconds = 30.0         # activity records accumulate in memory: a timeline is a window
    prof.open(output, {"pid": os.getpid()}, collectors=collectors,
              max_steps=int(steps) if steps else None,
              max_seconds=float(seconds) if seconds else None)
    return prof.state()
