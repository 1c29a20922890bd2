"""Hot restart of a single-process deployment: a successor process of the same command takes
the listening socket over while the process it replaces finishes the requests it took.

``POST /admin/restart`` starts ``python -m uniserve_v1_b200 serve ... --listen-fd N --ready-fd M``
with the listening socket and one end of a pipe inherited.  The successor loads the model,
starts serving on the SAME socket (both processes accept from one kernel queue for a moment)
and writes a line to the pipe (before that it reads the file of cached KV pages this process
wrote for it, ``--prefix-cache``: what was cached stays cached); this process then stops accepting and exits once its
connections have ended.  No connection is refused: one that arrives meanwhile waits in the
listener's queue until one of the two accepts it.  If the successor exits before it reports,
this process keeps serving as before.  The successor needs its own share of the GPU's memory
while both live (weights and a KV cache): a deployment sized to the whole GPU sleeps first
(``POST /admin/sleep``) or restarts cold.

Reference behaviour: crates/daemon/src/restart.rs:1-40 (reference project path; there the
engines are separate processes that the successor adopts, here the engine lives in the serving
process, so the successor builds its own).
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import threading
import time
from typing import Optional


class HotRestart:
    def __init__(self, server, listener, argv: list, snapshot=None):
        """``snapshot()``: writes this process's cached KV pages to a file and returns its
        path (``engine/prefix_store.py``); the successor reads it before it serves."""
        self.server, self.listener = server, listener
        self.snapshot = snapshot
        # the successor repeats this process's command line without hand-over arguments
        self.argv = self._strip(argv, ("--listen-fd", "--ready-fd", "--prefix-cache"))
        self.state = "serving"          # serving | starting | handed_over | failed
        self.successor: Optional[int] = None
        self.error: Optional[str] = None
        self._lock = threading.Lock()

    @staticmethod
    def _strip(argv: list, flags: tuple) -> list:
        out, skip = [], False
        for a in argv:
            if skip:
                skip = False
                continue
            if a in flags:
                skip = True
                continue
            if any(a.startswith(f + "=") for f in flags):
                continue
            out.append(a)
        return out

    def begin(self, timeout: float = 600.0) -> dict:
        with self._lock:
            if self.state == "starting":
                return self.status()
            self.state, self.error = "starting", None
        r, w = os.pipe()
        os.set_inheritable(w, True)
        fd = self.listener.fileno()
        cmd = [sys.executable, "-m", "uniserve_v1_b200"] + self.argv + \
            ["--listen-fd", str(fd), "--ready-fd", str(w)]
        if self.snapshot is not None:
            try:
                cmd += ["--prefix-cache", self.snapshot()]
            except Exception as e:       # the restart goes on with a cold cache
                self.error = f"prefix cache not saved: {e}"
        env = dict(os.environ)
        for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
            env.pop(k, None)
        proc = subprocess.Popen(cmd, pass_fds=(fd, w), env=env)
        os.close(w)
        self.successor = proc.pid
        threading.Thread(target=self._wait, args=(proc, r, timeout), daemon=True,
                         name="hot-restart").start()
        return self.status()

    def _wait(self, proc, r: int, timeout: float) -> None:
        deadline = time.monotonic() + timeout
        buf = b""
        os.set_blocking(r, False)
        try:
            while time.monotonic() < deadline and b"\n" not in buf:
                if proc.poll() is not None:
                    break
                try:
                    chunk = os.read(r, 4096)
                    if chunk:
                        buf += chunk
                        continue
                except BlockingIOError:
                    pass
                time.sleep(0.05)
        finally:
            os.close(r)
        ok = False
        if b"\n" in buf:
            try:
                ok = json.loads(buf.split(b"\n")[0]).get("state") == "listening"
            except ValueError:
                ok = False
        if ok:
            self.state = "handed_over"
            self.server.should_exit = True        # stop accepting, finish what was taken
        else:
            self.state = "failed"
            self.error = "the successor ended before it served" if proc.poll() is not None \
                else "the successor did not report in time"
            if proc.poll() is None:
                proc.terminate()

    def status(self) -> dict:
        return {"state": self.state, "pid": os.getpid(), "successor_pid": self.successor,
                "error": self.error}


class Standby:
    """A parked second process beside the serving one (``profiling_config.standby``).

    The serving process starts it with the listening socket and the read end of a pipe
    inherited.  The standby loads the model, builds its engine, optionally releases its KV
    cache again (``standby_storage``: ``suspended`` or ``auto``), reports ``parked`` and blocks
    on the pipe.  When the serving process ends for ANY reason the kernel closes the pipe's
    write end: the standby wakes, restores what it released, and serves on the same socket -
    connections that arrived meanwhile waited in the listener's queue - then starts a standby of
    its own (the next generation).  A clean shutdown writes ``stop`` first and the standby
    leaves too.  Requests that were in flight on the failed process are lost with it; their
    clients (or the replica router's migration) send them again.

    Reference behaviour: crates/daemon/src/standby/mod.rs:1-30, docs/configuration.md:534-535
    (reference project paths; there a standby repeats a rank of an engine group under a
    daemon, here the whole single-process deployment).
    """

    def __init__(self, listener, argv: list, generation: int = 0):
        self.listener = listener
        self.argv = HotRestart._strip(argv, ("--listen-fd", "--ready-fd", "--standby-fd",
                                             "--generation"))
        self.generation = generation
        self.state = "none"             # none | starting | parked | failed
        self.pid: Optional[int] = None
        self._w: Optional[int] = None

    def start(self) -> None:
        r, w = os.pipe()                # the standby blocks on r; this process keeps w
        pr, pw = os.pipe()              # the standby reports "parked" on pw
        os.set_inheritable(r, True)
        os.set_inheritable(pw, True)
        fd = self.listener.fileno()
        cmd = [sys.executable, "-m", "uniserve_v1_b200"] + self.argv + \
            ["--listen-fd", str(fd), "--standby-fd", str(r), "--ready-fd", str(pw),
             "--generation", str(self.generation + 1)]
        env = dict(os.environ)
        for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
            env.pop(k, None)
        proc = subprocess.Popen(cmd, pass_fds=(fd, r, pw), env=env)
        os.close(r)
        os.close(pw)
        self._w, self.pid, self.state = w, proc.pid, "starting"

        def watch():
            buf = b""
            try:
                while b"\n" not in buf:
                    chunk = os.read(pr, 4096)
                    if not chunk:
                        break
                    buf += chunk
            finally:
                os.close(pr)
            self.state = "parked" if b"parked" in buf else "failed"
        threading.Thread(target=watch, daemon=True, name="standby-watch").start()

    def stop(self) -> None:
        """Clean shutdown of the serving process: the standby leaves too."""
        if self._w is not None:
            try:
                os.write(self._w, b"stop\n")
                os.close(self._w)
            except OSError:
                pass
            self._w = None

    def status(self) -> dict:
        return {"state": self.state, "pid": self.pid, "generation": self.generation}


class PrefixSnapshots:
    """The serving process of a deployment with a standby writes its cached KV pages to a
    file every ``period_s`` seconds (``engine/prefix_store.py``, at most ``max_bytes``), so
    that a standby promoted after the process died starts with the prefixes of the last
    snapshot instead of an empty cache.  The file is named after the listening port, which
    the two processes share."""

    def __init__(self, service, path: str, period_s: float, max_bytes: int = 256 << 20):
        self.service, self.path, self.period_s, self.max_bytes = service, path, period_s, max_bytes
        self.written = 0
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True, name="prefix-snapshots")

    @staticmethod
    def path_for(listener, state_dir: Optional[str]) -> str:
        base = state_dir or ("/dev/shm" if os.path.isdir("/dev/shm") else "/tmp")
        return os.path.join(base, f"uniserve-prefix-port{listener.getsockname()[1]}.kv")

    def start(self) -> None:
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()

    def _run(self) -> None:
        from ..engine.prefix_store import save_prefix_cache
        while not self._stop.wait(self.period_s):
            try:
                self.service.call(lambda e: save_prefix_cache(e, self.path, self.max_bytes))
                self.written += 1
            except Exception:       # an engine that sleeps or restarts: try again next period
                pass


def park(standby_fd: int, ready_fd: Optional[int], engine, storage: str,
         prefix_path: Optional[str] = None) -> bool:
    """The standby's side: release what ``storage`` says, report, block until the serving
    process ends.  Returns True when this process is to serve now, False when it was told to
    leave.  With ``prefix_path`` the promoted standby reads the serving process's last
    snapshot of cached KV pages before it serves."""
    suspended = storage in ("suspended", "auto") and engine is not None and hasattr(engine, "sleep")
    if suspended:
        engine.sleep(1)
    if ready_fd is not None:
        os.write(ready_fd, json.dumps({"state": "parked", "pid": os.getpid()}).encode() + b"\n")
        os.close(ready_fd)
    buf = b""
    while True:
        chunk = os.read(standby_fd, 64)
        if not chunk:
            break                       # the writer is gone: the serving process ended
        buf += chunk
        if b"stop" in buf:
            return False
    os.close(standby_fd)
    if suspended:
        engine.wake()
    if prefix_path and engine is not None and hasattr(engine, "blocks") and \
            os.path.exists(prefix_path):
        from ..engine.prefix_store import load_prefix_cache
        got = load_prefix_cache(engine, prefix_path, remove=False)
        print(f"standby: prefix cache {got}", file=sys.stderr)
    return True


RESTARTS_ENV = "UNISERVE_RESTARTS"        # "consecutive relaunches:time of the last one"


def restart_delay(relaunches: int, restart_s: float, max_s: float) -> float:
    """Seconds a leader waits before it relaunches its ranks: nothing the first time, then
    ``restart_s`` doubling with every further relaunch in a row, up to ``max_s``
    (``storage_config.child_restart_s`` / ``child_restart_max_s`` of the reference's policy
    package: a deployment whose ranks die at once does not spin)."""
    if relaunches <= 0:
        return 0.0
    return float(min(max_s, restart_s * (2 ** min(relaunches - 1, 30))))


class Supervision:
    """The leader of a multi-rank deployment watches the rank processes it started.  When one
    ends while the deployment serves, the deployment cannot go on (its collectives would wait
    for the missing rank): the leader marks the engine failed (``/health`` answers 503, so a
    router moves the requests), stops the other ranks, and - unless ``relaunch`` is off - replaces
    its own image with a fresh ``serve`` of the next generation that inherits the listening
    socket, which starts the ranks again.  Connections that arrive meanwhile wait in the
    listener's queue.  Relaunches that follow one another within ``restart_max_s`` back off
    (``restart_delay``); an image that served longer than that starts the count again.

    Reference behaviour: crates/daemon/src/supervision (child supervision and relaunch of a
    failure domain; reference project path).
    """

    def __init__(self, children: list, listener, argv: list, generation: int, on_failure=None,
                 relaunch: bool = True, period: float = 0.5, restart_s: float = 5.0,
                 restart_max_s: float = 300.0, clock=time.time):
        self.restart_s, self.restart_max_s, self.clock = float(restart_s), float(restart_max_s), clock
        self.relaunches, self.waiting_s = 0, 0.0
        try:
            n, _, ts = os.environ.get(RESTARTS_ENV, "").partition(":")
            if n and clock() - float(ts) < self.restart_max_s:
                self.relaunches = max(0, int(n))
        except ValueError:
            pass
        self.children, self.listener = children, listener
        self.argv = HotRestart._strip(argv, ("--listen-fd", "--ready-fd", "--standby-fd",
                                             "--generation"))
        self.generation, self.on_failure, self.relaunch = generation, on_failure, relaunch
        self.period = period
        self.failed: Optional[str] = None
        self._stop = threading.Event()
        self.thread = threading.Thread(target=self._run, daemon=True, name="supervision")

    def start(self) -> None:
        self.thread.start()

    def stop(self) -> None:
        self._stop.set()

    def status(self) -> dict:
        return {"ranks": [{"rank": i + 1, "pid": c.pid, "alive": c.poll() is None}
                          for i, c in enumerate(self.children)],
                "failed": self.failed, "generation": self.generation,
                "relaunches": self.relaunches, "waiting_s": self.waiting_s}

    def _run(self) -> None:
        while not self._stop.wait(self.period):
            for i, c in enumerate(self.children):
                code = c.poll()
                if code is None:
                    continue
                self.failed = f"rank {i + 1} (pid {c.pid}) ended with code {code}"
                if self.on_failure is not None:
                    try:
                        self.on_failure(self.failed)
                    except Exception:
                        pass
                for other in self.children:
                    if other.poll() is None:
                        other.terminate()
                for other in self.children:
                    try:
                        other.wait(timeout=10)
                    except Exception:
                        other.kill()
                if self.relaunch and self.listener is not None:
                    self.waiting_s = restart_delay(self.relaunches, self.restart_s,
                                                   self.restart_max_s)
                    if self.waiting_s and self._stop.wait(self.waiting_s):
                        return                           # stopped while backing off
                    self._exec()
                return

    def _exec(self) -> None:
        fd = self.listener.fileno()
        os.set_inheritable(fd, True)
        env = {k: v for k, v in os.environ.items()
               if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT")}
        env[RESTARTS_ENV] = f"{self.relaunches + 1}:{self.clock():.3f}"
        cmd = [sys.executable, "-m", "uniserve_v1_b200"] + self.argv + \
            ["--listen-fd", str(fd), "--generation", str(self.generation + 1)]
        sys.stdout.flush()
        sys.stderr.flush()
        os.execve(sys.executable, cmd, env)
