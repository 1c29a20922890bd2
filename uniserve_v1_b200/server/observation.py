"""Observation store: two SQL tables, ``stats`` and ``events``, queried with SQL at
``/admin/query`` and rendered as Prometheus text at ``/metrics``.

Metric names follow the reference (``uniserve_ttft_seconds``,
``uniserve_tpot_seconds``, ``uniserve_requests_total{outcome}``,
``uniserve_kv_cache_used_pages{tier}``, ``uniserve_kernel_launches_total`` ...;
README.md:113, crates/daemon/src/observation/mod.rs:1-34, reference project paths).
The store is SQLite in memory (the reference embeds DataFusion); every row
carries the configuration revision it was measured under.
"""
from __future__ import annotations

import json
import sqlite3
import threading
import time
from typing import Optional


class ObservationStore:
    def __init__(self, revision: int = 0):
        self.db = sqlite3.connect(":memory:", check_same_thread=False)
        self.lock = threading.Lock()
        self.revision = revision
        self.db.executescript(
            "CREATE TABLE stats (ts REAL, name TEXT, labels TEXT, value REAL, revision INTEGER);"
            "CREATE TABLE events (ts REAL, kind TEXT, request_id TEXT, fields TEXT, revision INTEGER);"
            "CREATE INDEX stats_name ON stats(name); CREATE INDEX events_kind ON events(kind);")
        self.counters: dict = {}
        self.gauges: dict = {}
        self.hist: dict = {}

    @staticmethod
    def _key(name, labels):
        return name, tuple(sorted((labels or {}).items()))

    def inc(self, name: str, labels: Optional[dict] = None, by: float = 1.0) -> None:
        k = self._key(name, labels)
        with self.lock:
            self.counters[k] = self.counters.get(k, 0.0) + by

    def set(self, name: str, value: float, labels: Optional[dict] = None) -> None:
        with self.lock:
            self.gauges[self._key(name, labels)] = float(value)

    def observe(self, name: str, value: float, labels: Optional[dict] = None) -> None:
        k = self._key(name, labels)
        with self.lock:
            s = self.hist.setdefault(k, [0, 0.0])
            s[0] += 1
            s[1] += value
            self.db.execute("INSERT INTO stats VALUES (?,?,?,?,?)",
                            (time.time(), name, json.dumps(dict(k[1])), value, self.revision))

    def event(self, kind: str, request_id: str = "", **fields) -> None:
        with self.lock:
            self.db.execute("INSERT INTO events VALUES (?,?,?,?,?)",
                            (time.time(), kind, request_id, json.dumps(fields), self.revision))

    def snapshot(self) -> None:
        """Writes the current counters and gauges as one row each (once a second
        in the serving loop)."""
        now = time.time()
        with self.lock:
            rows = [(now, n, json.dumps(dict(l)), v, self.revision)
                    for (n, l), v in list(self.counters.items()) + list(self.gauges.items())]
            self.db.executemany("INSERT INTO stats VALUES (?,?,?,?,?)", rows)

    def query(self, sql: str) -> dict:
        s = sql.strip().rstrip(";")
        if not s.lower().startswith(("select", "with")) or ";" in s:
            raise ValueError("only a single SELECT statement is served")
        with self.lock:
            cur = self.db.execute(s)
            cols = [c[0] for c in cur.description]
            return {"columns": cols, "rows": [list(r) for r in cur.fetchall()]}

    def prometheus(self) -> str:
        def fmt(labels):
            return "{" + ",".join(f'{k}="{v}"' for k, v in labels) + "}" if labels else ""
        out = []
        with self.lock:
            for (n, l), v in sorted(self.counters.items()):
                out.append(f"{n}{fmt(l)} {v}")
            for (n, l), v in sorted(self.gauges.items()):
                out.append(f"{n}{fmt(l)} {v}")
            for (n, l), (c, s) in sorted(self.hist.items()):
                out.append(f"{n}_count{fmt(l)} {c}")
                out.append(f"{n}_sum{fmt(l)} {s}")
        return "\n".join(out) + "\n"
