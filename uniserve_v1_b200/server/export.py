"""What leaves the deployment for outside consumers: the observation store pushed to an
OpenTelemetry collector, and KV events for KV-aware routers.

**OTLP push.**  Every ``period`` the pusher sends what the store appended since the last push
the collector accepted: ``stats`` rows to ``<endpoint>/v1/metrics`` (a counter as a monotonic
sum point, a gauge as a gauge point, an observation as a gauge point named by its metric),
``events`` rows to ``<endpoint>/v1/logs`` (a log record named by its kind, the row's labels
and revision as attributes).  A push the collector refuses, or that does not reach it, is
sent again with what came after it.  Bodies are OTLP/HTTP in its JSON encoding (the
reference sends the Protobuf encoding of the same messages; a collector accepts both on the
same port).

**KV events.**  Each scheduler publishes which pages its prefix cache holds, in SGLang's ZMQ
format: a step's events are one batch of three frames - the topic, the batch's sequence
number (eight bytes, big-endian, from 0) and ``[ts, events, rank]`` in MessagePack.  Events:
``BlockStored`` (block_hashes, parent_block_hash, token_ids, block_size, medium),
``BlockRemoved`` (block_hashes, medium), ``AllBlocksCleared``.  A page's block hash is the
SHA-256 of the previous page's digest (none for the first) and the page's tokens as
little-endian 32-bit integers, its first eight bytes read as a big-endian signed integer,
so a consumer that hashes tokens itself needs no mapping of this package's page keys.

Reference behaviour: docs/configuration.md:566, :583, :607-611; crates/storage/src/events.rs,
crates/engine/src/scheduler/events.rs (reference project paths).
"""
from __future__ import annotations

import hashlib
import json
import struct
import threading
import time
import urllib.request
from typing import Callable, Optional


# ------------------------------------------------------------------- OTLP push --
def _attrs(d: dict) -> list:
    out = []
    for k, v in d.items():
        if isinstance(v, bool):
            val = {"boolValue": v}
        elif isinstance(v, int):
            val = {"intValue": str(v)}
        elif isinstance(v, float):
            val = {"doubleValue": v}
        else:
            val = {"stringValue": v if isinstance(v, str) else json.dumps(v)}
        out.append({"key": str(k), "value": val})
    return out


def _post_json(url: str, body: dict, timeout: float) -> int:
    req = urllib.request.Request(url, data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"}, method="POST")
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return r.status


class OtlpPusher:
    def __init__(self, store, endpoint: str, deployment: str = "uniserve", period: float = 10.0,
                 post: Optional[Callable] = None, timeout: float = 5.0):
        self.store, self.endpoint = store, endpoint.rstrip("/")
        self.period, self.timeout = period, timeout
        self.post = post or _post_json
        self.resource = {"attributes": _attrs({"service.name": "uniserve",
                                               "uniserve.deployment": deployment})}
        self.sent_stats = 0          # rowid of the last stats row a push delivered
        self.sent_events = 0
        self.pushes = self.failures = 0
        self._stop = threading.Event()
        self.thread: Optional[threading.Thread] = None

    # one push: everything after the last accepted row
    def push_once(self) -> bool:
        with self.store.lock:
            stats = self.store.db.execute(
                "SELECT rowid, ts, name, labels, value, revision FROM stats WHERE rowid > ? "
                "ORDER BY rowid", (self.sent_stats,)).fetchall()
            events = self.store.db.execute(
                "SELECT rowid, ts, kind, request_id, fields, revision FROM events WHERE rowid > ? "
                "ORDER BY rowid", (self.sent_events,)).fetchall()
            counters = {n for (n, _l) in self.store.counters}
        ok = True
        if stats:
            by_name: dict = {}
            for _rid, ts, name, labels, value, rev in stats:
                point = {"timeUnixNano": str(int(ts * 1e9)), "asDouble": float(value),
                         "attributes": _attrs(dict(json.loads(labels), revision=rev))}
                by_name.setdefault(name, []).append(point)
            metrics = []
            for name, points in by_name.items():
                if name in counters:
                    metrics.append({"name": name, "sum": {"dataPoints": points, "isMonotonic": True,
                                                          "aggregationTemporality": 2}})
                else:
                    metrics.append({"name": name, "gauge": {"dataPoints": points}})
            body = {"resourceMetrics": [{"resource": self.resource, "scopeMetrics": [
                {"scope": {"name": "uniserve.observation"}, "metrics": metrics}]}]}
            ok = self._send("/v1/metrics", body)
            if ok:
                self.sent_stats = stats[-1][0]
        if events and ok:
            records = [{"timeUnixNano": str(int(ts * 1e9)), "severityText": "INFO",
                        "body": {"stringValue": kind},
                        "attributes": _attrs(dict(json.loads(fields), request_id=rid_, revision=rev))}
                       for _rid, ts, kind, rid_, fields, rev in events]
            body = {"resourceLogs": [{"resource": self.resource, "scopeLogs": [
                {"scope": {"name": "uniserve.observation"}, "logRecords": records}]}]}
            ok = self._send("/v1/logs", body)
            if ok:
                self.sent_events = events[-1][0]
        return ok

    def _send(self, path: str, body: dict) -> bool:
        try:
            status = self.post(self.endpoint + path, body, self.timeout)
            good = 200 <= int(status) < 300
        except Exception:
            good = False
        self.pushes += 1
        if not good:
            self.failures += 1
        return good

    def start(self) -> None:
        def run():
            while not self._stop.wait(self.period):
                self.push_once()
        self.thread = threading.Thread(target=run, name="otlp-push", daemon=True)
        self.thread.start()

    def stop(self) -> None:
        self._stop.set()
        self.push_once()


# -------------------------------------------------------------------- KV events --
def block_digest(parent: Optional[bytes], tokens) -> bytes:
    """SHA-256 over the previous page's digest (nothing for a first page) and the page's
    tokens as little-endian 32-bit integers."""
    h = hashlib.sha256()
    if parent:
        h.update(parent)
    h.update(struct.pack(f"<{len(tokens)}i", *[int(t) for t in tokens]))
    return h.digest()


def block_hash(digest: bytes) -> int:
    return struct.unpack(">q", digest[:8])[0]


class KvEventPublisher:
    """One publisher per scheduler (``rank`` = the scheduler's number)."""

    def __init__(self, endpoint: Optional[str], topic: str = "kv-events", rank: int = 0,
                 block_size: int = 16, send: Optional[Callable] = None):
        self.topic, self.rank, self.block_size = topic.encode(), rank, block_size
        self.seq = 0
        self.pending: list = []
        self.page_hash: dict = {}             # device page -> block hash it holds
        self._sock = None
        self._send = send
        if send is None and endpoint:
            import zmq
            self._ctx = zmq.Context.instance()
            self._sock = self._ctx.socket(zmq.PUB)
            self._sock.bind(endpoint)
        self.cleared()                        # a publisher starts from an empty view

    # what the scheduler and the block manager report
    def stored(self, pages: list, digests: list, parent: Optional[bytes], tokens: list,
               medium: str = "GPU") -> None:
        hashes = [block_hash(d) for d in digests]
        for p, h in zip(pages, hashes):
            self.page_hash[p] = h
        self.pending.append({"type": "BlockStored", "block_hashes": hashes,
                             "parent_block_hash": block_hash(parent) if parent else None,
                             "token_ids": [int(t) for t in tokens],
                             "block_size": self.block_size, "medium": medium})

    def reused(self, pages: list) -> None:
        """Pages handed out again by the allocator: what they held is gone."""
        gone = [self.page_hash.pop(p) for p in pages if p in self.page_hash]
        if gone:
            self.pending.append({"type": "BlockRemoved", "block_hashes": gone, "medium": "GPU"})

    def cleared(self) -> None:
        self.page_hash.clear()
        self.pending.append({"type": "AllBlocksCleared"})

    def flush(self) -> Optional[list]:
        """One batch per step.  Returns the frames sent (None when nothing was pending)."""
        if not self.pending:
            return None
        import msgpack
        batch, self.pending = self.pending, []
        frames = [self.topic, struct.pack(">Q", self.seq),
                  msgpack.packb([time.time(), batch, self.rank])]
        self.seq += 1
        if self._send is not None:
            self._send(frames)
        elif self._sock is not None:
            self._sock.send_multipart(frames)
        return frames

    def close(self) -> None:
        if self._sock is not None:
            self._sock.close(linger=0)
            self._sock = None
