"""GPU quotas: what the engines of one process may hold on a device, and what they hold.

A device has one ledger.  Every engine that serves from the device (a deployment's serving
engine, the target engine an epoch update builds beside it, a standby) is a *holder*: it states
the fraction of the device its deployment may use and reserves its items against the ledger -

    weights        the model's weight tensors (once per holder, tied tensors once)
    cache_segment  the KV cache planes (pages x bytes per page, page scales included)
    graph_pool     captured graphs and their workspaces
    staging        pinned / device staging of the host KV tier and of hand-offs
    exclusive      anything else a holder keeps to itself

The limit is ``floor(total x fraction)``; while holders that state different fractions hold
storage on the device, the smaller limit holds.  A reservation that would take the usage of
the device past the limit is refused (``QuotaExceeded``) and nothing changes, so the usage
never exceeds the limit.  Reserving an item again replaces its amount (shrinking always
succeeds).  A storage that several holders map - the weights of a model that an epoch update's
target engine shares with the serving engine - is reserved by each of them under one ``key``
and counts once, for as long as any of them holds it.  A segment that a successor takes over
from its predecessor moves with ``hand_over``: the reservation changes holder, nothing is
released and allocated.

The ledger counts reservations, not allocations: it is what ``LLMEngine`` divides (what is
left after weights and graph pool goes to KV pages), what ``sleep`` gives back and ``wake``
takes again, and what ``GET /admin/status`` reports per device.

Reference behaviour: crates/storage-server/src/quota.rs (quotas per GPU and deployment, items,
limit as a fraction of the whole GPU, the smaller of two epochs' limits, refusal past the
limit, hand-over of segments at a commit), crates/engine/src/memory/division.rs (quota
division); reference project paths.  The reference keeps the ledger in its Storage Server,
across processes; this one is per process.
"""
from __future__ import annotations

import threading
from typing import Optional

ITEMS = ("weights", "cache_segment", "graph_pool", "staging", "exclusive")


class QuotaExceeded(RuntimeError):
    def __init__(self, holder: str, item: str, asked: int, usage: int, limit: int):
        super().__init__(f"quota: {holder} asked {asked} bytes of {item}; "
                         f"{usage} of {limit} bytes are reserved")
        self.holder, self.item, self.asked, self.usage, self.limit = \
            holder, item, asked, usage, limit


class DeviceQuota:
    def __init__(self, total: int, name: str = "cpu"):
        self.total, self.name = int(total), name
        self.fractions: dict[str, float] = {}
        self.items: dict[tuple, int] = {}
        self.keys: dict[tuple, str] = {}        # (holder, item) -> key of a shared storage
        self.refused = 0
        self.forced = 0
        self._lock = threading.Lock()

    # ------------------------------------------------------------- holders --
    def state_fraction(self, holder: str, fraction: float) -> None:
        if not (0.0 < fraction <= 1.0):
            raise ValueError("a quota's fraction is in (0, 1]")
        with self._lock:
            self.fractions[holder] = float(fraction)

    def _limit(self, extra: Optional[float] = None) -> int:
        held = {h for (h, _), b in self.items.items() if b > 0}
        fr = [f for h, f in self.fractions.items() if h in held]
        if extra is not None:
            fr.append(extra)
        return int(self.total * min(fr)) if fr else self.total

    def limit(self) -> int:
        with self._lock:
            return self._limit()

    def _usage(self) -> int:
        """Bytes reserved on the device: a shared storage counts once (its largest
        reservation)."""
        total, shared = 0, {}
        for k, b in self.items.items():
            key = self.keys.get(k)
            if key is None:
                total += b
            else:
                shared[key] = max(shared.get(key, 0), b)
        return total + sum(shared.values())

    def usage(self, holder: Optional[str] = None) -> int:
        """Bytes reserved on the device, or what ``holder`` itself reserved."""
        with self._lock:
            if holder is None:
                return self._usage()
            return sum(b for (h, _), b in self.items.items() if h == holder)

    # -------------------------------------------------------- reservations --
    def reserve(self, holder: str, item: str, nbytes: int, key: Optional[str] = None,
                force: bool = False) -> int:
        """Sets ``holder``'s reservation of ``item`` to ``nbytes``.  Growing is refused past
        the limit; the holder's own fraction counts from its first reservation.  ``key`` names
        a storage shared with other holders.  ``force`` records a reservation that is past the
        limit instead of refusing it (for memory that is allocated already; counted in
        ``forced``)."""
        if item not in ITEMS:
            raise ValueError(f"unknown quota item {item!r}")
        nbytes = max(0, int(nbytes))
        slot = (holder, item)
        with self._lock:
            had = self.items.get(slot, 0)
            before = self._usage()
            old_key = self.keys.get(slot)
            if nbytes:
                self.items[slot] = nbytes
                if key is not None:
                    self.keys[slot] = key
                else:
                    self.keys.pop(slot, None)
            else:
                self.items.pop(slot, None)
                self.keys.pop(slot, None)
            after = self._usage()
            if after > before:
                limit = self._limit()
                if after > limit:
                    if not force:
                        if had:                                  # undo
                            self.items[slot] = had
                            if old_key is not None:
                                self.keys[slot] = old_key
                            else:
                                self.keys.pop(slot, None)
                        else:
                            self.items.pop(slot, None)
                            self.keys.pop(slot, None)
                        self.refused += 1
                        raise QuotaExceeded(holder, item, nbytes, before, limit)
                    self.forced += 1
            return nbytes

    def room(self, holder: str, fraction: Optional[float] = None) -> int:
        """Bytes ``holder`` could still reserve."""
        with self._lock:
            f = fraction if fraction is not None else self.fractions.get(holder)
            return max(0, self._limit(f) - self._usage())

    def release(self, holder: str, item: Optional[str] = None) -> int:
        """Ends ``holder``'s reservation of ``item`` (of everything, and its stated fraction,
        without an item).  Returns the bytes released."""
        with self._lock:
            keys = [k for k in self.items if k[0] == holder and (item is None or k[1] == item)]
            before = self._usage()
            for k in keys:
                self.items.pop(k)
                self.keys.pop(k, None)
            freed = before - self._usage()
            if item is None:
                self.fractions.pop(holder, None)
            return freed

    def hand_over(self, src: str, dst: str, item: str) -> int:
        """``dst`` takes over ``src``'s reservation of ``item`` (added to what it holds
        already).  The usage of the device does not change, so nothing is refused."""
        with self._lock:
            moved = self.items.pop((src, item), 0)
            key = self.keys.pop((src, item), None)
            if moved:
                self.items[(dst, item)] = self.items.get((dst, item), 0) + moved
                if key is not None:
                    self.keys[(dst, item)] = key
            return moved

    # --------------------------------------------------------------- report --
    def report(self) -> dict:
        with self._lock:
            holders: dict[str, dict] = {}
            for (h, it), b in sorted(self.items.items()):
                holders.setdefault(h, {"fraction": self.fractions.get(h), "items": {}})
                holders[h]["items"][it] = b
            for h, d in holders.items():
                d["bytes"] = sum(d["items"].values())
            usage = self._usage()
            limit = self._limit()
            return {"device": self.name, "total": self.total, "limit": limit, "usage": usage,
                    "room": max(0, limit - usage), "refused": self.refused,
                    "forced": self.forced, "holders": holders}


_LEDGERS: dict[str, DeviceQuota] = {}
_LEDGERS_LOCK = threading.Lock()


def _device_total(device) -> int:
    import torch
    dev = torch.device(device)
    if dev.type == "cuda":
        return int(torch.cuda.get_device_properties(dev).total_memory)
    try:
        import psutil
        return int(psutil.virtual_memory().total)
    except Exception:                                   # pragma: no cover - psutil is present
        return 64 << 30


def quota_of(device, total: Optional[int] = None) -> DeviceQuota:
    """The process-wide ledger of ``device`` (made on first use; ``total`` overrides the
    device's own size, for tests and for a device shared with other deployments)."""
    import torch
    dev = torch.device(device)
    name = dev.type if dev.index is None and dev.type != "cuda" else \
        f"{dev.type}:{dev.index if dev.index is not None else torch.cuda.current_device()}"
    with _LEDGERS_LOCK:
        q = _LEDGERS.get(name)
        if q is None or (total is not None and q.total != int(total) and not q.items):
            q = DeviceQuota(total if total is not None else _device_total(dev), name)
            _LEDGERS[name] = q
        return q


def all_reports() -> list:
    with _LEDGERS_LOCK:
        ledgers = list(_LEDGERS.values())
    return [q.report() for q in ledgers]


def divide(quota: DeviceQuota, holder: str, fraction: float, weights: int, graph_pool: int,
           per_page: int, want_pages: int, min_pages: int = 64,
           weights_key: Optional[str] = None) -> int:
    """Quota division of one engine: states the fraction, reserves the weights and the graph
    pool, and gives what is left - at most ``want_pages`` - to the KV cache.  When not even
    ``min_pages`` fit, the weights' or the pool's refusal (``QuotaExceeded``) tells why."""
    quota.state_fraction(holder, fraction)
    try:
        quota.reserve(holder, "weights", weights, key=weights_key)
        quota.reserve(holder, "graph_pool", graph_pool)
        pages = int(min(want_pages, quota.room(holder) // max(1, per_page)))
        if pages < min_pages:
            pages = min(min_pages, want_pages)
        quota.reserve(holder, "cache_segment", pages * per_page)
    except QuotaExceeded:
        quota.release(holder)
        raise
    return pages
