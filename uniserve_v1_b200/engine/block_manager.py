"""Python face of the native paged-KV block manager (``csrc/host/block_manager.cpp``).

Page 0 is the padding sentinel.  Full pages are committed under chained SHA-256
content keys so later requests with the same prefix (and the same isolation
salt) reuse them; the last prompt token is always recomputed
(crates/storage/src/key.rs:1-30, reference project path).
"""
from __future__ import annotations

import ctypes
import hashlib
from typing import Optional, Sequence

import numpy as np

from ..ops import native as N

_bound = False


def _lib():
    global _bound
    lib = N.host()
    if not _bound:
        vp, i32p, u64p = ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_uint64)
        lib.us_bm_create.restype = vp
        lib.us_bm_create.argtypes = [ctypes.c_int, ctypes.c_int]
        lib.us_bm_destroy.argtypes = [vp]
        lib.us_bm_num_free.argtypes = [vp]
        lib.us_bm_num_cached.argtypes = [vp]
        lib.us_bm_alloc.argtypes = [vp, ctypes.c_int, vp]
        lib.us_bm_release.argtypes = [vp, vp, ctypes.c_int]
        lib.us_bm_hash_chain.argtypes = [vp, vp, ctypes.c_int, ctypes.c_int, vp]
        lib.us_bm_match_prefix.argtypes = [vp, vp, ctypes.c_int, vp]
        lib.us_bm_commit.argtypes = [vp, ctypes.c_int, ctypes.c_uint64, ctypes.c_uint64]
        lib.us_bm_enumerate.argtypes = [vp, vp, vp, ctypes.c_int]
        lib.us_bm_stats.argtypes = [vp, vp, vp, vp]
        lib.us_bm_refcount.argtypes = [vp, ctypes.c_int]
        lib.us_bm_flush.argtypes = [vp]
        lib.us_bm_enable_host.argtypes = [vp, ctypes.c_int]
        lib.us_bm_take_offloads.argtypes = [vp, vp, ctypes.c_int]
        lib.us_bm_match_host.argtypes = [vp, vp, ctypes.c_int, vp]
        lib.us_bm_host_stats.argtypes = [vp, vp, vp, vp]
        lib.us_bm_unpin_host.argtypes = [vp, vp, ctypes.c_int]
        _bound = True
    return lib


class BlockManager:
    def __init__(self, num_pages: int, page_size: int = 16, weights_identity: str = "",
                 enable_prefix_cache: bool = True):
        self.lib = _lib()
        self.num_pages = num_pages
        self.kv_events = None        # server.export.KvEventPublisher of this scheduler
        self.page_size = page_size
        self.enable_prefix_cache = enable_prefix_cache
        self.identity = weights_identity
        self.h = self.lib.us_bm_create(num_pages, page_size)
        if not self.h:
            raise ValueError("block manager needs at least 2 pages")

    def __del__(self):
        try:
            if getattr(self, "h", None):
                self.lib.us_bm_destroy(self.h)
                self.h = None
        except Exception:
            pass

    # -------------------------------------------------------------- host tier --
    def enable_host_tier(self, slots: int) -> None:
        """Pages that fall out of the device pool keep their content key in ``slots``
        host slots (LRU among themselves).  The manager only decides; the owner of the
        cache tensors copies: ``take_moves()`` before every step."""
        if slots > 0 and self.lib.us_bm_enable_host(self.h, int(slots)) == 0:
            self.host_slots = int(slots)
            self.fetches: list = []        # (host slot, device page) decided by fetch_prefix

    def take_moves(self):
        """(offloads [(device page, host slot)], fetches [(host slot, device page)]) decided
        since the last call.  Offloads must be copied first: a fetched page may be the one
        an offload just vacated.  A host slot with a pending fetch is pinned from its match
        until this call, so no offload of the batch names it; a slot recycled twice within
        the batch keeps its last page only (each slot appears once in the offloads)."""
        if not getattr(self, "host_slots", 0):
            return [], []
        out = np.empty(2 * 4096, dtype=np.int32)
        by_slot = {}
        while True:
            n = self.lib.us_bm_take_offloads(self.h, out.ctypes.data, 4096)
            for i in range(n):
                by_slot.pop(int(out[2 * i + 1]), None)      # keep the order of the last writers
                by_slot[int(out[2 * i + 1])] = int(out[2 * i])
            if n < 4096:
                break
        offloads = [(page, slot) for slot, page in by_slot.items()]
        fetches, self.fetches = self.fetches, []
        self._unpin([s for s, _ in fetches])
        return offloads, fetches

    def _unpin(self, slots) -> None:
        if slots:
            arr = np.asarray(slots, dtype=np.int32)
            self.lib.us_bm_unpin_host(self.h, arr.ctypes.data, len(arr))

    def fetch_prefix(self, keys: np.ndarray, start: int, limit: int) -> list:
        """Continues a device prefix match at page ``start``: keys the host tier holds get
        a device page each (pinned, committed under their key) and a pending host -> device
        copy.  Returns the new pages (possibly fewer than the host run when the pool is full)."""
        if not getattr(self, "host_slots", 0) or start >= limit:
            return []
        ks = np.ascontiguousarray(keys[start:limit], dtype=np.uint64)
        m, slots = self._match_host(ks)
        pages = []
        for i in range(m):
            got = self.allocate(1)
            if got is None:
                break
            page = got[0]
            owner = self.lib.us_bm_commit(self.h, page, int(ks[i][0]), int(ks[i][1]))
            if owner != page:          # cannot happen after a device miss; keep the books straight
                self.release([page])
                break
            self.fetches.append((int(slots[i]), page))
            pages.append(page)
        self._unpin([int(x) for x in slots[len(pages):m]])      # matched, not fetched
        return pages

    def _match_host(self, ks: np.ndarray):
        """(length of the leading run the host tier holds, its slots); the slots are pinned."""
        slots = np.empty(len(ks), dtype=np.int32)
        m = self.lib.us_bm_match_host(self.h, ks.ctypes.data, len(ks), slots.ctypes.data)
        return m, slots

    def host_stats(self) -> dict:
        a, b, c = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_int()
        self.lib.us_bm_host_stats(self.h, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
        return {"host_hits": a.value, "host_offloads": b.value, "host_used": c.value,
                "host_slots": getattr(self, "host_slots", 0)}

    # ------------------------------------------------------------------ verbs --
    @property
    def num_free(self) -> int:
        return self.lib.us_bm_num_free(self.h)

    @property
    def num_cached(self) -> int:
        return self.lib.us_bm_num_cached(self.h)

    def can_allocate(self, n: int) -> bool:
        return n <= self.num_free

    def allocate(self, n: int) -> Optional[list]:
        if n == 0:
            return []
        out = np.empty(n, dtype=np.int32)
        rc = self.lib.us_bm_alloc(self.h, n, out.ctypes.data)
        if rc != 0:
            return None
        pages = out.tolist()
        if self.kv_events is not None:      # whatever these pages cached is gone
            self.kv_events.reused(pages)
        return pages

    def release(self, pages: Sequence[int]) -> None:
        if not pages:
            return
        arr = np.asarray(pages, dtype=np.int32)
        self.lib.us_bm_release(self.h, arr.ctypes.data, len(arr))

    def page_keys(self, token_ids: Sequence[int], salt: Optional[str] = None) -> np.ndarray:
        """Chained keys of every full page of ``token_ids``: uint64 [n_full, 2]."""
        seed = hashlib.sha256((self.identity + "\0" + (salt or "")).encode()).digest()
        toks = np.asarray(token_ids, dtype=np.int32)
        n_full = len(toks) // self.page_size
        keys = np.zeros((max(n_full, 1), 2), dtype=np.uint64)
        seed_buf = (ctypes.c_uint8 * 32).from_buffer_copy(seed)
        self.lib.us_bm_hash_chain(ctypes.addressof(seed_buf), toks.ctypes.data, len(toks),
                                  self.page_size, keys.ctypes.data)
        return keys[:n_full]

    def chain_seed(self, salt: Optional[str] = None) -> bytes:
        """Root of a request's key chain (weights identity + isolation salt)."""
        return hashlib.sha256((self.identity + "\0" + (salt or "")).encode()).digest()

    def chain_next(self, state: bytes, page_tokens: Sequence[int]):
        """One link of the chain in Python: (next state, key of the page) - the same bytes
        as ``page_keys`` produces, so a request extends its chain by the page it just filled
        instead of hashing its whole history again."""
        assert len(page_tokens) == self.page_size
        state = hashlib.sha256(state + np.asarray(page_tokens, dtype="<i4").tobytes()).digest()
        k = np.frombuffer(state[:16], dtype="<u8")
        return state, (int(k[0]), int(k[1]))

    def match_prefix(self, keys: np.ndarray) -> list:
        """Pins and returns the pages of the longest cached leading run."""
        if not self.enable_prefix_cache or len(keys) == 0:
            return []
        keys = np.ascontiguousarray(keys, dtype=np.uint64)
        out = np.empty(len(keys), dtype=np.int32)
        m = self.lib.us_bm_match_prefix(self.h, keys.ctypes.data, len(keys), out.ctypes.data)
        return out[:m].tolist()

    def peek_prefix(self, keys: np.ndarray) -> int:
        """Pages of the longest cached leading run, without keeping them (a routing probe)."""
        pages = self.match_prefix(keys)
        if pages:
            self.release(pages)
        return len(pages)

    def committed(self):
        """(keys uint64 [n, 2], pages int32 [n]) of every content-keyed device page, the most
        recently released last."""
        cap = self.num_pages
        keys = np.zeros((cap, 2), dtype=np.uint64)
        pages = np.zeros(cap, dtype=np.int32)
        n = self.lib.us_bm_enumerate(self.h, keys.ctypes.data, pages.ctypes.data, cap)
        return keys[:n], pages[:n]

    def commit(self, page: int, key) -> int:
        if not self.enable_prefix_cache:
            return page
        return self.lib.us_bm_commit(self.h, int(page), int(key[0]), int(key[1]))

    def refcount(self, page: int) -> int:
        return self.lib.us_bm_refcount(self.h, page)

    def flush(self) -> int:
        if self.kv_events is not None:
            self.kv_events.cleared()
        return self.lib.us_bm_flush(self.h)

    def stats(self) -> dict:
        a, b, c = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
        self.lib.us_bm_stats(self.h, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
        return {"hits": a.value, "lookups": b.value, "evictions": c.value,
                "free": self.num_free, "cached": self.num_cached, "pages": self.num_pages}
