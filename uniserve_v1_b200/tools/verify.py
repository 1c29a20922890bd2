"""Bounded exhaustive checks of the KV block manager.

Every sequence of operations up to a depth - allocate, release, commit under a content
key, match a key chain, flush - is run against a fresh native block manager
(``csrc/host/block_manager.cpp``) next to a small abstract model that only tracks what a
client can know: which pages it holds how often, and which key it committed on which
page.  After every operation the invariants are checked:

  holds       refcount(page) equals the client's holds, for every page
  exclusive   allocate never hands out a page that is held
  capacity    allocate(n) succeeds exactly when n <= num_free, and num_free equals the
              pages nobody holds (free or cached-and-evictable)
  content     match returns a leading run of the chain, each page carrying the key it
              was committed under, and a chain whose pages were never reused is found
  pinning     matched pages are held (they cannot be evicted under the reader)

``record`` / ``replay`` do the same for real traffic: the calls an engine makes while it
serves requests (shared prefixes, preemption, eviction) are recorded and run again on a
fresh manager, which must answer identically and keep the invariants.

``explore_site_protocol`` walks every interleaving of the flag / epoch protocol of the fused
collectives for a few ranks, sites and passes (stale or overwritten partials, deadlock).

``mutants`` are wrappers that break one behaviour each (a dropped release, a match that
does not pin, a commit under the wrong key, a stale page kept after reuse); the checker
has to flag every one of them, which shows the invariants have teeth.

    python -m uniserve_v1_b200.tools.verify --pages 5 --depth 5

Reference behaviour: tools/verification/README.md (enumeration, replay and mutation checks
of the buffer pool and the KV data plane; the TLA+ models themselves are not restated) -
reference project path.
"""
from __future__ import annotations

import argparse
import json
from typing import Optional

import numpy as np


class Violation(Exception):
    pass


class Client:
    """What a client of the block manager knows."""

    def __init__(self, bm, pages: int):
        self.bm, self.pages = bm, pages
        self.holds: dict = {}          # page -> count
        self.key_of: dict = {}         # page -> key index (until the page is handed out again)

    # ---- operations (return False when not applicable in this state) ----
    def alloc(self, n: int) -> bool:
        free_before = self.bm.num_free
        got = self.bm.allocate(n)
        if (got is not None) != (n <= free_before):
            raise Violation(f"capacity: allocate({n}) with {free_before} free -> {got}")
        if got is None:
            return True
        if len(set(got)) != n or any(p <= 0 or p >= self.pages for p in got):
            raise Violation(f"exclusive: allocate returned {got}")
        for p in got:
            if self.holds.get(p, 0):
                raise Violation(f"exclusive: page {p} handed out while held")
            self.holds[p] = 1
            self.key_of.pop(p, None)               # reused: its old content is gone
        return True

    def release(self, i: int) -> bool:
        held = sorted(p for p, c in self.holds.items() if c)
        if i >= len(held):
            return False
        p = held[i]
        self.bm.release([p])
        self.holds[p] -= 1
        return True

    def commit(self, i: int, k: int, keys) -> bool:
        held = sorted(p for p, c in self.holds.items() if c)
        if i >= len(held):
            return False
        p = held[i]
        if p in self.key_of or k in self.key_of.values():
            return False                           # one key per page, one page per key here
        self.bm.commit(p, keys[k])
        self.key_of[p] = k
        return True

    def match(self, n: int, keys) -> bool:
        chain = np.ascontiguousarray(keys[:n], dtype=np.uint64)
        got = self.bm.match_prefix(chain)
        if len(got) > n:
            raise Violation(f"content: match of {n} keys returned {got}")
        for j, p in enumerate(got):
            if self.key_of.get(p) != j:
                raise Violation(f"content: page {p} returned for key {j}, holds {self.key_of.get(p)}")
            self.holds[p] = self.holds.get(p, 0) + 1
        want = 0
        by_key = {k: p for p, k in self.key_of.items()}
        while want < n and want in by_key:
            want += 1
        if len(got) != want:
            raise Violation(f"content: chain of {want} cached pages, match found {len(got)}")
        return True

    def flush(self) -> bool:
        self.bm.flush()
        for p in [p for p in self.key_of if not self.holds.get(p, 0)]:
            del self.key_of[p]
        return True

    # ---- invariants ----
    def check(self) -> None:
        held = 0
        for p in range(1, self.pages):
            c = self.holds.get(p, 0)
            if self.bm.refcount(p) != c:
                raise Violation(f"holds: page {p} refcount {self.bm.refcount(p)}, client holds {c}")
            held += 1 if c else 0
        if self.bm.num_free != self.pages - 1 - held:
            raise Violation(f"capacity: num_free {self.bm.num_free}, "
                            f"{self.pages - 1 - held} pages are not held")


def operations(n_keys: int) -> list:
    ops = [("alloc", 1), ("alloc", 2), ("flush",)]
    ops += [("release", i) for i in range(2)]
    ops += [("commit", i, k) for i in range(2) for k in range(n_keys)]
    ops += [("match", n) for n in range(1, n_keys + 1)]
    return ops


def explore(make_bm, pages: int = 5, depth: int = 5, n_keys: int = 2) -> dict:
    """Runs every operation sequence up to ``depth``; returns counts and the first
    violation (sequence + message) if any."""
    ops = operations(n_keys)
    probe = make_bm(pages)
    keys = probe.page_keys(list(range(n_keys * probe.page_size)))
    ran = {"sequences": 0, "operations": 0, "violation": None}

    def run(seq) -> Optional[str]:
        c = Client(make_bm(pages), pages)
        try:
            for op in seq:
                kind = op[0]
                ok = c.alloc(op[1]) if kind == "alloc" else \
                    c.release(op[1]) if kind == "release" else \
                    c.commit(op[1], op[2], keys) if kind == "commit" else \
                    c.match(op[1], keys) if kind == "match" else c.flush()
                if not ok:
                    return "skip"
                c.check()
                ran["operations"] += 1
        except Violation as v:
            return str(v)
        return None

    def dfs(seq):
        if ran["violation"]:
            return
        if seq:
            r = run(seq)
            if r == "skip":
                return
            ran["sequences"] += 1
            if r:
                ran["violation"] = {"sequence": [list(o) for o in seq], "message": r}
                return
        if len(seq) < depth:
            for op in ops:
                dfs(seq + [op])
    dfs([])
    return ran


# ------------------------------------------------------------------ mutants --
def mutants(base):
    """(name, factory) of block managers with one broken behaviour each."""
    class DropsRelease(base):
        def release(self, pages):
            self._n = getattr(self, "_n", 0) + 1
            if self._n % 2:
                super().release(pages)

    class MatchDoesNotPin(base):
        def match_prefix(self, keys):
            got = super().match_prefix(keys)
            if got:
                super().release(got)
            return got

    class CommitsWrongKey(base):
        def commit(self, page, key):
            return super().commit(page, (int(key[0]) ^ 1, int(key[1])))

    class KeepsStalePage(base):
        def allocate(self, n):
            got = super().allocate(n)
            if got and getattr(self, "_last", None) and n == 1:
                super().release(got)
                return [self._last]
            if got:
                self._last = got[0]
            return got
    return [("drops every second release", DropsRelease), ("match does not pin", MatchDoesNotPin),
            ("commit under another key", CommitsWrongKey), ("hands out a held page", KeepsStalePage)]


# ---------------------------------------------------------------- host tier --
def explore_host_tier(make_bm, pages: int = 4, host_slots: int = 1, depth: int = 5,
                      n_keys: int = 2, prefix: tuple = ()) -> dict:
    """Every operation sequence up to ``depth`` on a block manager with a host tier of
    ``host_slots`` slots, with the page *contents* simulated: an allocated page is written
    with a fresh tag, a commit records the tag under its key, the copies of ``take_moves``
    run in its order (offloads, then fetches) once per "step".  ``fetch`` matches the key
    chain on the device first and continues on the host tier, as the scheduler does.
    Checked after every step: a page returned for key k holds the tag committed under k
    (so a host slot with a pending fetch was not recycled by an offload of the same step,
    including when host_slots <= matched + offloads), and no host slot is written twice in
    one batch.  ``prefix`` is run before every enumerated sequence (``HOST_FULL`` leaves the
    first key on the host tier and every device page held, one of them committed under the
    second key: the state from which two more operations reach the recycled-slot fault).
    ``host_mutant`` is a manager without the pins; the check has to flag it."""
    probe = make_bm(pages)
    keys = probe.page_keys(list(range(n_keys * probe.page_size)))
    ops = [("alloc", 1), ("alloc", 2), ("step",)] + [("release", i) for i in range(2)] + \
        [("commit", i, k) for i in range(2) for k in range(n_keys)] + \
        [("fetch", n) for n in range(1, n_keys + 1)]
    ran = {"sequences": 0, "violation": None}

    def run(seq):
        bm = make_bm(pages)
        bm.enable_host_tier(host_slots)
        dev, host, tag_of_key, held, key_of, fresh = {}, {}, {}, [], {}, [0]
        pending = []                    # (page, key index) fetched, checked after the moves

        def step():
            off, fet = bm.take_moves()
            if len({s for _, s in off}) != len(off):
                raise Violation(f"host: a slot written twice in one batch {off}")
            for page, slot in off:
                host[slot] = dev.get(page)
            for slot, page in fet:
                dev[page] = host.get(slot)
            for page, k in pending:
                if dev.get(page) != tag_of_key[k]:
                    raise Violation(f"host: page {page} fetched for key {k} holds "
                                    f"{dev.get(page)}, committed {tag_of_key[k]}")
            pending.clear()
        try:
            for op in list(prefix) + list(seq):
                kind = op[0]
                if kind == "alloc":
                    got = bm.allocate(op[1])
                    if got is None:
                        continue
                    step()              # pages about to be overwritten are saved first
                    for p_ in got:
                        fresh[0] += 1
                        dev[p_] = fresh[0]
                        key_of.pop(p_, None)
                        held.append(p_)
                elif kind == "release":
                    if op[1] >= len(held):
                        return "skip"
                    bm.release([held.pop(op[1])])
                elif kind == "commit":
                    if op[1] >= len(held) or held[op[1]] in key_of or op[2] in tag_of_key:
                        return "skip"
                    if op[2] > 0 and (op[2] - 1) not in tag_of_key:
                        return "skip"                  # chains are committed in order
                    page = held[op[1]]
                    bm.commit(page, keys[op[2]])
                    key_of[page] = op[2]
                    tag_of_key[op[2]] = dev[page]
                elif kind == "fetch":
                    chain = np.ascontiguousarray(keys[:op[1]], dtype=np.uint64)
                    got = bm.match_prefix(chain)
                    pending.extend((p_, j) for j, p_ in enumerate(got))   # its copy may be queued
                    more = bm.fetch_prefix(chain, len(got), op[1])
                    pending.extend((p_, len(got) + j) for j, p_ in enumerate(more))
                    held.extend(list(got) + list(more))
                    for j, p_ in enumerate(more):
                        key_of[p_] = len(got) + j
                else:
                    step()
            step()
        except Violation as v:
            return str(v)
        return None

    def dfs(seq):
        if ran["violation"]:
            return
        if seq:
            r = run(seq)
            if r == "skip":
                return
            ran["sequences"] += 1
            if r:
                ran["violation"] = {"sequence": [list(o) for o in seq], "message": r}
                return
        if len(seq) < depth:
            for op in ops:
                dfs(seq + [op])
    dfs([])
    return ran


# 4 pages (3 usable), 1 host slot: key 0 committed and pushed to the host, key 1 committed on
# a held device page, no free page left
HOST_FULL = (("alloc", 1), ("commit", 0, 0), ("release", 0), ("alloc", 2), ("alloc", 1),
             ("step",), ("commit", 0, 1))


def host_mutant(base):
    """A block manager whose matched host slots are not pinned (they return to the LRU list
    at once, so an offload of the same step may recycle them before their fetch)."""
    class UnpinnedHostSlots(base):
        def _match_host(self, ks):
            m, slots = super()._match_host(ks)
            self._unpin([int(x) for x in slots[:m]])
            return m, slots

        def _unpin(self, slots):
            if not getattr(self, "_in_match", False):
                self._in_match = True
                super()._unpin(slots)
                self._in_match = False
    return UnpinnedHostSlots


# ------------------------------------------------------------ trace / replay --
def record(bm) -> list:
    """Starts recording every call a client makes on ``bm`` (allocate, release, commit,
    match_prefix, flush) with its result; returns the list that fills up."""
    trace: list = []

    def wrap(name, encode):
        inner = getattr(bm, name)

        def call(*args):
            out = inner(*args)
            trace.append(encode(args, out))
            return out
        setattr(bm, name, call)
    wrap("allocate", lambda a, out: ("allocate", int(a[0]), None if out is None else list(out)))
    wrap("release", lambda a, out: ("release", [int(p) for p in a[0]]))
    wrap("commit", lambda a, out: ("commit", int(a[0]), (int(a[1][0]), int(a[1][1]))))
    wrap("match_prefix", lambda a, out: ("match", [(int(k[0]), int(k[1])) for k in a[0]],
                                         list(out)))
    wrap("flush", lambda a, out: ("flush",))
    return trace


def replay(trace: list, make_bm, pages: int) -> dict:
    """Runs a recorded serving trace against a fresh block manager: the calls must give the
    recorded results again (the manager is deterministic) and the client-side invariants
    (holds, exclusivity, capacity, content) must hold after every call."""
    bm = make_bm(pages)
    holds: dict = {}
    key_of: dict = {}
    n = 0
    try:
        for op in trace:
            kind = op[0]
            if kind == "allocate":
                free = bm.num_free
                got = bm.allocate(op[1])
                if got != op[2]:
                    raise Violation(f"replay: allocate({op[1]}) gave {got}, recorded {op[2]}")
                if (got is not None) != (op[1] <= free):
                    raise Violation(f"capacity: allocate({op[1]}) with {free} free -> {got}")
                for p in got or []:
                    if holds.get(p, 0):
                        raise Violation(f"exclusive: page {p} handed out while held")
                    holds[p] = 1
                    key_of.pop(p, None)
            elif kind == "release":
                bm.release(op[1])
                for p in op[1]:
                    holds[p] = holds.get(p, 0) - 1
                    if holds[p] < 0:
                        raise Violation(f"holds: page {p} released more often than held")
            elif kind == "commit":
                bm.commit(op[1], op[2])
                if op[2] not in key_of.values():
                    key_of[op[1]] = op[2]
            elif kind == "match":
                got = bm.match_prefix(np.asarray(op[1], dtype=np.uint64).reshape(-1, 2))
                if list(got) != op[2]:
                    raise Violation(f"replay: match gave {list(got)}, recorded {op[2]}")
                for j, p in enumerate(got):
                    if key_of.get(p) != op[1][j]:
                        raise Violation(f"content: page {p} returned for another key")
                    holds[p] = holds.get(p, 0) + 1
            else:
                bm.flush()
                for p in [p for p in key_of if not holds.get(p, 0)]:
                    del key_of[p]
            n += 1
            for p in range(1, pages):
                if bm.refcount(p) != holds.get(p, 0):
                    raise Violation(f"holds: page {p} refcount {bm.refcount(p)}, "
                                    f"client holds {holds.get(p, 0)} after call {n}")
    except Violation as v:
        return {"calls": n, "violation": str(v)}
    return {"calls": n, "violation": None}


# ------------------------------------------------------------ site protocol --
def explore_site_protocol(world: int = 2, sites: int = 2, passes: int = 2) -> dict:
    """Every interleaving of the fused collectives' flag protocol (``csrc/fused/peer_comm.cu``)
    for ``world`` ranks that run ``passes`` forward passes over ``sites`` collective sites.

    A rank's program at a site: write its partial into its own buffer of the site; store the
    site's next epoch into its flag slot on every peer (one store per peer, any order); wait
    until every peer's slot on this rank shows that epoch; read every peer's buffer.  Kernels
    of one rank run in stream order, ranks run freely against each other.  Checked: a read
    always finds the partial of the *same* pass (neither the previous pass's nor one a fast
    rank already overwrote), and no interleaving blocks for good.  Buffers are reused one
    pass later without a second barrier, which is safe only because another site's barrier
    lies in between: with ``sites = 1`` the exploration finds the overwrite."""
    peers = [[q for q in range(world) if q != r] for r in range(world)]
    prog = []
    for r in range(world):
        ops = []
        for n in range(passes):
            for st in range(sites):
                ops.append(("write", st, n))
                ops.extend(("announce", st, n, q) for q in peers[r])
                ops.append(("wait", st, n))
                ops.extend(("read", st, n, q) for q in peers[r])
        prog.append(ops)
    # state: program counters, buffer[r][site] = pass of its content, flag[r][site][from] = epoch
    start = (tuple([0] * world), tuple(tuple([-1] * sites) for _ in range(world)),
             tuple(tuple(tuple([0] * world) for _ in range(sites)) for _ in range(world)))
    seen, frontier, steps = {start}, [start], 0
    while frontier:
        nxt = []
        for pcs, buf, flag in frontier:
            moved = False
            for r in range(world):
                if pcs[r] >= len(prog[r]):
                    continue
                op = prog[r][pcs[r]]
                b2, f2 = buf, flag
                if op[0] == "write":
                    row = list(buf[r])
                    row[op[1]] = op[2]
                    b2 = buf[:r] + (tuple(row),) + buf[r + 1:]
                elif op[0] == "announce":
                    q, st = op[3], op[1]
                    slots = list(flag[q][st])
                    slots[r] = op[2] + 1
                    site_rows = list(flag[q])
                    site_rows[st] = tuple(slots)
                    f2 = flag[:q] + (tuple(site_rows),) + flag[q + 1:]
                elif op[0] == "wait":
                    if any(flag[r][op[1]][q] < op[2] + 1 for q in peers[r]):
                        continue                     # blocked
                else:
                    got = buf[op[3]][op[1]]
                    if got != op[2]:
                        return {"states": len(seen), "violation":
                                f"rank {r} reads rank {op[3]}'s site {op[1]} in pass {op[2]} "
                                f"and finds pass {got}"}
                moved = True
                steps += 1
                state = (pcs[:r] + (pcs[r] + 1,) + pcs[r + 1:], b2, f2)
                if state not in seen:
                    seen.add(state)
                    nxt.append(state)
            if not moved and any(pcs[r] < len(prog[r]) for r in range(world)):
                return {"states": len(seen), "violation": f"deadlock at {pcs}"}
        frontier = nxt
    return {"states": len(seen), "violation": None}


def explore_programs(programs: list, n_bufs: int, n_bars: int) -> dict:
    """Generic explorer: ``programs[r]`` is rank r's list of steps, run in order; ranks
    interleave freely.  Steps: ("store", rank, buf, value) writes slot [buf][me] of ``rank``'s
    memory; ("announce", rank, bar, epoch) raises flag [bar][me] on ``rank``; ("wait", bar,
    epoch, peers) blocks until every peer's flag on this rank reached the epoch; ("load", buf,
    src, value) reads slot [buf][src] of the own memory and expects ``value``."""
    world = len(programs)
    zero = tuple(tuple([None] * world) for _ in range(n_bufs))
    start = (tuple([0] * world), tuple(zero for _ in range(world)),
             tuple(tuple(tuple([0] * world) for _ in range(n_bars)) for _ in range(world)))

    def put(mem, rank, a, b, val):
        row = list(mem[rank][a])
        row[b] = val
        inner = list(mem[rank])
        inner[a] = tuple(row)
        return mem[:rank] + (tuple(inner),) + mem[rank + 1:]
    seen, frontier = {start}, [start]
    while frontier:
        nxt = []
        for pcs, mem, flag in frontier:
            moved = False
            for r in range(world):
                if pcs[r] >= len(programs[r]):
                    continue
                op = programs[r][pcs[r]]
                m2, f2 = mem, flag
                if op[0] == "store":
                    m2 = put(mem, op[1], op[2], r, op[3])
                elif op[0] == "announce":
                    f2 = put(flag, op[1], op[2], r, op[3])
                elif op[0] == "wait":
                    if any(flag[r][op[1]][q] < op[2] for q in op[3]):
                        continue
                else:
                    got = mem[r][op[1]][op[2]]
                    if got != op[3]:
                        return {"states": len(seen), "violation":
                                f"rank {r} loads buffer {op[1]} slot {op[2]}: expects {op[3]}, finds {got}"}
                moved = True
                state = (pcs[:r] + (pcs[r] + 1,) + pcs[r + 1:], m2, f2)
                if state not in seen:
                    seen.add(state)
                    nxt.append(state)
            if not moved and any(pcs[r] < len(programs[r]) for r in range(world)):
                return {"states": len(seen), "violation": f"deadlock at {pcs}"}
        frontier = nxt
    return {"states": len(seen), "violation": None}


def explore_ulysses_protocol(world: int = 2, layers: int = 2, second_barrier: bool = True) -> dict:
    """The sequence-parallel attention of the video transformer (``parallel/ulysses.py``): per
    layer every rank stores its share of q / k / v into every peer's QKV buffer (the projection
    GEMM's epilogue), barrier, reads the whole QKV buffer and pushes its attention output into
    every peer's output buffer (the flash kernel's epilogue), barrier, reads the output buffer
    (the local output projection).  Both buffers are reused by the next layer without a third
    barrier; the exploration shows that the two barriers per layer suffice in every interleaving
    (a fast rank's next-layer q / k / v cannot land under a slow rank's attention, nor its next
    output under a slow rank's projection).  Without the second barrier a rank reads the output
    buffer before its peers pushed into it, which the exploration reports.

    The expert exchange (``csrc/fused/ep_exchange.cu``) has the same shape with flags in place
    of barriers: dispatch into every expert rank's window, "dispatched" flags, sort / GEMMs read
    the window and push into the token owners' combine buffers, "combined" flags, combine reads;
    its single-buffered windows are covered by the same exploration."""
    QKV, ATT = 0, 1
    programs = []
    for r in range(world):
        peers = [q for q in range(world) if q != r]
        ops = []
        for layer in range(layers):
            for q in range(world):
                ops.append(("store", q, QKV, layer))
            ops.extend(("announce", q, 0, layer + 1) for q in peers)
            ops.append(("wait", 0, layer + 1, peers))
            ops.extend(("load", QKV, q, layer) for q in range(world))
            for q in range(world):
                ops.append(("store", q, ATT, layer))
            if second_barrier:
                ops.extend(("announce", q, 1, layer + 1) for q in peers)
                ops.append(("wait", 1, layer + 1, peers))
            ops.extend(("load", ATT, q, layer) for q in range(world))
        programs.append(ops)
    return explore_programs(programs, 2, 2)


def explore_tp_protocol(world: int = 2, blocks: int = 3, norm_sites: int = 2) -> dict:
    """Tensor parallelism with the collectives fused into the GEMMs (``parallel/tp_fused.py``):
    per MLP block the normalised rows of the previous block sit in every rank's gathered buffer
    (written by all owners), barrier B0, the column-parallel GEMM reads them and the row-parallel
    GEMM stores partial sums into the owners' slot buffers, barrier B1, the owner sums its slots
    and stores the next normalised rows into every rank's gathered buffer of the next block.
    The slot buffer is reused by every block and the gathered buffers alternate; the exploration
    passes with two buffers and also with one (``norm_sites = 1``): a peer's B1 arrival already
    lies after its reads of the gathered rows, so the alternation is a margin, not a need."""
    SLOTS = norm_sites
    programs = []
    for r in range(world):
        peers = [q for q in range(world) if q != r]
        ops = [("store", q, 0, -1) for q in range(world)]          # rows of the embedding
        for b in range(blocks):
            src, dst = b % norm_sites, (b + 1) % norm_sites
            ops.extend(("announce", q, 0, b + 1) for q in peers)
            ops.append(("wait", 0, b + 1, peers))
            ops.extend(("load", src, q, b - 1) for q in range(world))      # gathered rows
            ops.extend(("store", q, SLOTS, b) for q in range(world))       # reduce-scatter
            ops.extend(("announce", q, 1, b + 1) for q in peers)
            ops.append(("wait", 1, b + 1, peers))
            ops.extend(("load", SLOTS, q, b) for q in range(world))        # slot sum
            ops.extend(("store", q, dst, b) for q in range(world))         # all-gather
        programs.append(ops)
    return explore_programs(programs, norm_sites + 1, 2)


def main(argv=None) -> int:
    from ..engine.block_manager import BlockManager
    ap = argparse.ArgumentParser(prog="uniserve_v1_b200.tools.verify")
    ap.add_argument("--pages", type=int, default=5)
    ap.add_argument("--depth", type=int, default=5)
    ap.add_argument("--keys", type=int, default=2)
    a = ap.parse_args(argv)
    mk = lambda cls: (lambda pages: cls(pages, page_size=4))
    report = {"native": explore(mk(BlockManager), a.pages, a.depth, a.keys), "mutants": {}}
    for name, cls in mutants(BlockManager):
        r = explore(mk(cls), a.pages, min(a.depth, 4), a.keys)
        report["mutants"][name] = "caught" if r["violation"] else "MISSED"
    report["host_tier"] = {f"{hs} host slot(s)": explore_host_tier(mk(BlockManager), 4, hs,
                                                                   min(a.depth, 5), a.keys)
                           for hs in (1, 2)}
    report["mutants"]["host slots not pinned"] = "caught" if explore_host_tier(
        mk(host_mutant(BlockManager)), 4, 1, 3, 2, HOST_FULL)["violation"] else "MISSED"
    report["host_tier"]["1 host slot, from a full tier"] = explore_host_tier(
        mk(BlockManager), 4, 1, 4, 2, HOST_FULL)
    report["site_protocol"] = {"2 ranks x 2 sites x 3 passes": explore_site_protocol(2, 2, 3),
                               "3 ranks x 2 sites x 2 passes": explore_site_protocol(3, 2, 2),
                               "1 site (must fail)": explore_site_protocol(2, 1, 2)}
    report["tp_protocol"] = {"2 ranks x 4 blocks": explore_tp_protocol(2, 4),
                             "3 ranks x 2 blocks": explore_tp_protocol(3, 2),
                             "one gathered buffer": explore_tp_protocol(2, 3, 1)}
    report["ulysses_protocol"] = {"2 ranks x 3 layers": explore_ulysses_protocol(2, 3),
                                  "3 ranks x 2 layers": explore_ulysses_protocol(3, 2),
                                  "one barrier per layer (must fail)":
                                      explore_ulysses_protocol(2, 2, second_barrier=False)}
    bad = report["native"]["violation"] or "MISSED" in report["mutants"].values() or \
        any(r["violation"] for r in report["host_tier"].values()) or \
        report["site_protocol"]["2 ranks x 2 sites x 3 passes"]["violation"] or \
        report["site_protocol"]["3 ranks x 2 sites x 2 passes"]["violation"] or \
        not report["site_protocol"]["1 site (must fail)"]["violation"] or \
        report["tp_protocol"]["2 ranks x 4 blocks"]["violation"] or \
        report["tp_protocol"]["3 ranks x 2 blocks"]["violation"] or \
        report["tp_protocol"]["one gathered buffer"]["violation"] or \
        report["ulysses_protocol"]["2 ranks x 3 layers"]["violation"] or \
        report["ulysses_protocol"]["3 ranks x 2 layers"]["violation"] or \
        not report["ulysses_protocol"]["one barrier per layer (must fail)"]["violation"]
    print(json.dumps(report, indent=1))
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
