"""Copy manifests: which slices of which rank's KV pages go where when a request's cache
moves between deployments of different parallel layouts.

A deployment with tensor-parallel degree ``tp`` over ``heads`` KV heads gives rank r the
heads ``[r * heads / tp, (r + 1) * heads / tp)``; when ``tp`` exceeds ``heads`` every head is
replicated on ``tp / heads`` consecutive ranks.  A manifest lists, for every destination rank,
the source ranks to read and the head interval to take from each (replicated sources are read
from the copy whose rank is nearest the destination's, so that the copies spread over the
sources).  ``route`` picks each destination rank's shards out of the exporting ranks'
hand-offs; ``engine/handoff.py::import_request`` then re-cuts them (``reshard_heads``).

Reference behaviour: crates/storage/src/manifest (resharding plans between parallel
configurations; reference project path).
"""
from __future__ import annotations

from dataclasses import dataclass


def head_range(heads: int, tp: int, rank: int) -> tuple:
    """(first head, head count) of ``rank`` in a degree-``tp`` layout over ``heads`` heads."""
    if tp <= heads:
        assert heads % tp == 0, (heads, tp)
        n = heads // tp
        return rank * n, n
    assert tp % heads == 0, (heads, tp)
    return rank // (tp // heads), 1


@dataclass(frozen=True)
class Copy:
    src_rank: int
    dst_rank: int
    head_lo: int          # global index of the first head moved
    heads: int
    src_offset: int       # position of head_lo inside the source rank's shard
    dst_offset: int       # position inside the destination rank's shard


@dataclass(frozen=True)
class CopyManifest:
    heads: int
    src_tp: int
    dst_tp: int
    copies: tuple

    @staticmethod
    def plan(heads: int, src_tp: int, dst_tp: int) -> "CopyManifest":
        copies = []
        for d in range(dst_tp):
            dlo, dn = head_range(heads, dst_tp, d)
            h = dlo
            while h < dlo + dn:
                # source ranks that hold head h (several when the source replicates heads)
                holders = [s for s in range(src_tp)
                           if head_range(heads, src_tp, s)[0] <= h <
                           sum(head_range(heads, src_tp, s))]
                s = min(holders, key=lambda r: (abs(r * dst_tp - d * src_tp), r))
                slo, sn = head_range(heads, src_tp, s)
                take = min(slo + sn, dlo + dn) - h
                copies.append(Copy(s, d, h, take, h - slo, h - dlo))
                h += take
        return CopyManifest(heads, src_tp, dst_tp, tuple(copies))

    def sources_of(self, dst_rank: int) -> list:
        return sorted({c.src_rank for c in self.copies if c.dst_rank == dst_rank})

    def bytes_moved(self, pages: int, page_size: int, head_dim: int, layers: int,
                    elem: int = 2) -> int:
        per_head = 2 * pages * page_size * head_dim * elem * layers        # K and V planes
        return sum(c.heads for c in self.copies) * per_head

    def route(self, exports: dict) -> dict:
        """``exports[src_rank]`` -> for every destination rank the hand-offs it needs."""
        return {d: [exports[s] for s in self.sources_of(d)] for d in range(self.dst_tp)}

    def check(self) -> None:
        """Every destination head is written exactly once, from a rank that holds it."""
        for d in range(self.dst_tp):
            dlo, dn = head_range(self.heads, self.dst_tp, d)
            got = sorted((c.head_lo, c.heads) for c in self.copies if c.dst_rank == d)
            at = dlo
            for lo, n in got:
                assert lo == at and n >= 1, (d, got)
                at += n
            assert at == dlo + dn, (d, got)
        for c in self.copies:
            slo, sn = head_range(self.heads, self.src_tp, c.src_rank)
            assert slo <= c.head_lo and c.head_lo + c.heads <= slo + sn, c
            assert c.src_offset == c.head_lo - slo
