"""Video sparse attention (VSA): tile selection, the compressed branch and the
block-sparse attention over the selected key blocks.

The sequence is cut into 128-row tiles (``sizes[t]`` valid rows each, the rest
padding).  A layer runs::

    pool_tiles_        zero the padding rows of q, k, v and pool per-tile, per-head means
    scores             <mean_q, mean_k> / sqrt(width) per (head, query tile, key tile)
    select_tiles       the key tiles each query tile keeps (per segment, best `keep`)
    sparse_attention   attend the selected blocks only
    compress_pooled    softmax of the pooled scores over live tiles, weighting pooled values
    add_gated_tiles_   out += compressed[:, tile] * gate

Every function has a CUDA path (csrc/vsa.cu, the block-sparse mode of
csrc/flash_attn_tc05.cu) and a plain PyTorch restatement used on CPU and as
the test oracle.  Reference: crates/nn/src/functional/vsa.rs:1-30,
crates/ops/src/attention/sparse.rs:1-40 (reference project paths).  Tiles are
128 rows here; the reference also serves 64-row tiles.
"""
from __future__ import annotations

import math

import torch

from . import native as N
from .functional import _cuda

TILE = 128
BF16 = torch.bfloat16

N.register_signatures({
    "us_vsa_pool_tiles": (N.I, [N.P, N.P, N.P, N.L, N.L, N.L, N.P, N.P, N.P, N.P, N.I, N.I, N.I,
                                N.P]),
    "us_vsa_scores": (N.I, [N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.P]),
    "us_vsa_select_tiles": (N.I, [N.P, N.P, N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.P]),
    "us_vsa_compress_pooled": (N.I, [N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.P]),
    "us_vsa_add_gated_tiles": (N.I, [N.P, N.L, N.P, N.P, N.L, N.I, N.I, N.I, N.I, N.I, N.P]),
    "us_sparse_attn_block128": (N.I, [N.P, N.P, N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.L, N.L, N.L,
                                      N.L, N.F, N.P, N.P, N.P, N.I, N.P, N.P]),
})


def pool_tiles_(q, k, v, sizes):
    """q, k, v: [tiles * 128, heads, 128] bf16 (row-strided views allowed), padding
    rows zeroed in place.  Returns FP32 means (pq, pk, pv), each [tiles, heads, 128]."""
    rows, H, W = q.shape
    tiles = rows // TILE
    if not _cuda(q):
        outs = []
        pad = (torch.arange(TILE)[None, :] >= sizes[:, None].clamp(0, TILE)).reshape(-1)
        for t in (q, k, v):
            t[pad] = 0
            s = t.float().view(tiles, TILE, H, W).sum(1)
            outs.append(s / sizes.clamp(min=1).float()[:, None, None] *
                        (sizes > 0).float()[:, None, None])
        return tuple(outs)
    pq, pk, pv = (torch.empty(tiles, H, W, dtype=torch.float32, device=q.device) for _ in range(3))
    N.call("us_vsa_pool_tiles", N.ptr(q), N.ptr(k), N.ptr(v), q.stride(0), k.stride(0),
           v.stride(0), N.ptr(sizes), N.ptr(pq), N.ptr(pk), N.ptr(pv), tiles, H, W, N.stream())
    return pq, pk, pv


def scores(pq, pk):
    """[query tiles, heads, W] x [tiles, heads, W] -> [heads, query tiles, tiles] FP32."""
    qt, H, W = pq.shape
    t = pk.shape[0]
    if not _cuda(pq):
        return torch.einsum("ihw,jhw->hij", pq, pk) / math.sqrt(W)
    out = torch.empty(H, qt, t, dtype=torch.float32, device=pq.device)
    N.call("us_vsa_scores", N.ptr(pq), N.ptr(pk), N.ptr(out), qt, t, H, W, N.stream())
    return out


def select_tiles(sc, sizes, segments, keep, query_offset=0):
    """sc [heads, query tiles, tiles] FP32; sizes/segments/keep int32 [tiles] (keep is read
    by segment).  Returns (indices [heads, query tiles, tiles], counts [heads, query tiles])."""
    H, qt, t = sc.shape
    if not _cuda(sc):
        idx = torch.zeros(H, qt, t, dtype=torch.int32)
        cnt = torch.zeros(H, qt, dtype=torch.int32)
        live = sizes > 0
        for h in range(H):
            for i in range(qt):
                g = query_offset + i
                kept = torch.zeros(t, dtype=torch.bool)
                if bool(live[g]):
                    if int(segments[g]) < 0:
                        kept = live.clone()
                    else:
                        kept = live & (segments < 0)
                        for s in torch.unique(segments[live & (segments >= 0)]).tolist():
                            members = torch.nonzero(live & (segments == s)).flatten()
                            # descending score, ties to the lower tile
                            order = sorted(members.tolist(),
                                           key=lambda j: (-float(sc[h, i, j]), j))
                            for j in order[:int(keep[s])]:
                                kept[j] = True
                ks = torch.nonzero(kept).flatten()
                rs = torch.nonzero(~kept).flatten()
                idx[h, i] = torch.cat([ks, rs]).to(torch.int32)
                cnt[h, i] = ks.numel()
        return idx, cnt
    idx = torch.empty(H, qt, t, dtype=torch.int32, device=sc.device)
    cnt = torch.empty(H, qt, dtype=torch.int32, device=sc.device)
    N.call("us_vsa_select_tiles", N.ptr(sc.contiguous()), N.ptr(sizes), N.ptr(segments),
           N.ptr(keep), N.ptr(idx), N.ptr(cnt), H, qt, t, query_offset, N.stream())
    return idx, cnt


def compress_pooled(sc, pv, sizes):
    """softmax_j(sc[h, i, j]) over live tiles, weighting pv [tiles, heads, W] ->
    [heads, query tiles, W] bf16."""
    H, qt, t = sc.shape
    if not _cuda(sc):
        masked = sc.masked_fill(~(sizes > 0)[None, None, :], float("-inf"))
        w = torch.softmax(masked, -1)
        w = torch.nan_to_num(w, nan=0.0)
        return torch.einsum("hij,jhw->hiw", w, pv).to(BF16)
    out = torch.empty(H, qt, pv.shape[2], dtype=BF16, device=sc.device)
    N.call("us_vsa_compress_pooled", N.ptr(sc.contiguous()), N.ptr(pv), N.ptr(sizes), N.ptr(out),
           H, qt, t, pv.shape[2], N.stream())
    return out


def add_gated_tiles_(fine, compressed, gate, tile_offset=0):
    """fine [rows, heads, W] += compressed[heads, tiles, W][:, row // 128 + tile_offset] * gate;
    the product and the sum each round to bf16."""
    rows, H, W = fine.shape
    qt = compressed.shape[1]
    if not _cuda(fine):
        tiles = rows // TILE
        per_row = compressed[:, tile_offset:tile_offset + tiles].float().permute(1, 0, 2)
        per_row = per_row[:, None].expand(tiles, TILE, H, W).reshape(rows, H, W)
        prod = (per_row * gate.float()).to(BF16).float()
        fine.copy_((fine.float() + prod).to(fine.dtype))
        return fine
    N.call("us_vsa_add_gated_tiles", N.ptr(fine), fine.stride(0), N.ptr(compressed), N.ptr(gate),
           gate.stride(0), rows, H, W, qt, tile_offset, N.stream())
    return fine


def sparse_attention(q, k, v, indices, counts, valid, scale, lse=False, out=None):
    """Block-sparse attention: query tile t of head h reads key blocks
    indices[h, t, :counts[h, t]]; key rows at or past valid[block] are not visible.
    q [Tq, H, 128], k/v [Tk, H, 128] in whole tiles.  Returns out (and lse [H, Tq])."""
    Tq, H, D = q.shape
    Tk = k.shape[0]
    if not _cuda(q):
        o = torch.zeros(Tq, H, D, dtype=torch.float32)
        l = torch.full((H, Tq), float("-inf"))
        for h in range(H):
            for t in range(Tq // TILE):
                rows = slice(t * TILE, (t + 1) * TILE)
                cols = []
                for b in indices[h, t, :int(counts[h, t])].tolist():
                    cols += list(range(b * TILE, b * TILE + int(valid[b])))
                if not cols:
                    continue
                s = q[rows, h].float() @ k[cols, h].float().t() * scale
                l[h, rows] = torch.logsumexp(s, -1)
                o[rows, h] = torch.softmax(s, -1) @ v[cols, h].float()
        o = o.to(q.dtype)
        return (o, l) if lse else o
    assert q.dtype == BF16 and q.stride(2) == 1 and q.stride(1) == D
    if out is None:
        out = torch.empty(Tq, H, D, dtype=BF16, device=q.device)
    l = torch.empty(H, Tq, dtype=torch.float32, device=q.device) if lse else None
    cu_q = torch.tensor([0, Tq], dtype=torch.int32, device=q.device)
    cu_k = torch.tensor([0, Tk], dtype=torch.int32, device=q.device)
    N.call("us_sparse_attn_block128", N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(out), N.ptr(cu_q),
           N.ptr(cu_k), Tq, Tk, H, q.stride(0), k.stride(0), v.stride(0), out.stride(0), scale,
           N.ptr(indices), N.ptr(counts), N.ptr(valid), indices.shape[2],
           N.ptr(l) if l is not None else None, N.stream())
    return (out, l) if lse else out


def vsa_attention(q, k, v, gate, sizes, segments, keep, scale):
    """The whole layer on normalised, rotated q/k: fine (sparse) branch plus the
    gated compressed branch.  q, k, v, gate: [tiles * 128, heads, 128] bf16."""
    pq, pk, pv = pool_tiles_(q, k, v, sizes)
    sc = scores(pq, pk)
    idx, cnt = select_tiles(sc, sizes, segments, keep)
    out = sparse_attention(q, k, v, idx, cnt, sizes, scale)
    comp = compress_pooled(sc, pv, sizes)
    return add_gated_tiles_(out, comp, gate)
