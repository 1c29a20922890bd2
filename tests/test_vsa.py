"""Video sparse attention: selection rule on CPU, CUDA kernels against the CPU
restatements."""
import math

import pytest
import torch

from uniserve_v1_b200.ops import vsa as V

BF = torch.bfloat16


def _case(tiles=6, H=2, seed=0, dev="cpu"):
    g = torch.Generator().manual_seed(seed)
    rows = tiles * 128
    mk = lambda: (torch.randn(rows, H, 128, generator=g) * 0.7).to(BF).to(dev)
    sizes = torch.full((tiles,), 128, dtype=torch.int32)
    sizes[-1] = 50                       # partial last tile
    segments = torch.zeros(tiles, dtype=torch.int32)
    segments[0] = -1                     # a tile every query attends (text)
    keep = torch.zeros(tiles, dtype=torch.int32)
    keep[0] = 2
    return mk(), mk(), mk(), mk(), sizes.to(dev), segments.to(dev), keep.to(dev)


def test_select_rule_cpu():
    sc = torch.tensor([[[0.1, 0.9, 0.5, 0.9, -1.0, 0.3]]])          # one head, one query tile
    sizes = torch.tensor([128, 128, 128, 128, 128, 0], dtype=torch.int32)
    segments = torch.tensor([-1, 0, 0, 0, 0, 0], dtype=torch.int32)
    keep = torch.tensor([2, 0, 0, 0, 0, 0], dtype=torch.int32)
    idx, cnt = V.select_tiles(sc, sizes, segments, keep, query_offset=1)
    # tile 0 (outside the segments) always; of segment 0 the two best: 1 and 3 (tie -> lower first)
    assert cnt.tolist() == [[3]] and idx[0, 0, :3].tolist() == [0, 1, 3]
    assert idx[0, 0, 3:].tolist() == [2, 4, 5]
    # a query tile outside the segments keeps every live tile; an empty one keeps none
    idx, cnt = V.select_tiles(sc, sizes, segments, keep, query_offset=0)
    assert cnt.tolist() == [[5]]
    idx, cnt = V.select_tiles(sc, sizes, segments, keep, query_offset=5)
    assert cnt.tolist() == [[0]]


def test_vsa_layer_cpu_full_keep_equals_dense():
    """Keeping every tile, the fine branch is dense attention over the valid rows."""
    q, k, v, gate, sizes, segments, keep = _case()
    keep[0] = 99
    pq, pk, pv = V.pool_tiles_(q, k, v, sizes)
    sc = V.scores(pq, pk)
    idx, cnt = V.select_tiles(sc, sizes, segments, keep)
    assert (cnt == 6).all()
    out = V.sparse_attention(q, k, v, idx, cnt, sizes, 1 / math.sqrt(128))
    used = 5 * 128 + 50
    s = torch.einsum("qhd,khd->hqk", q.float(), k[:used].float()) / math.sqrt(128)
    ref = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v[:used].float())
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
def test_vsa_kernels_match_cpu():
    q, k, v, gate, sizes, segments, keep = _case(tiles=9, H=3, seed=3)
    qc, kc, vc = q.clone(), k.clone(), v.clone()
    d = lambda t: t.cuda()
    qg, kg, vg = d(q), d(k), d(v)
    pq, pk, pv = V.pool_tiles_(qc, kc, vc, sizes)
    gq, gk, gv = V.pool_tiles_(qg, kg, vg, d(sizes))
    torch.testing.assert_close(gk.cpu(), pk, atol=1e-5, rtol=1e-5)
    assert torch.equal(kg.cpu(), kc)                     # padding rows zeroed alike
    sc = V.scores(pq, pk)
    gs = V.scores(gq, gk)
    torch.testing.assert_close(gs.cpu(), sc, atol=1e-5, rtol=1e-4)
    keep[0] = 3
    idx, cnt = V.select_tiles(sc, sizes, segments, keep)
    gi, gc = V.select_tiles(d(sc), d(sizes), d(segments), d(keep))
    assert torch.equal(gc.cpu(), cnt) and torch.equal(gi.cpu(), idx)
    out, lse = V.sparse_attention(qc, kc, vc, idx, cnt, sizes, 1 / math.sqrt(128), lse=True)
    go, gl = V.sparse_attention(qg, kg, vg, gi, gc, d(sizes), 1 / math.sqrt(128), lse=True)
    torch.testing.assert_close(go.float().cpu(), out.float(), atol=2e-2, rtol=2e-2)
    live = torch.isfinite(lse)
    torch.testing.assert_close(gl.cpu()[live], lse[live], atol=2e-3, rtol=2e-3)
    comp = V.compress_pooled(sc, pv, sizes)
    gcomp = V.compress_pooled(d(sc), d(pv), d(sizes))
    torch.testing.assert_close(gcomp.float().cpu(), comp.float(), atol=1e-2, rtol=1e-2)
    fine = out.clone()
    V.add_gated_tiles_(fine, comp, gate)
    gfine = d(out)
    V.add_gated_tiles_(gfine, d(comp), d(gate))
    torch.testing.assert_close(gfine.float().cpu(), fine.float(), atol=1e-2, rtol=1e-2)
    # the whole layer
    whole = V.vsa_attention(d(q), d(k), d(v), d(gate), d(sizes), d(segments), d(keep),
                            1 / math.sqrt(128))
    ref = V.vsa_attention(q.clone(), k.clone(), v.clone(), gate, sizes, segments, keep,
                          1 / math.sqrt(128))
    torch.testing.assert_close(whole.float().cpu(), ref.float(), atol=3e-2, rtol=3e-2)
