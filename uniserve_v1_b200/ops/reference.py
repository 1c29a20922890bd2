"""Plain PyTorch FP32 restatements of every fused op.

These are the numerics oracle for the CUDA kernels (GPU tests compare a kernel
with the function of the same name here) and the CPU execution path of the
models.  They follow the formulas the reference keeps beside each device launch
(crates/nn/src/functional/mod.rs:173-199, reference project path): FP32
arithmetic, one rounding to the output dtype at the end.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x, w, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if w is not None:
        y = y * w.float()
    return y.to(x.dtype)


def add_rmsnorm(x, residual, w, eps):
    """residual (FP32) += x; returns (rmsnorm(residual) * w, residual)."""
    r = x.float() if residual is None else residual.float() + x.float()
    y = r * torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype), r


def modulated_rmsnorm(x, w, table, idx, vectors_per_row, shift_slot, scale_slot, eps):
    xf = x.float()
    n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if w is not None:
        n = n * w.float()
    rows = idx.long() * vectors_per_row
    shift = table[rows + shift_slot]
    scale = table[rows + scale_slot]
    return (n * (1.0 + scale) + shift).to(x.dtype)


def gated_residual(h, u, table, idx, vectors_per_row, gate_slot):
    gate = table[idx.long() * vectors_per_row + gate_slot]
    return (h.float() + gate * u.float()).to(h.dtype)


def layer_norm(x, w, b, eps):
    return F.layer_norm(x.float(), (x.shape[-1],), None if w is None else w.float(),
                        None if b is None else b.float(), eps).to(x.dtype)


def rope_inv_freq(rot: int, theta: float, device=None):
    return 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32, device=device) / rot))


def _rotate(x, cos, sin, interleaved: bool):
    # x: [..., rot]; cos/sin: [..., rot/2]
    if interleaved:
        x1, x2 = x[..., 0::2], x[..., 1::2]
        o1 = x1 * cos - x2 * sin
        o2 = x2 * cos + x1 * sin
        return torch.stack([o1, o2], dim=-1).flatten(-2)
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def qk_norm_rope(q, k, qw, kw, positions, inv_freq, rot, interleaved, eps):
    """q [T,Hq,D], k [T,Hk,D] -> normalised + rotated, rounded once."""
    def one(x, w):
        xf = x.float()
        if w is not None:
            xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
        ang = positions.float()[:, None] * inv_freq.float()[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        out = torch.cat([_rotate(xf[..., :rot], cos, sin, interleaved), xf[..., rot:]], dim=-1)
        return out.to(x.dtype)
    return one(q, qw), one(k, kw)


def qk_norm_rope3(q, k, qw, kw, coords, inv_freq, freqs_per_axis, eps):
    """Three-axis rotary of the video transformer.  coords [3,T]; axis a owns
    channels [a*2F, (a+1)*2F) as half-split pairs."""
    Fq = freqs_per_axis

    def one(x, w):
        xf = x.float()
        if w is not None:
            xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
        parts = []
        for a in range(3):
            ang = coords[a].float()[:, None] * inv_freq.float()[None, :]
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
            parts.append(_rotate(xf[..., a * 2 * Fq:(a + 1) * 2 * Fq], cos, sin, False))
        parts.append(xf[..., 6 * Fq:])
        return torch.cat(parts, dim=-1).to(x.dtype)
    return one(q, qw), one(k, kw)


def kv_write(kcache, vcache, k, v, slots):
    """Scatter k/v rows [T,Hkv,D] into caches viewed as [slots_total,Hkv,D]."""
    kc = kcache.view(-1, *kcache.shape[-2:])
    vc = vcache.view(-1, *vcache.shape[-2:])
    ok = slots >= 0
    kc[slots[ok].long()] = k[ok]
    vc[slots[ok].long()] = v[ok]


E4M3_MAX = 448.0


def _to_e4m3(x):
    return x.clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)


def kv_write_scaled(kcache, vcache, k_scale, v_scale, k, v, slots):
    """The scaled FP8 page write, one page at a time: caches uint8 [pages, page, Hkv, D] holding
    E4M3 bytes, scales FP32 [pages].  A page's scale grows to max|values| / 448 of what a call
    brings; rows the page already holds (offsets below the call's first) are re-encoded when
    it grows; a row at offset 0 starts the page afresh."""
    page = kcache.shape[1]
    for cache, scale, src in ((kcache, k_scale, k), (vcache, v_scale, v)):
        c8 = cache.view(torch.float8_e4m3fn)
        done = set()
        sl = slots.tolist()
        for t, s in enumerate(sl):
            if s < 0 or s // page in done:
                continue
            p = s // page
            done.add(p)
            rows = [i for i in range(t, len(sl)) if sl[i] >= 0 and sl[i] // page == p]
            off0 = s - p * page
            amax = float(src[rows].float().abs().max())
            old = float(scale[p]) if off0 > 0 else 0.0
            now = max(old, max(amax, 1e-12) / E4M3_MAX)
            if now > old and off0 > 0:
                c8[p, :off0] = _to_e4m3(c8[p, :off0].float() * (old / now))
            for i in rows:
                c8[p, sl[i] - p * page] = _to_e4m3(src[i].float() * (1.0 / now))
            scale[p] = now


def kv_dequant(cache, scale):
    """E4M3 pages [pages, page, Hkv, D] (uint8) and their scales -> FP32 values."""
    return cache.view(torch.float8_e4m3fn).float() * scale.float()[:, None, None, None]


def paged_decode_attention(q, kcache, vcache, page_table, seq_lens, scale, window=0,
                           k_scale=None, v_scale=None):
    """q [B,Hq,D]; caches [pages,page,Hkv,D] -> [B,Hq,D].  With scales the caches are E4M3."""
    if k_scale is not None:
        kcache, vcache = kv_dequant(kcache, k_scale), kv_dequant(vcache, v_scale)
    B, Hq, D = q.shape
    pages, page, Hkv, _ = kcache.shape
    G = Hq // Hkv
    out = torch.zeros_like(q)
    for b in range(B):
        n = int(seq_lens[b])
        if n <= 0:
            continue
        start = max(0, n - window) if window > 0 else 0
        npages = (n + page - 1) // page
        idx = page_table[b, :npages].long()
        kk = kcache[idx].reshape(-1, Hkv, D)[start:n].float()
        vv = vcache[idx].reshape(-1, Hkv, D)[start:n].float()
        qq = q[b].float().view(Hkv, G, D)
        s = torch.einsum("hgd,nhd->hgn", qq, kk) * scale
        p = s.softmax(-1)
        o = torch.einsum("hgn,nhd->hgd", p, vv)
        out[b] = o.reshape(Hq, D).to(q.dtype)
    return out


def varlen_attention(q, k, v, cu_q, cu_k, scale, causal):
    """q [Tq,Hq,D], k/v [Tk,Hkv,D]; cu_* int [n+1].  Causal masks are aligned to
    the bottom right (query i of a sequence sees keys <= i + (len_k - len_q))."""
    Tq, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    out = torch.zeros_like(q)
    n = cu_q.numel() - 1
    for i in range(n):
        q0, q1 = int(cu_q[i]), int(cu_q[i + 1])
        k0, k1 = int(cu_k[i]), int(cu_k[i + 1])
        if q1 <= q0:
            continue
        qq = q[q0:q1].float().view(q1 - q0, Hkv, G, D)
        kk = k[k0:k1].float()
        vv = v[k0:k1].float()
        s = torch.einsum("qhgd,khd->hgqk", qq, kk) * scale
        if causal:
            lq, lk = q1 - q0, k1 - k0
            qi = torch.arange(lq, device=q.device)[:, None] + (lk - lq)
            ki = torch.arange(lk, device=q.device)[None, :]
            s = s.masked_fill(ki > qi, float("-inf"))
        p = s.softmax(-1)
        p = torch.nan_to_num(p)
        o = torch.einsum("hgqk,khd->qhgd", p, vv)
        out[q0:q1] = o.reshape(q1 - q0, Hq, D).to(q.dtype)
    return out


def linear(x, w, bias=None, out_dtype=None):
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype or x.dtype)


def gated_act(first, second, act: str, stepwise: bool):
    """first * act(second); stepwise rounds the activation and the operands to
    bf16 before the product (crates/nn/src/modules/mlp.rs:1-7, reference path)."""
    if act == "gelu_tanh":
        return first * F.gelu(second, approximate="tanh")
    if stepwise:
        s = F.silu(second.to(torch.bfloat16).float()).to(torch.bfloat16).float()
        return first.to(torch.bfloat16).float() * s
    return first * F.silu(second)


def linear_gated(x, w, act="silu", stepwise=False, out_dtype=None):
    """w stacks [first; second] rows: out = (x w_first^T) * act(x w_second^T)."""
    y = x.float() @ w.float().t()
    half = w.shape[0] // 2
    return gated_act(y[:, :half], y[:, half:], act, stepwise).to(out_dtype or x.dtype)


def topk_softmax(logits, top_k, renorm):
    p = logits.float().softmax(-1)
    # repeated argmax with ties to the lower id == stable descending sort
    order = torch.sort(p, dim=-1, descending=True, stable=True)
    w, ids = order.values[:, :top_k], order.indices[:, :top_k]
    if renorm:
        w = w / w.sum(-1, keepdim=True).clamp_min(torch.finfo(torch.float32).eps)
    return ids.to(torch.int32), w


def moe_experts(x, ids, weights, w13, w2, e_lo=0, act="silu", stepwise=False):
    """Dense loop over experts.  w13 [E,2I,H] (first rows, then gate rows),
    w2 [E,H,I]; ids [T,k] global expert ids (-1 drops); returns [T,H] in x.dtype."""
    T, H = x.shape
    E = w13.shape[0]
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for e in range(E):
        sel = ids == (e + e_lo)
        if not sel.any():
            continue
        tok, slot = sel.nonzero(as_tuple=True)
        h = linear_gated(x[tok], w13[e], act, stepwise, out_dtype=x.dtype)
        y = linear(h, w2[e], out_dtype=x.dtype)
        out.index_add_(0, tok, y.float() * weights[tok, slot].float()[:, None])
    return out.to(x.dtype)


def argmax(logits):
    return logits.float().argmax(-1).to(torch.int32)


def logits_shape(logits, ban_mask=None, bias=None, out_counts=None, prompt_mask=None,
                 rep=None, freq=None, pres=None, temp=None):
    """vLLM order: bans -> bias -> penalties -> temperature (0 divides by 1)."""
    x = logits.float().clone()
    B, V = x.shape
    if ban_mask is not None:
        x = x.masked_fill(ban_mask.bool(), float("-inf"))
    if bias is not None:
        for b, entries in enumerate(bias):
            for tok, val in entries:
                x[b, tok] += val
    if out_counts is not None or prompt_mask is not None:
        oc = out_counts.float() if out_counts is not None else torch.zeros_like(x)
        seen = oc > 0
        if prompt_mask is not None:
            seen = seen | prompt_mask.bool()
        if rep is not None:
            r = rep.float()[:, None]
            x = torch.where(seen, torch.where(x > 0, x / r, x * r), x)
        if freq is not None:
            x = x - freq.float()[:, None] * oc
        if pres is not None:
            x = x - pres.float()[:, None] * (oc > 0).float()
    if temp is not None:
        t = temp.float().clone()
        t[t == 0] = 1.0
        x = x / t[:, None]
    return x


def philox_uniform(seed: int, position: int, stage: int = 0, draw: int = 0) -> float:
    from ..utils.philox import philox_uniform as f
    return f(seed, position, stage, draw)


def sample_from_logits(logits, top_k, top_p, min_p, seeds, positions):
    """Same candidate set and inverse-CDF rule as the kernel, with float64 sums
    (the kernel uses 2^-40 integer masses, so results can differ only when the
    uniform lands within ~1e-12 of a CDF step)."""
    x = logits.double()
    B, V = x.shape
    out = torch.zeros(B, dtype=torch.int32)
    for b in range(B):
        row = x[b]
        mx = row.max()
        keep = torch.isfinite(row)
        k = int(top_k[b]) if top_k is not None else 0
        if 0 < k < V:
            kth = torch.topk(row, k).values[-1]
            keep &= row >= kth
        if min_p is not None and float(min_p[b]) > 0:
            keep &= row >= mx + math.log(float(min_p[b]))
        w = torch.where(keep, torch.exp(row - mx), torch.zeros_like(row))
        tp = float(top_p[b]) if top_p is not None else 1.0
        if tp < 1.0:
            total = w.sum()
            srt = torch.sort(w, descending=True)
            csum = srt.values.cumsum(0)
            # smallest prefix (by descending weight) whose mass reaches tp * total
            n = int((csum < tp * total).sum().item()) + 1
            thr = srt.values[min(n, V) - 1]
            keep &= w >= thr
            w = torch.where(keep, w, torch.zeros_like(w))
        u = philox_uniform(int(seeds[b]), int(positions[b]))
        c = w.cumsum(0)
        target = u * c[-1]
        idx = int((c <= target).sum().item())
        idx = min(idx, V - 1)
        out[b] = idx
    return out


def logprob_stats(logits, chosen):
    lf = logits.float()
    lse = torch.logsumexp(lf, -1)
    cv = lf.gather(1, chosen.long()[:, None])[:, 0]
    rank = (lf > cv[:, None]).sum(-1).to(torch.int32) + 1
    return lse, cv - lse, rank


def embedding(ids, table, vocab_lo=0, vocab_hi=None):
    vocab_hi = table.shape[0] + vocab_lo if vocab_hi is None else vocab_hi
    ok = (ids >= vocab_lo) & (ids < vocab_hi)
    local = (ids - vocab_lo).clamp(0, table.shape[0] - 1).long()
    out = table[local]
    return out * ok[:, None].to(out.dtype)


def persist_segments(seq_lens, Hkv: int, n_cta: int, tile: int = 128):
    """The work partition of the persistent decode-attention kernel
    (``csrc/attn_decode_persist.cu``), restated on the host: the tiles of all (sequence, kv
    head) pairs form one list ordered by (sequence, kv head, tile); range c of ``n`` =
    min(n_cta, tiles) takes tiles [c T // n, (c + 1) T // n).  Returns, per range, its
    segments ``(b, hk, first_tile, count, whole, slot)``: ``whole`` segments cover their pair
    and are written directly, the others leave a partial result in ``slot`` (0: the range's
    first segment, 1: a later one, which is then its last) and arrive at the pair's counter."""
    tiles = [(int(l) + tile - 1) // tile for l in seq_lens]
    pre = [0]
    for t in tiles:
        pre.append(pre[-1] + t)
    total = Hkv * pre[-1]
    if total == 0:
        return []
    n = min(n_cta, total)
    pairs = [(b, hk) for b in range(len(tiles)) if tiles[b] for hk in range(Hkv)]
    where = []                                   # tile index -> (pair index, tile of the pair)
    for i, (b, _) in enumerate(pairs):
        where.extend((i, t) for t in range(tiles[b]))
    out = []
    for c in range(n):
        g, g1 = (c * total) // n, ((c + 1) * total) // n
        segs = []
        while g < g1:
            i, t0 = where[g]
            b, hk = pairs[i]
            count = min(tiles[b] - t0, g1 - g)
            whole = t0 == 0 and count == tiles[b]
            segs.append((b, hk, t0, count, whole, 0 if not segs else 1))
            g += count
        out.append(segs)
    return out


def persist_merge_slots(seq_lens, Hkv: int, n_cta: int, b: int, hk: int, tile: int = 128):
    """(range, slot) of every partial result of pair (b, hk), as the merging CTA derives them
    from the partition alone: the ranges from the one that holds the pair's first tile to the
    one that holds its last; slot 0 where the range starts inside the pair, else 1."""
    tiles = [(int(l) + tile - 1) // tile for l in seq_lens]
    pre = [0]
    for t in tiles:
        pre.append(pre[-1] + t)
    total = Hkv * pre[-1]
    n = min(n_cta, total)
    start = lambda c: (c * total) // n

    def cta_of(g):
        c = (g * n) // total
        while c + 1 < n and start(c + 1) <= g:
            c += 1
        while c > 0 and start(c) > g:
            c -= 1
        return c
    begin = Hkv * pre[b] + hk * tiles[b]
    last = begin + tiles[b] - 1
    return [(c, 0 if start(c) >= begin else 1) for c in range(cta_of(begin), cta_of(last) + 1)]
