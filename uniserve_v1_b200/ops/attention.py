"""Prefill / dense attention entry points over the varlen flash kernel.

``prefill_attention`` serves the token path: rows of the fused QKV projection
(already normalised and rotated, K/V already written to the paged cache) attend
causally to their sequence.  A sequence with keys already in the cache (chunked
prefill, prefix-cache hit) reads those pages back into a contiguous buffer in
front of the new keys.

``dense_attention`` serves the video transformer: bidirectional varlen attention
with separate query and key offset tables (queries = every row, keys = used rows;
reference: crates/models/src/minimax_h3/transformer.py:247-256 equivalent
behaviour, reference project path).
"""
from __future__ import annotations

import torch

from . import native as N
from . import reference as R

BF16 = torch.bfloat16


def have_flash() -> bool:
    try:
        return hasattr(N.kernels(), "us_flash_attn_varlen")
    except N.NativeMissing:
        return False


def varlen_attention(q, k, v, cu_q, cu_k, max_q, max_k, scale, causal, out=None):
    """q [Tq, Hq, D], k/v [Tk, Hkv, D] (row-strided views allowed, last dim and
    head dim contiguous); cu_* int32 [n+1].  Returns [Tq, Hq, D] bf16."""
    if not q.is_cuda:
        return R.varlen_attention(q, k, v, cu_q, cu_k, scale, causal)
    from .flash import flash_attn_varlen
    return flash_attn_varlen(q, k, v, cu_q, cu_k, max_q, max_k, scale, causal, out=out)


def prefill_attention(qkv, Hq, Hkv, D, meta, kcache, vcache, scale):
    T = qkv.shape[0]
    real = getattr(meta, "rows_real", None)
    if real is not None and real < T:
        # rows padded up to an agreed capacity: they attend to nothing and stay zero
        out = torch.zeros(T, Hq, D, dtype=qkv.dtype, device=qkv.device)
        if real > 0:
            import copy
            m2 = copy.copy(meta)
            m2.rows_real = None
            out[:real] = prefill_attention(qkv[:real], Hq, Hkv, D, m2, kcache, vcache, scale)
        return out
    v3 = qkv.view(T, Hq + 2 * Hkv, D)
    q, k, v = v3[:, :Hq], v3[:, Hq:Hq + Hkv], v3[:, Hq + Hkv:]
    ctx_lens = meta.context_lens
    k_scale = getattr(kcache, "page_scale", None)
    v_scale = getattr(vcache, "page_scale", None)
    if ctx_lens is not None and any(c > 0 for c in ctx_lens):
        tables = getattr(meta, "ctx_tables", None)
        if qkv.is_cuda and tables is not None:
            # Keys already cached sit in front of this call's keys of each sequence: one
            # gather launch through the page table (bf16 or E4M3 pages) and one row scatter
            # of the new keys; nothing returns to the host.
            from . import functional as F
            ctx_cu, new_dst, ctx_total = tables
            total = ctx_total + new_dst.shape[0]
            kb = torch.empty(total, Hkv, D, dtype=qkv.dtype, device=qkv.device)
            vb = torch.empty(total, Hkv, D, dtype=qkv.dtype, device=qkv.device)
            F.kv_gather(kcache, vcache, meta.page_table, ctx_cu, ctx_total, k_scale, v_scale,
                        out=(kb, vb), out_cu=meta.cu_k)
            kb.index_copy_(0, new_dst, k[:new_dst.shape[0]])
            vb.index_copy_(0, new_dst, v[:new_dst.shape[0]])
            k, v = kb, vb
        else:
            page = kcache.shape[1]
            kc, vc = kcache, vcache
            if k_scale is not None:
                kc, vc = R.kv_dequant(kcache, k_scale).to(qkv.dtype), \
                    R.kv_dequant(vcache, v_scale).to(qkv.dtype)
            ks, vs = [], []
            cu_q = meta.cu_q.tolist()
            for i, c in enumerate(ctx_lens):
                if c > 0:
                    npg = (c + page - 1) // page
                    idx = meta.page_table[i, :npg].long()
                    ks.append(kc[idx].reshape(-1, Hkv, D)[:c])
                    vs.append(vc[idx].reshape(-1, Hkv, D)[:c])
                ks.append(k[cu_q[i]:cu_q[i + 1]])
                vs.append(v[cu_q[i]:cu_q[i + 1]])
            k, v = torch.cat(ks, 0), torch.cat(vs, 0)
    return varlen_attention(q, k, v, meta.cu_q, meta.cu_k, meta.max_q, meta.max_k, scale, True)


def context_tables(ctx: list, cu_q: list, cu_k: list, device):
    """Device tables for a prefill whose sequences have cached context (all built from the
    scheduler's host-side plan): cumulative context lengths [B + 1] (int32), the row of every
    new key in the combined per-sequence [cached; new] buffer [T] (int64), and the total
    number of cached rows."""
    ctx_cu, new_dst = [0], []
    for i, c in enumerate(ctx):
        ctx_cu.append(ctx_cu[-1] + c)
        n = cu_q[i + 1] - cu_q[i]
        new_dst.extend(range(cu_k[i] + c, cu_k[i] + c + n))
    pin = torch.device(device).type == "cuda"
    a = torch.tensor(ctx_cu, dtype=torch.int32, pin_memory=pin).to(device, non_blocking=True)
    b = torch.tensor(new_dst, dtype=torch.int64, pin_memory=pin).to(device, non_blocking=True)
    return a, b, ctx_cu[-1]


def cached_causal_attention(q, k_all, v_all, scale):
    """One sequence whose T newest rows ``q`` [T, Hq, D] attend causally to all of its keys
    ``k_all`` / ``v_all`` [N, Hkv, D] (the T newest included, aligned to the end).  bf16 on a
    GPU with a head width the flash kernel serves: the varlen flash kernel; otherwise the
    FP32 restatement.  Returns [T, Hq, D] FP32 (restatement) or bf16 (kernel)."""
    T, Hq, D = q.shape
    N_, Hkv = k_all.shape[0], k_all.shape[1]
    if q.is_cuda and q.dtype == BF16 and D % 8 == 0 and D <= 128:
        dev = q.device
        cu_q = torch.tensor([0, T], dtype=torch.int32, device=dev)
        cu_k = torch.tensor([0, N_], dtype=torch.int32, device=dev)
        q, k_all, v_all = (t if (t.stride(2) == 1 and t.stride(1) == D) else t.contiguous()
                           for t in (q, k_all, v_all))
        return varlen_attention(q, k_all.to(BF16), v_all.to(BF16), cu_q, cu_k, T, N_, scale, True)
    rep = Hq // Hkv
    K = k_all.float().repeat_interleave(rep, 1)
    V = v_all.float().repeat_interleave(rep, 1)
    s_ = torch.einsum("thd,nhd->htn", q.float(), K) * scale
    seq = torch.arange(N_ - T, N_, device=q.device)
    s_ = s_.masked_fill((torch.arange(N_, device=q.device)[None, :] > seq[:, None])[None],
                        float("-inf"))
    return torch.einsum("htn,nhd->thd", s_.softmax(-1), V)
