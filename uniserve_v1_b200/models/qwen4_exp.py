"""Building blocks of the Qwen4-exp ("Qwen3.8 Flash Next") family: the gated hyper-connection
around every block, the hashed n-gram embedding and the layer that gates it into the residual
streams.  The family's decoder (gated delta net or indexed attention, then experts with a gated
shared expert, each between two hyper-connections) is not assembled here, nor is the indexed
(sparse-token) attention with its group index.

**Hyper-connection.**  The residual is C streams of width H, ``S`` [tokens, C * H]::

    norm      Sn_c = S_c * rsqrt(mean(S_c^2) + eps) * (1 + w_c)
    mix       d = Sn @ down^T  [tokens, rank]     r = Sn @ inject^T  [tokens, C]
              g = silu(d / C) @ up^T  [tokens, C * H]
              h = mean_c( sigmoid(g_c) * Sn_c )                      the block's input
    combine   S'_c = S_c + y * 2 * sigmoid(r_c / C)                  y the block's output

A block's combine is deferred into the next read (``read(S, pending=(y, r))``).

**N-gram embedding.**  Token t0 with the n - 1 ids before it (an end-of-text id ends the
n-gram: everything before it reads as end-of-text)::

    mix_1 = t0 * m_0;  mix_k = mix_{k-1} xor (p_{k-1} * m_{k-1})        64-bit, wrapping
    id_h  = (mix_k mod P_h) + O_h       for the heads h of n-gram length k, 2 <= k <= n
    e     = [table[id_0] | table[id_1] | ...] * scale                   E4M3 table, one scale

**PLE layer.**  ``key = e @ key_proj^T`` [tokens, C, H], ``value = e @ value_proj^T``; with
``gemma(x; w) = x * rsqrt(mean(x^2) + eps) * (1 + w)``::

    d_c  = sum_j gemma(key_c; nk_c)[j] * gemma(S_c; nq_c)[j] / sqrt(H)
    g_c  = sigmoid(sign(d_c) * sqrt(max(|d_c|, 1e-6)))
    gv_c = g_c * value;   out = gv + silu(conv(gemma(gv; nc)))       dilated, causal, stateful

Reference behaviour: crates/models/src/qwen4_exp/hyper_connection.rs:1-31,
crates/models/src/qwen4_exp/ngram.rs:1-47 (reference project paths).
"""
from __future__ import annotations

import math
from typing import Optional

import torch


def gemma_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w.float())).to(x.dtype)


class HyperConnection:
    def __init__(self, hidden: int, streams: int, rank: int, eps: float = 1e-6,
                 injects: bool = True, dtype=torch.float32, device="cpu"):
        self.H, self.C, self.rank, self.eps, self.injects = hidden, streams, rank, eps, injects
        W = hidden * streams
        self.hc_norm = torch.zeros(W, dtype=dtype, device=device)
        self.down = torch.zeros(rank + (streams if injects else 0), W, dtype=dtype, device=device)
        self.up = torch.zeros(W, rank, dtype=dtype, device=device)

    def init_random(self, seed: int = 0, std: float = 0.05) -> "HyperConnection":
        g = torch.Generator().manual_seed(seed)
        for name in ("hc_norm", "down", "up"):
            t = getattr(self, name)
            t.copy_((torch.randn(t.shape, generator=g) * std).to(t.dtype))
        return self

    @staticmethod
    def fold(S: torch.Tensor, y: torch.Tensor, logits: Optional[torch.Tensor], streams: int):
        """The combine: every stream takes the block's output under its own gain."""
        T, W = S.shape
        upd = y.float()[:, None, :]
        if logits is not None:
            upd = upd * (2.0 * torch.sigmoid(logits.float() / streams))[:, :, None]
        return (S.float().view(T, streams, W // streams) + upd).to(S.dtype).view(T, W)

    def read(self, S: torch.Tensor, pending=None):
        """Folds the previous block's (output, logits) into the streams, then normalises and
        mixes them.  Returns (streams, the block's input [tokens, H], its combine logits)."""
        if pending is not None:
            S = self.fold(S, pending[0], pending[1], self.C)
        T = S.shape[0]
        Sn = gemma_norm(S.view(T * self.C, self.H),
                        self.hc_norm.view(self.C, self.H).repeat(T, 1), self.eps).view(T, -1)
        both = (Sn.float() @ self.down.float().t()).to(S.dtype)
        low, logits = (both[:, :self.rank], both[:, self.rank:].contiguous()) if self.injects \
            else (both, None)
        low = torch.nn.functional.silu(low.float() / self.C).to(S.dtype)
        gate = (low.float() @ self.up.float().t()).to(S.dtype)
        h = (torch.sigmoid(gate.float()).view(T, self.C, self.H) *
             Sn.float().view(T, self.C, self.H)).mean(1).to(S.dtype)
        return S, h, logits


def ngram_ids(tokens: torch.Tensor, eos: int, multipliers: torch.Tensor, partitions: torch.Tensor,
              offsets: torch.Tensor, heads_per_ngram: int) -> torch.Tensor:
    """tokens [T] int64 (one request, oldest first) -> table rows [T, heads] int64.
    ``multipliers`` [n] (the token's own first), ``partitions`` / ``offsets`` [heads]; heads are
    grouped by n-gram length 2 .. n, ``heads_per_ngram`` each."""
    T, n = tokens.shape[0], multipliers.shape[0]
    toks = tokens.to(torch.int64)
    mix = toks * multipliers[0]                                     # wraps like 64-bit integers
    stopped = torch.zeros(T, dtype=torch.bool, device=toks.device)
    out = []
    for k in range(1, n):
        prev = torch.full((T,), eos, dtype=torch.int64, device=toks.device)
        prev[k:] = toks[:T - k]                                     # before the request: end of text
        stopped = stopped | (prev == eos)
        prev = torch.where(stopped, torch.full_like(prev, eos), prev)
        mix = mix ^ (prev * multipliers[k])
        for h in range((k - 1) * heads_per_ngram, k * heads_per_ngram):
            out.append(torch.remainder(mix, partitions[h]) + offsets[h])
    return torch.stack(out, 1)


class NgramEmbedding:
    def __init__(self, table_e4m3: torch.Tensor, scale: float, eos: int, multipliers, partitions,
                 offsets, heads_per_ngram: int):
        self.table, self.scale, self.eos = table_e4m3, float(scale), eos
        self.m, self.P, self.O, self.hpn = multipliers, partitions, offsets, heads_per_ngram

    def forward(self, tokens: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
        ids = ngram_ids(tokens, self.eos, self.m, self.P, self.O, self.hpn)
        rows = self.table.view(torch.float8_e4m3fn)[ids]            # [T, heads, dim]
        scale = torch.tensor(self.scale, dtype=dtype)
        return (rows.to(dtype) * scale).reshape(tokens.shape[0], -1)


class PleLayer:
    def __init__(self, hidden: int, streams: int, embed: int, kernel: int = 4, dilation: int = 1,
                 eps: float = 1e-6, dtype=torch.float32):
        self.H, self.C, self.E, self.K, self.dil, self.eps = hidden, streams, embed, kernel, \
            dilation, eps
        z = lambda *s: torch.zeros(*s, dtype=dtype)
        self.key_proj, self.value_proj = z(streams * hidden, embed), z(hidden, embed)
        self.norm_key, self.norm_query, self.norm_conv = z(streams, hidden), z(streams, hidden), \
            z(streams, hidden)
        self.conv = z(streams * hidden, kernel)

    def init_random(self, seed: int = 0, std: float = 0.05) -> "PleLayer":
        g = torch.Generator().manual_seed(seed)
        for name in ("key_proj", "value_proj", "norm_key", "norm_query", "norm_conv", "conv"):
            t = getattr(self, name)
            t.copy_((torch.randn(t.shape, generator=g) * std).to(t.dtype))
        return self

    def forward(self, e: torch.Tensor, S: torch.Tensor, state: Optional[torch.Tensor] = None):
        """e [T, E], S [T, C * H] -> (what is added to the streams [T, C * H], new conv state:
        the last (K - 1) * dilation rows of the normalised gated values)."""
        T, C, H = e.shape[0], self.C, self.H
        key = (e.float() @ self.key_proj.float().t()).to(S.dtype).view(T, C, H)
        value = (e.float() @ self.value_proj.float().t()).to(S.dtype)
        kn = gemma_norm(key, self.norm_key, self.eps)
        qn = gemma_norm(S.view(T, C, H), self.norm_query, self.eps)
        d = ((kn.float() * qn.float()).to(S.dtype).float().sum(-1) / math.sqrt(H)).to(S.dtype).float()
        g = torch.sigmoid(torch.sign(d) * torch.sqrt(d.abs().clamp_min(1e-6))).to(S.dtype)
        gv = (g.float()[:, :, None] * value.float()[:, None, :]).to(S.dtype)         # [T, C, H]
        gvn = gemma_norm(gv, self.norm_conv, self.eps).view(T, C * H)
        span = (self.K - 1) * self.dil
        if state is None:
            state = torch.zeros(span, C * H, dtype=S.dtype)
        full = torch.cat([state, gvn], 0).float()
        conv = torch.zeros(T, C * H)
        for k in range(self.K):
            back = (self.K - 1 - k) * self.dil
            conv += self.conv.float()[:, k][None, :] * full[span - back:span - back + T]
        out = gv.view(T, C * H).float() + torch.nn.functional.silu(conv.to(S.dtype).float())
        return out.to(S.dtype), full[-span:].to(S.dtype) if span else state
