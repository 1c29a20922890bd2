"""Building blocks of the Qwen4-exp ("Qwen3.8 Flash Next") family: the gated hyper-connection
around every block, the hashed n-gram embedding and the layer that gates it into the residual
streams, the indexed (sparse-token) attention with its group index, and the decoder that puts
them together (``Qwen4ExpModel``: gated delta net or indexed attention, then experts with a gated
shared expert, each behind a hyper-connection) as FP32 formulas for one request.

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


def partial_rope(x: torch.Tensor, pos: torch.Tensor, rotary_dim: int, theta: float) -> torch.Tensor:
    """Half-rotation rotary embedding over the leading ``rotary_dim`` channels of x [T, n, d]."""
    half = rotary_dim // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float32) / half)
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    a, b, rest = xf[..., :half], xf[..., half:rotary_dim], xf[..., rotary_dim:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, rest], -1).to(x.dtype)


class IndexedAttention:
    """Gated attention over the tokens an indexer selects, one request at a time.

    Tokens form groups of ``ratio``; a complete group has one index key, the normalised and
    rotated mean of its tokens' raw index keys at the position of its first token.  A row at
    position t sees the ``(t + 1) // ratio`` complete groups, scores them
    ``sum_h relu(q_idx[h] . key)``, keeps the tokens of the best ``budget // ratio`` in rank order
    and then the ``(t + 1) % ratio`` tokens of its own unfinished group: ``budget + ratio - 1``
    entries, -1 where it has fewer.  Softmax attention runs over those tokens only; the output is
    ``o_proj(o * sigmoid(gate))`` with the gate taken from the query projection.

    ``cache`` holds the request's rotated keys, values and raw index keys; index keys of complete
    groups are pooled from the raw ones at every call.  Reference behaviour:
    crates/models/src/qwen4_exp/attention.rs:1-40, 408-526 (reference project paths).
    """

    def __init__(self, hidden, heads, kv_heads, head_dim, index_heads, index_dim, ratio, budget,
                 rotary_dim=None, theta=10000.0, eps=1e-6, dtype=torch.float32):
        assert budget % ratio == 0 and heads % kv_heads == 0
        self.hidden, self.heads, self.kv, self.hd = hidden, heads, kv_heads, head_dim
        self.ih, self.idim, self.ratio, self.budget = index_heads, index_dim, ratio, budget
        self.rot = rotary_dim or head_dim
        self.irot = min(self.rot, index_dim)
        self.theta, self.eps = theta, eps
        z = lambda *s: torch.zeros(*s, dtype=dtype)
        self.q_proj = z(heads * 2 * head_dim, hidden)             # per head: query rows, gate rows
        self.k_proj, self.v_proj = z(kv_heads * head_dim, hidden), z(kv_heads * head_dim, hidden)
        self.o_proj = z(hidden, heads * head_dim)
        self.q_norm, self.k_norm = z(head_dim), z(head_dim)
        self.index_qk_proj = z((index_heads + 1) * index_dim, hidden)
        self.q_layernorm, self.k_layernorm = z(index_dim), z(index_dim)

    def init_random(self, seed: int = 0, std: float = 0.2) -> "IndexedAttention":
        g = torch.Generator().manual_seed(seed)
        for name in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm", "index_qk_proj",
                     "q_layernorm", "k_layernorm"):
            t = getattr(self, name)
            t.copy_((torch.randn(t.shape, generator=g) * std).to(t.dtype))
        return self

    def index_keys(self, raw: torch.Tensor) -> torch.Tensor:
        """raw [n, idim] from position 0 -> [n // ratio, idim], one key per complete group."""
        G = raw.shape[0] // self.ratio
        pooled = raw[:G * self.ratio].float().view(G, self.ratio, self.idim).mean(1).to(raw.dtype)
        first = torch.arange(G) * self.ratio
        return partial_rope(gemma_norm(pooled, self.k_layernorm, self.eps)[:, None, :], first,
                            self.irot, self.theta)[:, 0]

    def select(self, q_idx: torch.Tensor, keys: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """q_idx [T, ih, idim], keys [G, idim], pos [T] -> selection [T, budget + ratio - 1]."""
        T, r, top = q_idx.shape[0], self.ratio, self.budget // self.ratio
        visible, partial = (pos + 1) // r, (pos + 1) % r
        sel = torch.full((T, self.budget + r - 1), -1, dtype=torch.int64)
        G = keys.shape[0]
        if G:
            s = torch.relu(torch.einsum("thd,gd->thg", q_idx.float(), keys.float())).sum(1)
            s = s.masked_fill(torch.arange(G)[None, :] >= visible[:, None], float("-inf"))
            kept = min(top, G)
            best = s.topk(kept, dim=1).indices                                   # rank order
            named = torch.arange(kept)[None, :] < visible.clamp_max(kept)[:, None]
            toks = best[:, :, None] * r + torch.arange(r)[None, None, :]
            toks = torch.where(named[:, :, None], toks, torch.full_like(toks, -1))
            sel[:, :kept * r] = toks.reshape(T, kept * r)
        tail = visible[:, None] * r + torch.arange(r - 1)[None, :]
        sel[:, self.budget:] = torch.where(torch.arange(r - 1)[None, :] < partial[:, None], tail,
                                           torch.full_like(tail, -1))
        return sel

    def forward(self, x: torch.Tensor, cache: Optional[dict] = None):
        """x [T, hidden], the request's next T tokens -> (output [T, hidden], cache, selection)."""
        T, H, hd = x.shape[0], self.heads, self.hd
        cache = cache if cache is not None else {"k": x.new_zeros(0, self.kv, hd),
                                                 "v": x.new_zeros(0, self.kv, hd),
                                                 "raw": x.new_zeros(0, self.idim)}
        pos = cache["k"].shape[0] + torch.arange(T)
        lin = lambda w: (x.float() @ w.float().t()).to(x.dtype)
        qg = lin(self.q_proj).view(T, H, 2, hd)
        q, gate = qg[:, :, 0], qg[:, :, 1]
        q = partial_rope(gemma_norm(q, self.q_norm, self.eps), pos, self.rot, self.theta)
        k = partial_rope(gemma_norm(lin(self.k_proj).view(T, self.kv, hd), self.k_norm, self.eps),
                         pos, self.rot, self.theta)
        iq = lin(self.index_qk_proj).view(T, self.ih + 1, self.idim)
        q_idx = partial_rope(gemma_norm(iq[:, :self.ih], self.q_layernorm, self.eps), pos,
                             self.irot, self.theta)
        cache = {"k": torch.cat([cache["k"], k]),
                 "v": torch.cat([cache["v"], lin(self.v_proj).view(T, self.kv, hd)]),
                 "raw": torch.cat([cache["raw"], iq[:, self.ih]])}
        sel = self.select(q_idx, self.index_keys(cache["raw"]), pos)
        valid = sel >= 0
        at = sel.clamp_min(0)
        rep = H // self.kv
        ks = cache["k"][at].repeat_interleave(rep, 2).float()                   # [T, S, H, hd]
        vs = cache["v"][at].repeat_interleave(rep, 2).float()
        sc = torch.einsum("thd,tshd->ths", q.float(), ks) * hd ** -0.5
        sc = sc.masked_fill(~valid[:, None, :], float("-inf"))
        o = torch.einsum("ths,tshd->thd", torch.softmax(sc, -1), vs).to(x.dtype)
        o = (o.float() * torch.sigmoid(gate.float())).to(x.dtype).reshape(T, H * hd)
        return (o.float() @ self.o_proj.float().t()).to(x.dtype), cache, sel


class Qwen4ExpModel:
    """The decoder over hyper-connected streams, one request at a time (FP32 formulas)::

        x = embed(ids);  S = [x | x | ...]  (C copies);  pending = none
        per layer:  PLE layers first fold ``pending`` and add ple(S, ngram(ids))
                    S, h, r = attn_hc.read(S, pending);  y = linear_attn(h) or self_attn(h)
                    S, h, r = mlp_hc.read(S, (y, r));     y = experts(h) + gated shared expert
                    pending = (y, r)
        read-out:   S = fold(S, pending);  logits = lm_head(mixer.read(S))      no final norm

    A layer has no norm of its own: each read normalises the streams.  The gated delta network
    and the experts are the hybrid family's (``Qwen35MoeModel``), built at the same widths; full
    attention layers become indexed attention.  Reference behaviour:
    crates/models/src/qwen4_exp/decoder.rs:1-17, crates/models/src/qwen4_exp/causal_lm.rs:1-30
    (reference project paths).
    """

    def __init__(self, cfg, streams: int = 2, rank: int = 8, index_heads: int = 2,
                 index_dim: int = 16, ratio: int = 4, budget: int = 8, ple_layers=(),
                 ngram: Optional[NgramEmbedding] = None):
        from .qwen3_5 import Qwen35MoeModel
        self.cfg, self.C, self.device = cfg, streams, torch.device("cpu")
        self.tap = None          # called with (state, ids, streams) after every forward
        self.inner = Qwen35MoeModel(cfg, "cpu", torch.float32)
        self.ngram, self.ple_layers = ngram, tuple(ple_layers)
        self._hc = lambda injects=True: HyperConnection(cfg.hidden_size, streams, rank,
                                                        cfg.rms_norm_eps, injects)
        self._att = lambda: IndexedAttention(
            cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
            index_heads, index_dim, ratio, budget,
            rotary_dim=int(cfg.head_dim * cfg.partial_rotary_factor), theta=cfg.rope_theta,
            eps=cfg.rms_norm_eps)
        self.layers: list = []

    @classmethod
    def tiny(cls, seed: int = 0) -> "Qwen4ExpModel":
        """A small random model of every part (tests, ``random:qwen4_exp:tiny`` deployments)."""
        from .qwen3_5 import Qwen35MoeModel
        cfg = Qwen35MoeModel.tiny_config()
        g = torch.Generator().manual_seed(seed + 17)
        table = torch.randn(518, 6, generator=g).to(torch.float8_e4m3fn).view(torch.uint8)
        mult = torch.tensor([0x9E3779B97F4A7C15 - (1 << 64), 0x2545F4914F6CDD1D],
                            dtype=torch.int64)
        ngram = NgramEmbedding(table, 0.25, cfg.eos_token_id, mult, torch.tensor([211, 307]),
                               torch.tensor([0, 211]), 2)
        return cls(cfg, ple_layers=(0, 3), ngram=ngram).init_random(seed)

    def init_random(self, seed: int = 0) -> "Qwen4ExpModel":
        self.inner.init_random(seed)
        c = self.cfg
        for i, kind in enumerate(c.layer_types):
            L = {"attn_hc": self._hc().init_random(seed * 100 + 2 * i, 0.2),
                 "mlp_hc": self._hc().init_random(seed * 100 + 2 * i + 1, 0.2)}
            if kind == "full_attention":
                L["self_attn"] = self._att().init_random(seed * 100 + i)
            if i in self.ple_layers:
                # every PLE layer has a table of its own (``ple.ple_embedding``) over the same
                # hashing constants, and its convolution is dilated by the n-gram length
                ng = self.ngram
                g = torch.Generator().manual_seed(seed * 100 + 50 + i)
                table = torch.randn(ng.table.shape, generator=g).to(torch.float8_e4m3fn).view(
                    torch.uint8)
                L["ple_embedding"] = NgramEmbedding(table, ng.scale, ng.eos, ng.m, ng.P, ng.O,
                                                    ng.hpn)
                dim = ng.table.shape[1] * ng.P.shape[0]
                L["ple"] = PleLayer(c.hidden_size, self.C, dim, dilation=int(ng.m.shape[0]),
                                    eps=c.rms_norm_eps).init_random(seed * 100 + i, 0.2)
            self.layers.append(L)
        self.mixer = self._hc(False).init_random(seed * 100 + 99, 0.2)
        return self

    # ---------------------------------------------------------- checkpoints --
    _HC = (("hc_norm.weight", "hc_norm"), ("input_mix_weight_up.weight", "up"))
    _ATT = (("q_proj.weight", "q_proj"), ("k_proj.weight", "k_proj"), ("v_proj.weight", "v_proj"),
            ("o_proj.weight", "o_proj"), ("q_norm.weight", "q_norm"), ("k_norm.weight", "k_norm"),
            ("indexer.index_qk_proj.weight", "index_qk_proj"),
            ("indexer.q_layernorm.weight", "q_layernorm"),
            ("indexer.k_layernorm.weight", "k_layernorm"))
    _PLE = (("key_proj.weight", "key_proj"), ("value_proj.weight", "value_proj"))

    def hf_config(self) -> dict:
        c, ng = self.cfg, self.ngram
        att = next((L["self_attn"] for L in self.layers if "self_attn" in L), None)
        text = {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size,
                "num_hidden_layers": c.num_hidden_layers,
                "num_attention_heads": c.num_attention_heads,
                "num_key_value_heads": c.num_key_value_heads, "head_dim": c.head_dim,
                "rms_norm_eps": c.rms_norm_eps, "eos_token_id": c.eos_token_id,
                "layer_types": list(c.layer_types), "rope_theta": c.rope_theta,
                "partial_rotary_factor": c.partial_rotary_factor,
                "linear_num_key_heads": c.linear_num_key_heads,
                "linear_num_value_heads": c.linear_num_value_heads,
                "linear_key_head_dim": c.linear_key_head_dim,
                "linear_value_head_dim": c.linear_value_head_dim,
                "linear_conv_kernel_dim": c.linear_conv_kernel_dim,
                "num_experts": c.num_experts, "num_experts_per_tok": c.num_experts_per_tok,
                "moe_intermediate_size": c.moe_intermediate_size,
                "shared_expert_intermediate_size": c.shared_expert_intermediate_size,
                "hc_count": self.C, "hc_lowrank": self.mixer.rank,
                "ple_layer_ids": list(self.ple_layers)}
        if att is not None:
            text.update(indexer_n_heads=att.ih, indexer_head_dim=att.idim,
                        indexer_budget=att.budget, indexer_compress_ratio=att.ratio)
        if ng is not None:
            text.update(ngram_size=int(ng.m.shape[0]), heads_per_ngram=ng.hpn,
                        ple_embed_dim=int(ng.table.shape[1] * ng.P.shape[0]),
                        ple_conv_kernel_size=next(L["ple"].K for L in self.layers if "ple" in L))
        return {"architectures": ["Qwen4ExpForConditionalGeneration"], "text_config": text}

    def export_state(self) -> dict:
        """Tensors under the names the family's checkpoints use (the hybrid family's names for
        the gated delta network and the experts)."""
        w, out, c = self.inner.w, {}, self.cfg
        m = "model.language_model."
        out[m + "embed_tokens.weight"], out["lm_head.weight"] = w["embed"], w["lm_head"]

        def hc(prefix, h):
            for name, attr in self._HC:
                out[prefix + name] = getattr(h, attr)
            out[prefix + "input_mix_weight_down.weight"] = h.down[:h.rank]
            if h.injects:
                out[prefix + "block_inject_weight.weight"] = h.down[h.rank:]
        hc(m + "hyper_connection_mixer.", self.mixer)
        kd = c.linear_num_key_heads * c.linear_key_head_dim
        vd = c.linear_num_value_heads * c.linear_value_head_dim
        I = c.moe_intermediate_size
        for i, L in enumerate(self.layers):
            p, W = f"{m}layers.{i}.", w[i]
            hc(p + "attn_hyper_connection.", L["attn_hc"])
            hc(p + "mlp_hyper_connection.", L["mlp_hc"])
            if "self_attn" in L:
                for name, attr in self._ATT:
                    out[p + "self_attn." + name] = getattr(L["self_attn"], attr)
            else:
                a, q = p + "linear_attn.", W["qkvz"]
                out[a + "in_proj_qkv.weight"], out[a + "in_proj_z.weight"] = \
                    q[:2 * kd + vd], q[2 * kd + vd:2 * kd + 2 * vd]
                Hv = c.linear_num_value_heads
                out[a + "in_proj_b.weight"] = q[2 * kd + 2 * vd:2 * kd + 2 * vd + Hv]
                out[a + "in_proj_a.weight"] = q[2 * kd + 2 * vd + Hv:]
                out[a + "conv1d.weight"] = W["conv"].unsqueeze(1)
                out[a + "dt_bias"], out[a + "A_log"] = W["dt_bias"], (-W["A"]).log()
                out[a + "norm.weight"], out[a + "out_proj.weight"] = W["gnorm"], W["out"]
            x = p + "mlp."
            out[x + "gate.weight"] = W["router"]
            out[x + "experts.gate_up_proj"] = torch.cat([W["w13"][:, I:], W["w13"][:, :I]], 1)
            out[x + "experts.down_proj"] = W["w2"]
            S = c.shared_expert_intermediate_size
            out[x + "shared_expert.up_proj.weight"] = W["s13"][:S]
            out[x + "shared_expert.gate_proj.weight"] = W["s13"][S:]
            out[x + "shared_expert.down_proj.weight"] = W["s2"]
            out[x + "shared_expert_gate.weight"] = W["sgate"]
            if "ple" in L:
                e, ple, ng = p + "ple.", L["ple"], L["ple_embedding"]
                for name, attr in self._PLE:
                    out[e + name] = getattr(ple, attr)
                for n in ("norm_key", "norm_query", "norm_conv"):
                    out[e + n + ".weight"] = getattr(ple, n).reshape(-1)
                out[e + "conv1d.weight"] = ple.conv.unsqueeze(1)
                t = e + "ple_embedding."
                out[t + "ngram_embedding.shard_0.weight"] = ng.table.view(torch.float8_e4m3fn)
                out[t + "ngram_embedding.weight_scale"] = torch.tensor([ng.scale])
                out[t + "layer_multipliers"], out[t + "ngram_heads_vocab_sizes"] = ng.m, ng.P
                out[t + "ngram_heads_offsets"] = ng.O
        return {k: v.contiguous() for k, v in out.items()}

    @classmethod
    def from_checkpoint(cls, loader) -> "Qwen4ExpModel":
        """The model a checkpoint directory states (``config.json`` with ``text_config``:
        ``hc_count``, ``hc_lowrank``, ``indexer_*``, ``ple_layer_ids``, ``ngram_size`` ...)."""
        from .qwen3_5 import Qwen35Config
        t = dict(loader.config.get("text_config") or loader.config)
        cfg = Qwen35Config.from_hf({"text_config": t})
        f32 = lambda n: loader.get(n).to(torch.float32)
        m = "model.language_model."
        self = cls(cfg, streams=int(t["hc_count"]), rank=int(t["hc_lowrank"]),
                   index_heads=int(t.get("indexer_n_heads", 1)),
                   index_dim=int(t.get("indexer_head_dim", cfg.head_dim)),
                   ratio=int(t.get("indexer_compress_ratio", 1)),
                   budget=int(t.get("indexer_budget", 1)),
                   ple_layers=tuple(t.get("ple_layer_ids") or ()))
        self.inner.init_random(0)                       # shapes; every tensor is replaced below
        w, c = self.inner.w, cfg
        w["embed"] = f32(m + "embed_tokens.weight")
        w["lm_head"] = f32("lm_head.weight") if loader.has("lm_head.weight") else w["embed"]

        def hc(prefix, injects=True):
            h = self._hc(injects)
            for name, attr in self._HC:
                setattr(h, attr, f32(prefix + name))
            parts = [f32(prefix + "input_mix_weight_down.weight")]
            if injects:
                parts.append(f32(prefix + "block_inject_weight.weight"))
            h.down = torch.cat(parts, 0)
            return h
        self.mixer = hc(m + "hyper_connection_mixer.", False)
        I = c.moe_intermediate_size
        for i, kind in enumerate(c.layer_types):
            p, W = f"{m}layers.{i}.", w[i]
            L = {"attn_hc": hc(p + "attn_hyper_connection."),
                 "mlp_hc": hc(p + "mlp_hyper_connection.")}
            if kind == "full_attention":
                L["self_attn"] = self._att()
                for name, attr in self._ATT:
                    setattr(L["self_attn"], attr, f32(p + "self_attn." + name))
            else:
                a = p + "linear_attn."
                W["qkvz"] = torch.cat([f32(a + "in_proj_qkv.weight"), f32(a + "in_proj_z.weight"),
                                       f32(a + "in_proj_b.weight"), f32(a + "in_proj_a.weight")], 0)
                W["conv"], W["dt_bias"] = f32(a + "conv1d.weight").squeeze(1), f32(a + "dt_bias")
                W["A"], W["gnorm"] = -f32(a + "A_log").exp(), f32(a + "norm.weight")
                W["out"] = f32(a + "out_proj.weight")
            x = p + "mlp."
            gu = f32(x + "experts.gate_up_proj")
            W["router"], W["w13"] = f32(x + "gate.weight"), torch.cat([gu[:, I:], gu[:, :I]], 1)
            W["w2"] = f32(x + "experts.down_proj")
            W["s13"] = torch.cat([f32(x + "shared_expert.up_proj.weight"),
                                  f32(x + "shared_expert.gate_proj.weight")], 0)
            W["s2"], W["sgate"] = f32(x + "shared_expert.down_proj.weight"), \
                f32(x + "shared_expert_gate.weight")
            if i in self.ple_layers:
                e = p + "ple."
                t_ = e + "ple_embedding."
                shards = sorted((n for n in loader.names()
                                 if n.startswith(t_ + "ngram_embedding.shard_")),
                                key=lambda n: int(n.split("shard_")[1].split(".")[0]))
                table = torch.cat([loader.get(n).view(torch.uint8) for n in shards], 0) \
                    if shards else loader.get(t_ + "ngram_embedding.weight").view(torch.uint8)
                ng = NgramEmbedding(table, float(loader.get(t_ + "ngram_embedding.weight_scale")
                                                 .float().reshape(-1)[0]),
                                    c.eos_token_id, loader.get(t_ + "layer_multipliers"),
                                    loader.get(t_ + "ngram_heads_vocab_sizes"),
                                    loader.get(t_ + "ngram_heads_offsets"),
                                    int(t["heads_per_ngram"]))
                self.ngram = self.ngram or ng
                conv = f32(e + "conv1d.weight").squeeze(1)
                ple = PleLayer(c.hidden_size, self.C, int(t["ple_embed_dim"]),
                               kernel=conv.shape[1], dilation=int(ng.m.shape[0]),
                               eps=c.rms_norm_eps)
                for name, attr in self._PLE:
                    setattr(ple, attr, f32(e + name))
                for n in ("norm_key", "norm_query", "norm_conv"):
                    setattr(ple, n, f32(e + n + ".weight").view(self.C, c.hidden_size))
                ple.conv = conv
                L["ple"], L["ple_embedding"] = ple, ng
            self.layers.append(L)
        return self

    def new_state(self) -> dict:
        return {"inner": self.inner.new_state(), "attn": {}, "ple": {}, "ids": []}

    def forward(self, ids: torch.Tensor, state: dict, pos0: Optional[int] = None,
                return_streams: bool = False):
        """The request's next tokens ``ids`` [T] on top of ``state`` -> FP32 logits [T, vocab]
        (with ``return_streams`` also the read-out streams [T, C * H], which the drafter reads).
        Positions follow from the state; ``pos0`` (what the dense-state engine passes) is
        checked against it where the state counts tokens."""
        w, T = self.inner.w, ids.shape[0]
        if pos0 is not None and self.ngram is not None and pos0 != len(state["ids"]):
            raise ValueError(f"state holds {len(state['ids'])} tokens, the step starts at {pos0}")
        x = w["embed"][ids.long()]
        S = x.repeat(1, self.C)
        pending = None
        if self.ngram is not None:
            seen = len(state["ids"])
            state["ids"] = state["ids"] + ids.tolist()
            # an n-gram reaches n - 1 tokens back (further back reads as end of text only when
            # the request starts there)
            back = min(seen, int(self.ngram.m.shape[0]) - 1) if seen else 0
            recent = torch.tensor(state["ids"][seen - back:])
        for i, L in enumerate(self.layers):
            if "ple" in L:
                if pending is not None:
                    S, pending = HyperConnection.fold(S, pending[0], pending[1], self.C), None
                e = self._ngram_rows(L["ple_embedding"], recent, back, seen)
                add, state["ple"][i] = L["ple"].forward(e, S, state["ple"].get(i))
                S = S + add
            S, h, r = L["attn_hc"].read(S, pending)
            if "self_attn" in L:
                y, state["attn"][i], _ = L["self_attn"].forward(h, state["attn"].get(i))
            else:
                y = self.inner._linear_attention(w[i], h, state["inner"][i])
            S, h, r = L["mlp_hc"].read(S, (y, r))
            pending = (self.inner._mlp(w[i], h), r)
        S = HyperConnection.fold(S, pending[0], pending[1], self.C)
        logits = self.mixer.read(S)[1].float() @ w["lm_head"].float().t()
        if self.tap is not None:
            self.tap(state, ids, S)
        return (logits, S) if return_streams else logits

    @staticmethod
    def _ngram_rows(emb: NgramEmbedding, recent: torch.Tensor, back: int, seen: int):
        """Embedding rows of the new tokens; ``recent`` is the ``back`` tokens before them (the
        n-gram's reach, or the whole history when it is shorter) and them.  The window's first
        rows are computed and dropped."""
        return emb.forward(recent, torch.float32)[back:]

    def generate(self, prompt_ids: list, max_tokens: int) -> list:
        state, out = self.new_state(), []
        logits = self.forward(torch.tensor(prompt_ids), state)
        for _ in range(max_tokens):
            out.append(int(logits[-1].argmax()))
            if out[-1] == self.cfg.eos_token_id:
                break
            logits = self.forward(torch.tensor(out[-1:]), state)
        return out


class Qwen4Mtp:
    """The family's multi-token-prediction module.  An entry at position i reads the model's
    streams S of position i and the embedding e of the token at i + 1::

        e'   = fc_embedding(gemma(e; pre_fc_norm_embedding))
        S0_c = fc_hidden(gemma(S; pre_fc_norm_hidden)_c) + e'        one RMS over all C * H values
        S'   = layer(S0)       indexed attention with a cache of its own, then experts, each
                               behind a hyper-connection; the last combine folded
        draft logits = lm_head(mixer.read(S'))                      the model's head

    ``observe`` runs the entries of positions the model has computed (the drafter's cache then
    holds every committed position); ``draft`` chains further entries on the drafter's own
    streams and cuts the cache back to the committed length afterwards.  Reference behaviour:
    crates/models/src/qwen4_exp/mtp.rs:1-43 (reference project path).
    """

    def __init__(self, model: Qwen4ExpModel):
        self.model = model
        c, C = model.cfg, model.C
        H = c.hidden_size
        z = lambda *sh: torch.zeros(*sh)
        self.pre_fc_norm_embedding, self.pre_fc_norm_hidden = z(H), z(C * H)
        self.fc_embedding, self.fc_hidden = z(H, H), z(H, H)
        self.attn_hc, self.mlp_hc, self.mixer = model._hc(), model._hc(), model._hc(False)
        self.self_attn = model._att()
        self.mlp: dict = {}

    def init_random(self, seed: int = 0, std: float = 0.2) -> "Qwen4Mtp":
        c, g = self.model.cfg, torch.Generator().manual_seed(seed)
        rnd = lambda *sh: torch.randn(*sh, generator=g) * std
        H, I, S, E = c.hidden_size, c.moe_intermediate_size, c.shared_expert_intermediate_size, \
            c.num_experts
        self.pre_fc_norm_embedding, self.pre_fc_norm_hidden = rnd(H), rnd(self.model.C * H)
        self.fc_embedding, self.fc_hidden = rnd(H, H) / H ** 0.5 * 5, rnd(H, H) / H ** 0.5 * 5
        for j, m in enumerate((self.attn_hc, self.mlp_hc, self.mixer, self.self_attn)):
            m.init_random(seed * 10 + j, std)
        self.mlp = {"router": rnd(E, H), "w13": rnd(E, 2 * I, H) * 0.25, "w2": rnd(E, H, I) * 0.25,
                    "s13": rnd(2 * S, H) * 0.25, "s2": rnd(H, S) * 0.25, "sgate": rnd(1, H)}
        return self

    def _hcs(self):
        return (("mtp.layers.0.attn_hyper_connection.", "attn_hc"),
                ("mtp.layers.0.mlp_hyper_connection.", "mlp_hc"),
                ("mtp.hyper_connection_mixer.", "mixer"))

    def export_state(self) -> dict:
        """The module's tensors under ``mtp.*`` (one layer; the embedding and the head are the
        model's)."""
        c, out = self.model.cfg, {}
        for n in ("pre_fc_norm_embedding", "pre_fc_norm_hidden", "fc_embedding", "fc_hidden"):
            out[f"mtp.{n}.weight"] = getattr(self, n)
        for prefix, attr in self._hcs():
            h = getattr(self, attr)
            for name, field in Qwen4ExpModel._HC:
                out[prefix + name] = getattr(h, field)
            out[prefix + "input_mix_weight_down.weight"] = h.down[:h.rank]
            if h.injects:
                out[prefix + "block_inject_weight.weight"] = h.down[h.rank:]
        for name, field in Qwen4ExpModel._ATT:
            out["mtp.layers.0.self_attn." + name] = getattr(self.self_attn, field)
        x, W, I, S = "mtp.layers.0.mlp.", self.mlp, c.moe_intermediate_size, \
            c.shared_expert_intermediate_size
        out[x + "gate.weight"] = W["router"]
        out[x + "experts.gate_up_proj"] = torch.cat([W["w13"][:, I:], W["w13"][:, :I]], 1)
        out[x + "experts.down_proj"] = W["w2"]
        out[x + "shared_expert.up_proj.weight"] = W["s13"][:S]
        out[x + "shared_expert.gate_proj.weight"] = W["s13"][S:]
        out[x + "shared_expert.down_proj.weight"] = W["s2"]
        out[x + "shared_expert_gate.weight"] = W["sgate"]
        return {k: v.contiguous() for k, v in out.items()}

    def load_state(self, loader) -> "Qwen4Mtp":
        if loader.has("mtp.layers.1.self_attn.q_proj.weight"):
            raise ValueError("a multi-token-prediction module of more than one layer is not "
                             "served: a forward is not told its step")
        c = self.model.cfg
        f32 = lambda n: loader.get(n).to(torch.float32)
        for n in ("pre_fc_norm_embedding", "pre_fc_norm_hidden", "fc_embedding", "fc_hidden"):
            setattr(self, n, f32(f"mtp.{n}.weight"))
        for prefix, attr in self._hcs():
            h = getattr(self, attr)
            for name, field in Qwen4ExpModel._HC:
                setattr(h, field, f32(prefix + name))
            parts = [f32(prefix + "input_mix_weight_down.weight")]
            if h.injects:
                parts.append(f32(prefix + "block_inject_weight.weight"))
            h.down = torch.cat(parts, 0)
        for name, field in Qwen4ExpModel._ATT:
            setattr(self.self_attn, field, f32("mtp.layers.0.self_attn." + name))
        x, I = "mtp.layers.0.mlp.", c.moe_intermediate_size
        gu = f32(x + "experts.gate_up_proj")
        self.mlp = {"router": f32(x + "gate.weight"), "w13": torch.cat([gu[:, I:], gu[:, :I]], 1),
                    "w2": f32(x + "experts.down_proj"),
                    "s13": torch.cat([f32(x + "shared_expert.up_proj.weight"),
                                      f32(x + "shared_expert.gate_proj.weight")], 0),
                    "s2": f32(x + "shared_expert.down_proj.weight"),
                    "sgate": f32(x + "shared_expert_gate.weight")}
        return self

    def new_state(self) -> dict:
        return {"attn": None}

    def forward(self, S: torch.Tensor, next_ids: torch.Tensor, state: dict):
        """S [T, C * H] of positions p .. p + T - 1 with the tokens at p + 1 .. p + T ->
        (the entries' streams [T, C * H], draft logits [T, vocab] for positions p + 2 ..)."""
        m, C = self.model, self.model.C
        T, H = S.shape[0], m.cfg.hidden_size
        e = gemma_norm(m.inner.w["embed"][next_ids.long()].float(), self.pre_fc_norm_embedding,
                       m.cfg.rms_norm_eps) @ self.fc_embedding.t()
        Sn = gemma_norm(S.float(), self.pre_fc_norm_hidden, m.cfg.rms_norm_eps).view(T * C, H)
        S0 = ((Sn @ self.fc_hidden.t()).view(T, C, H) + e[:, None, :]).reshape(T, C * H)
        S1, h, r = self.attn_hc.read(S0)
        y, state["attn"], _ = self.self_attn.forward(h, state["attn"])
        S1, h, r = self.mlp_hc.read(S1, (y, r))
        S1 = HyperConnection.fold(S1, m.inner._mlp(self.mlp, h), r, C)
        return S1, self.mixer.read(S1)[1].float() @ m.inner.w["lm_head"].float().t()

    observe = forward

    def draft(self, S_last: torch.Tensor, logits_last: torch.Tensor, k: int, state: dict) -> list:
        """After ``observe`` over the committed positions: ``S_last`` [1, C * H] and
        ``logits_last`` [vocab] are its last entry's.  Returns k draft tokens: the first is the
        last entry's own prediction, the others come from entries chained on the drafter's
        streams, whose cache rows are cut away again."""
        out = [int(logits_last.argmax())]
        kept = None if state["attn"] is None else {n: t.shape[0] for n, t in state["attn"].items()}
        S = S_last
        for _ in range(k - 1):
            S, logits = self.forward(S, torch.tensor(out[-1:]), state)
            out.append(int(logits[-1].argmax()))
        if k > 1:
            state["attn"] = None if kept is None else \
                {n: t[:kept[n]] for n, t in state["attn"].items()}
        return out


class Qwen4MtpDrafter:
    """Drafts with the family's own multi-token-prediction module inside the dense-state
    engine.  The drafter's cache lives in the request's state (``state["mtp"]``), so the
    engine's snapshots, prefix restores and replays after a refused draft carry it along.
    After every forward of the model the entries of the positions whose next token is known
    are run; the last position waits for its token, which ``propose_from_state`` supplies
    before it chains the further drafts and cuts the cache back."""

    def __init__(self, mtp: Qwen4Mtp, k: int = 3):
        self.mtp, self.k = mtp, k
        mtp.model.tap = self._tap

    def _tap(self, state: dict, ids: torch.Tensor, S: torch.Tensor) -> None:
        ms = state.setdefault("mtp", {"attn": None, "S": None})
        rows = S[:-1] if ms["S"] is None else torch.cat([ms["S"], S[:-1]])
        nxt = ids[1:] if ms["S"] is None else ids
        if rows.shape[0]:
            self.mtp.observe(rows, nxt.to(torch.int64), ms)
        ms["S"] = S[-1:].clone()

    def propose(self, token_ids) -> list:
        return []                       # without the request's state there is nothing to read

    def propose_from_state(self, token_ids, state: dict) -> list:
        ms = state.get("mtp")
        if ms is None or ms["S"] is None:
            return []
        kept = None if ms["attn"] is None else {n: t.shape[0] for n, t in ms["attn"].items()}
        S, logits = self.mtp.forward(ms["S"], torch.tensor(list(token_ids[-1:])), ms)
        out = self.mtp.draft(S, logits[-1], self.k, ms)
        ms["attn"] = None if kept is None else {n: t[:kept[n]] for n, t in ms["attn"].items()}
        return out
