"""Qwen3.5-MoE text decoder: hybrid layers (three gated-delta-net layers for every
full-attention layer), attention with an output gate and partial rotary embedding,
experts plus a gated shared expert, zero-centred RMSNorm weights.

The decoder keeps a *dense* per-sequence state - key / value rows for the attention
layers, (convolution window, delta-rule matrix) for the linear layers - so a prompt
can be run in chunks and decoding is one more chunk of one token.  Projections, MLPs
and expert GEMMs go through the package's operators (tensor-core kernels on a GPU);
the recurrences and the dense attention are the FP32 formulas of
``ops/gated_delta.py`` / PyTorch.  Serving this family through the paged engine
(pages for its attention layers, state slots for its linear layers) is not wired.

Hugging Face names (``Qwen3_5MoeForCausalLM``): ``linear_attn.{in_proj_qkv,in_proj_z,
in_proj_b,in_proj_a,conv1d,out_proj,norm}``, ``dt_bias``, ``A_log``, ``self_attn.q_proj``
(queries and gates interleaved per head), ``mlp.experts.gate_up_proj`` (stacked),
``mlp.shared_expert*``.

Reference behaviour: crates/models/src/qwen3/decoder.rs:82-120,
crates/nn/src/modules/gated_delta_net.rs, crates/models/src/qwen3/config.rs
(reference project paths).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch

from ..ops import functional as F
from ..ops import gated_delta as GD
from ..ops import reference as R


@dataclass
class Qwen35Config:
    vocab_size: int = 248320
    hidden_size: int = 2048
    num_hidden_layers: int = 40
    layer_types: list = field(default_factory=list)
    num_attention_heads: int = 16
    num_key_value_heads: int = 2
    head_dim: int = 256
    partial_rotary_factor: float = 0.25
    rope_theta: float = 1e7
    rms_norm_eps: float = 1e-6
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    num_experts: int = 256
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 512
    shared_expert_intermediate_size: int = 512
    intermediate_size: int = 0              # dense variant (num_experts = 0): MLP width
    eos_token_id: int = 0
    mrope_section: tuple = (11, 11, 10)     # rotary frequencies owned by (t, h, w), interleaved
    image_token_id: int = 248056
    video_token_id: int = 248057

    @classmethod
    def from_hf(cls, d: dict) -> "Qwen35Config":
        outer = d
        d = d.get("text_config", d)
        rp = d.get("rope_parameters") or {}
        keys = {f for f in cls.__dataclass_fields__}
        kw = {k: v for k, v in d.items() if k in keys and v is not None}
        kw["rope_theta"] = float(rp.get("rope_theta", d.get("rope_theta", 1e7)))
        kw["partial_rotary_factor"] = float(rp.get("partial_rotary_factor",
                                                   d.get("partial_rotary_factor", 0.25)))
        kw["mrope_section"] = tuple(rp.get("mrope_section", (11, 11, 10)))
        if "num_experts" not in d and "num_local_experts" not in d:
            kw["num_experts"] = 0            # the dense variant of the family
        for k in ("image_token_id", "video_token_id"):
            if outer.get(k) is not None:
                kw[k] = int(outer[k])
        cfg = cls(**kw)
        if not cfg.layer_types:
            every = int(d.get("full_attention_interval", 4))
            cfg.layer_types = ["full_attention" if (i + 1) % every == 0 else "linear_attention"
                               for i in range(cfg.num_hidden_layers)]
        if isinstance(cfg.eos_token_id, (list, tuple)):
            cfg.eos_token_id = int(cfg.eos_token_id[0])
        return cfg


def norm_mrope(x, w, pos3, inv_freq, rot: int, section, eps: float):
    """Per-head RMSNorm (weight ``w``), then rotary embedding over the first ``rot`` channels
    whose frequency j turns with the temporal, row or column position according to the
    interleaved sections (t h w t h w ... t t).  x [T, H, D], pos3 [3, T]."""
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    nf = rot // 2
    axis = torch.zeros(nf, dtype=torch.long, device=x.device)
    for a, off in ((1, 1), (2, 2)):
        axis[off:section[a] * 3:3] = a
    ang = pos3.to(x.device).float()[axis, :].t() * inv_freq.float()[None, :]          # [T, nf]
    cos = torch.cat([ang.cos(), ang.cos()], -1)[:, None, :]
    sin = torch.cat([ang.sin(), ang.sin()], -1)[:, None, :]
    r = xf[..., :rot]
    turned = torch.cat([-r[..., nf:], r[..., :nf]], -1)
    return torch.cat([r * cos + turned * sin, xf[..., rot:]], -1).to(x.dtype)


@dataclass
class LayerState:
    k: Optional[torch.Tensor] = None        # attention: [n, Hkv, D]
    v: Optional[torch.Tensor] = None
    conv: Optional[torch.Tensor] = None     # linear: [K - 1, conv channels]
    rule: Optional[torch.Tensor] = None     # linear: [Hv, Dk, Dv] FP32


class SequenceState(list):
    """The per-layer states of one sequence; ``mtp`` is where a drafter keeps its own cache, so
    that copies of the state (snapshots, replays) carry it."""
    mtp = None


class Qwen35MoeModel:
    def __init__(self, cfg: Qwen35Config, device="cpu", dtype=torch.bfloat16):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.tap = None      # called with (state, ids, hidden rows before the final norm, pos0)
        self.rot = int(cfg.head_dim * cfg.partial_rotary_factor)
        self.inv_freq = R.rope_inv_freq(self.rot, cfg.rope_theta, self.device)
        self.w: dict = {}

    # ------------------------------------------------------------- weights --
    def load_state(self, loader) -> "Qwen35MoeModel":
        cfg = self.cfg
        names = set(loader.names())
        prefix = "model.language_model." if any(n.startswith("model.language_model.")
                                                for n in names) else "model."

        def get(n, dtype=None):
            return loader.get(n).to(device=self.device, dtype=dtype or self.dtype)
        w = self.w
        w["embed"] = get(prefix + "embed_tokens.weight")
        w["norm"] = get(prefix + "norm.weight", torch.float32) + 1.0
        w["lm_head"] = get("lm_head.weight") if "lm_head.weight" in names else w["embed"]
        I = cfg.moe_intermediate_size
        for i, kind in enumerate(cfg.layer_types):
            p = f"{prefix}layers.{i}."
            L = {"kind": kind,
                 "in_norm": get(p + "input_layernorm.weight", torch.float32) + 1.0,
                 "post_norm": get(p + "post_attention_layernorm.weight", torch.float32) + 1.0}
            if kind == "full_attention":
                a = p + "self_attn."
                L["q"], L["k"], L["v"], L["o"] = (get(a + f"{n}_proj.weight") for n in "qkvo")
                L["q_norm"] = get(a + "q_norm.weight", torch.float32) + 1.0
                L["k_norm"] = get(a + "k_norm.weight", torch.float32) + 1.0
            else:
                a = p + "linear_attn."
                if (a + "in_proj_qkvz.weight") in names:
                    # Qwen3-Next packs the projections per key head: [q k v.. z..] and [b.. a..]
                    Hk, Dk, Dv = (cfg.linear_num_key_heads, cfg.linear_key_head_dim,
                                  cfg.linear_value_head_dim)
                    r = cfg.linear_num_value_heads // Hk
                    qkvz = get(a + "in_proj_qkvz.weight").view(Hk, 2 * Dk + 2 * r * Dv, -1)
                    ba = get(a + "in_proj_ba.weight").view(Hk, 2 * r, -1)
                    parts = [qkvz[:, :Dk], qkvz[:, Dk:2 * Dk], qkvz[:, 2 * Dk:2 * Dk + r * Dv],
                             qkvz[:, 2 * Dk + r * Dv:], ba[:, :r], ba[:, r:]]
                    L["qkvz"] = torch.cat([t.reshape(-1, t.shape[-1]) for t in parts], 0).contiguous()
                else:
                    L["qkvz"] = torch.cat([get(a + "in_proj_qkv.weight"),
                                           get(a + "in_proj_z.weight"),
                                           get(a + "in_proj_b.weight"),
                                           get(a + "in_proj_a.weight")], 0)
                L["conv"] = get(a + "conv1d.weight", torch.float32).squeeze(1)     # [C, K]
                L["dt_bias"] = get(a + "dt_bias", torch.float32)
                L["A"] = -get(a + "A_log", torch.float32).exp()
                L["gnorm"] = get(a + "norm.weight")
                L["out"] = get(a + "out_proj.weight")
            m = p + "mlp."
            if not cfg.num_experts:          # dense variant: one gated MLP a layer
                L["d13"] = torch.cat([get(m + "up_proj.weight"), get(m + "gate_proj.weight")], 0)
                L["d2"] = get(m + "down_proj.weight")
                w[i] = L
                continue
            L["router"] = get(m + "gate.weight")
            gu = get(m + "experts.gate_up_proj")                 # [E, 2I, H]: gate rows, up rows
            L["w13"] = torch.cat([gu[:, I:], gu[:, :I]], 1).contiguous()
            L["w2"] = get(m + "experts.down_proj").contiguous()
            L["s13"] = torch.cat([get(m + "shared_expert.up_proj.weight"),
                                  get(m + "shared_expert.gate_proj.weight")], 0)
            L["s2"] = get(m + "shared_expert.down_proj.weight")
            L["sgate"] = get(m + "shared_expert_gate.weight")
            w[i] = L
        return self

    def init_random(self, seed: int = 0, std: float = 0.05) -> "Qwen35MoeModel":
        """Random weights of the configured shapes (tests, ``random:`` deployments)."""
        c, g = self.cfg, torch.Generator().manual_seed(seed)
        if not c.layer_types:
            c.layer_types = ["full_attention" if (i + 1) % 4 == 0 else "linear_attention"
                             for i in range(c.num_hidden_layers)]

        def rnd(*shape, dtype=None):
            return (torch.randn(*shape, generator=g) * std).to(device=self.device,
                                                               dtype=dtype or self.dtype)

        def ones(n):
            return torch.ones(n, dtype=torch.float32, device=self.device)
        H, D, I = c.hidden_size, c.head_dim, c.moe_intermediate_size
        kd = c.linear_num_key_heads * c.linear_key_head_dim
        vd = c.linear_num_value_heads * c.linear_value_head_dim
        w = self.w
        w["embed"], w["norm"], w["lm_head"] = rnd(c.vocab_size, H), ones(H), rnd(c.vocab_size, H)
        for i, kind in enumerate(c.layer_types):
            L = {"kind": kind, "in_norm": ones(H), "post_norm": ones(H)}
            if kind == "full_attention":
                L["q"] = rnd(c.num_attention_heads * 2 * D, H)
                L["k"], L["v"] = rnd(c.num_key_value_heads * D, H), rnd(c.num_key_value_heads * D, H)
                L["o"] = rnd(H, c.num_attention_heads * D)
                L["q_norm"], L["k_norm"] = ones(D), ones(D)
            else:
                L["qkvz"] = rnd(2 * kd + 2 * vd + 2 * c.linear_num_value_heads, H)
                L["conv"] = rnd(2 * kd + vd, c.linear_conv_kernel_dim, dtype=torch.float32) * 4
                L["dt_bias"] = ones(c.linear_num_value_heads)
                L["A"] = -(torch.rand(c.linear_num_value_heads, generator=g) * 4 + 0.5).to(self.device)
                L["gnorm"] = ones(c.linear_value_head_dim).to(self.dtype)
                L["out"] = rnd(H, vd)
            L["router"] = rnd(c.num_experts, H)
            L["w13"], L["w2"] = rnd(c.num_experts, 2 * I, H), rnd(c.num_experts, H, I)
            S = c.shared_expert_intermediate_size
            L["s13"], L["s2"], L["sgate"] = rnd(2 * S, H), rnd(H, S), rnd(1, H)
            w[i] = L
        return self

    @classmethod
    def tiny_config(cls) -> Qwen35Config:
        return Qwen35Config(vocab_size=1024, hidden_size=64, num_hidden_layers=4,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                            linear_num_key_heads=2, linear_num_value_heads=4,
                            linear_key_head_dim=16, linear_value_head_dim=16, num_experts=8,
                            num_experts_per_tok=2, moe_intermediate_size=32,
                            shared_expert_intermediate_size=32, eos_token_id=1023)

    # ------------------------------------------------------------- forward --
    def new_state(self) -> list:
        return SequenceState(LayerState() for _ in self.cfg.layer_types)

    def _norm_mrope(self, x, w, pos3):
        return norm_mrope(x, w, pos3, self.inv_freq, self.rot, self.cfg.mrope_section,
                          self.cfg.rms_norm_eps)

    def _attention(self, L, n, st: LayerState, pos0: int, pos3=None):
        c, D = self.cfg, self.cfg.head_dim
        T = n.shape[0]
        Hq, Hkv = c.num_attention_heads, c.num_key_value_heads
        qg = F.linear(n, L["q"]).view(T, Hq, 2 * D)
        q, gate = qg[..., :D], qg[..., D:].reshape(T, Hq * D)
        k = F.linear(n, L["k"]).view(T, Hkv, D)
        v = F.linear(n, L["v"]).view(T, Hkv, D)
        pos = torch.arange(pos0, pos0 + T, device=n.device)
        if pos3 is None:
            q, k = R.qk_norm_rope(q.contiguous(), k, L["q_norm"], L["k_norm"], pos, self.inv_freq,
                                  self.rot, False, c.rms_norm_eps)
        else:
            q, k = self._norm_mrope(q, L["q_norm"], pos3), self._norm_mrope(k, L["k_norm"], pos3)
        st.k = k if st.k is None else torch.cat([st.k, k], 0)
        st.v = v if st.v is None else torch.cat([st.v, v], 0)
        from ..ops.attention import cached_causal_attention
        att = cached_causal_attention(q, st.k, st.v, 1.0 / math.sqrt(D)).reshape(T, Hq * D)
        att = (att * torch.sigmoid(gate.float())).to(n.dtype)
        return F.linear(att, L["o"])

    def _linear_attention(self, L, n, st: LayerState):
        c = self.cfg
        T = n.shape[0]
        Hk, Hv, Dk, Dv = (c.linear_num_key_heads, c.linear_num_value_heads,
                          c.linear_key_head_dim, c.linear_value_head_dim)
        kd, vd = Hk * Dk, Hv * Dv
        proj = F.linear(n, L["qkvz"])
        mixed, z = proj[:, :2 * kd + vd], proj[:, 2 * kd + vd:2 * kd + 2 * vd]
        b, a = proj[:, 2 * kd + 2 * vd:2 * kd + 2 * vd + Hv], proj[:, 2 * kd + 2 * vd + Hv:]
        if n.is_cuda and GD.USE_KERNELS and Dk in GD._KERNEL_DK:
            # kernels: the convolution reads the projection in place, the rule reads q / k / v
            # as views of the convolved rows (a key head serves Hv / Hk value heads) and forms
            # the gates from the raw projections; the state is updated where it lives
            mixed, st.conv = GD.causal_conv1d(mixed, L["conv"], st.conv)
            if st.rule is None:
                st.rule = torch.zeros(Hv, Dk, Dv, dtype=torch.float32, device=n.device)
            cu, slots = GD._one_sequence(T, n.device)
            o = GD.gated_delta_rule_packed(
                mixed[:, :kd].view(T, Hk, Dk), mixed[:, kd:2 * kd].view(T, Hk, Dk),
                mixed[:, 2 * kd:].view(T, Hv, Dv), st.rule.unsqueeze(0), cu, slots,
                raw=(a, b, L["A"].float().contiguous(), L["dt_bias"].float().contiguous()))
            o = GD.rmsnorm_gated(o, L["gnorm"], z.unflatten(1, (Hv, Dv)), c.rms_norm_eps)
            return F.linear(o.reshape(T, vd), L["out"])
        mixed, st.conv = GD.causal_conv1d(mixed.contiguous(), L["conv"], st.conv)
        q = mixed[:, :kd].reshape(T, Hk, Dk)
        k = mixed[:, kd:2 * kd].reshape(T, Hk, Dk)
        v = mixed[:, 2 * kd:].reshape(T, Hv, Dv)
        if Hv // Hk > 1:
            q, k = q.repeat_interleave(Hv // Hk, 1), k.repeat_interleave(Hv // Hk, 1)
        beta = torch.sigmoid(b.float())
        g = L["A"] * torch.nn.functional.softplus(a.float() + L["dt_bias"])
        o, st.rule = GD.gated_delta_rule(q, k, v, g, beta, st.rule)
        o = GD.rmsnorm_gated(o.to(n.dtype), L["gnorm"], z.reshape(T, Hv, Dv), c.rms_norm_eps)
        return F.linear(o.reshape(T, vd), L["out"])

    def _mlp(self, L, n):
        c = self.cfg
        if "d13" in L:
            return F.linear(F.linear_gated(n, L["d13"]), L["d2"])
        logits = F.linear(n, L["router"], out_dtype=torch.float32)
        ids, wts = F.topk_softmax(logits, c.num_experts_per_tok, True)
        y = F.moe_experts(n, ids, wts, L["w13"], L["w2"])
        shared = F.linear(F.linear_gated(n, L["s13"]), L["s2"])
        sg = torch.sigmoid(F.linear(n, L["sgate"], out_dtype=torch.float32))
        return y + (shared.float() * sg).to(n.dtype)

    def forward(self, ids: torch.Tensor, state: list, pos0: int = 0, embeds=None,
                positions3=None, deepstack=None) -> torch.Tensor:
        """Runs ``ids`` [T] at positions pos0 .. on top of ``state``; returns FP32 logits
        [T, vocab].  ``embeds`` [T, hidden] replaces the embedding lookup (vision rows spliced
        in); ``positions3`` [3, T] are the (temporal, row, column) rotary positions of a
        multimodal prompt (text tokens carry the same value on all three)."""
        c, w = self.cfg, self.w
        x = w["embed"][ids.to(self.device).long()] if embeds is None else \
            embeds.to(device=self.device, dtype=self.dtype)
        for i in range(c.num_hidden_layers):
            L, st = w[i], state[i]
            n = R.rmsnorm(x, L["in_norm"], c.rms_norm_eps)
            mix = self._attention(L, n, st, pos0, positions3) if L["kind"] == "full_attention" \
                else self._linear_attention(L, n, st)
            x = x + mix
            n = R.rmsnorm(x, L["post_norm"], c.rms_norm_eps)
            x = x + self._mlp(L, n)
        if self.tap is not None:
            self.tap(state, ids, x, pos0)
        return F.linear(R.rmsnorm(x, w["norm"], c.rms_norm_eps), w["lm_head"],
                        out_dtype=torch.float32)

    def decode_batch(self, tokens: torch.Tensor, states: list, pos3: torch.Tensor) -> torch.Tensor:
        """One decode position of B sequences at once: ``tokens`` [B], ``states`` a list of B
        per-sequence states, ``pos3`` [3, B] rotary positions.  Projections, MLPs and experts
        run on all rows together; the delta rule and the convolution advance as one batched
        step; attention reads each sequence's own keys.  Returns FP32 logits [B, vocab]."""
        c, w = self.cfg, self.w
        B = tokens.shape[0]
        x = w["embed"][tokens.to(self.device).long()]
        Hq, Hkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        Hk, Hv, Dk, Dv = (c.linear_num_key_heads, c.linear_num_value_heads,
                          c.linear_key_head_dim, c.linear_value_head_dim)
        kd, vd = Hk * Dk, Hv * Dv
        for i in range(c.num_hidden_layers):
            L = w[i]
            n = R.rmsnorm(x, L["in_norm"], c.rms_norm_eps)
            if L["kind"] == "full_attention":
                qg = F.linear(n, L["q"]).view(B, Hq, 2 * D)
                q, gate = qg[..., :D], qg[..., D:].reshape(B, Hq * D)
                k = F.linear(n, L["k"]).view(B, Hkv, D)
                v = F.linear(n, L["v"]).view(B, Hkv, D)
                q = self._norm_mrope(q, L["q_norm"], pos3)
                k = self._norm_mrope(k, L["k_norm"], pos3)
                from ..ops.attention import cached_causal_attention
                att = torch.empty(B, Hq * D, dtype=torch.float32, device=x.device)
                for b in range(B):
                    st = states[b][i]
                    st.k = k[b:b + 1] if st.k is None else torch.cat([st.k, k[b:b + 1]], 0)
                    st.v = v[b:b + 1] if st.v is None else torch.cat([st.v, v[b:b + 1]], 0)
                    att[b] = cached_causal_attention(q[b:b + 1], st.k, st.v,
                                                     1.0 / math.sqrt(D)).reshape(Hq * D)
                mix = F.linear((att * torch.sigmoid(gate.float())).to(n.dtype), L["o"])
            else:
                proj = F.linear(n, L["qkvz"])
                mixed, z = proj[:, :2 * kd + vd], proj[:, 2 * kd + vd:2 * kd + 2 * vd]
                bb, aa = proj[:, 2 * kd + 2 * vd:2 * kd + 2 * vd + Hv], proj[:, 2 * kd + 2 * vd + Hv:]
                Kc = L["conv"].shape[1]
                if x.is_cuda and GD.USE_KERNELS and Dk in GD._KERNEL_DK:
                    # one packed launch per operator over the batch; the per-request states
                    # are slots of a pool that the kernels update in place
                    pool_c = torch.stack([states[b][i].conv if states[b][i].conv is not None else
                                          torch.zeros(Kc - 1, mixed.shape[1], dtype=mixed.dtype,
                                                      device=mixed.device) for b in range(B)])
                    pool_r = torch.stack([states[b][i].rule if states[b][i].rule is not None else
                                          torch.zeros(Hv, Dk, Dv, device=x.device) for b in range(B)])
                    cu = torch.arange(B + 1, dtype=torch.int32, device=x.device)
                    y, _ = GD.causal_conv1d(mixed, L["conv"], pool_c, cu=cu, slots=cu[:B])
                    o = GD.gated_delta_rule_packed(
                        y[:, :kd].view(B, Hk, Dk), y[:, kd:2 * kd].view(B, Hk, Dk),
                        y[:, 2 * kd:].view(B, Hv, Dv), pool_r, cu, cu[:B],
                        raw=(aa, bb, L["A"].float().contiguous(), L["dt_bias"].float().contiguous()))
                    for b in range(B):
                        states[b][i].conv, states[b][i].rule = pool_c[b], pool_r[b]
                    o = GD.rmsnorm_gated(o, L["gnorm"], z.unflatten(1, (Hv, Dv)), c.rms_norm_eps)
                    x = x + F.linear(o.reshape(B, vd), L["out"])
                    x = x + self._mlp(L, R.rmsnorm(x, L["post_norm"], c.rms_norm_eps))
                    continue
                conv = torch.stack([states[b][i].conv if states[b][i].conv is not None else
                                    torch.zeros(Kc - 1, mixed.shape[1], dtype=mixed.dtype,
                                                device=mixed.device) for b in range(B)])
                win = torch.cat([conv, mixed[:, None, :]], 1).float()            # [B, K, C]
                y = torch.nn.functional.silu((win * L["conv"].float().t()[None]).sum(1)).to(mixed.dtype)
                q = GD.l2norm(y[:, :kd].reshape(B, Hk, Dk).float()) * (Dk ** -0.5)
                k = GD.l2norm(y[:, kd:2 * kd].reshape(B, Hk, Dk).float())
                v = y[:, 2 * kd:].reshape(B, Hv, Dv).float()
                if Hv // Hk > 1:
                    q, k = q.repeat_interleave(Hv // Hk, 1), k.repeat_interleave(Hv // Hk, 1)
                beta = torch.sigmoid(bb.float())
                g = L["A"] * torch.nn.functional.softplus(aa.float() + L["dt_bias"])
                S = torch.stack([states[b][i].rule if states[b][i].rule is not None else
                                 torch.zeros(Hv, Dk, Dv, device=x.device) for b in range(B)])
                S = S * g.exp()[:, :, None, None]
                d = (v - torch.einsum("bhkv,bhk->bhv", S, k)) * beta[:, :, None]
                S = S + k[:, :, :, None] * d[:, :, None, :]
                o = torch.einsum("bhkv,bhk->bhv", S, q)
                for b in range(B):
                    states[b][i].conv = win[b, 1:].to(mixed.dtype)
                    states[b][i].rule = S[b]
                o = GD.rmsnorm_gated(o.to(n.dtype), L["gnorm"], z.reshape(B, Hv, Dv), c.rms_norm_eps)
                mix = F.linear(o.reshape(B, vd), L["out"])
            x = x + mix
            x = x + self._mlp(L, R.rmsnorm(x, L["post_norm"], c.rms_norm_eps))
        if self.tap is not None:
            for b in range(B):
                self.tap(states[b], tokens[b:b + 1], x[b:b + 1], int(pos3[0, b]))
        return F.linear(R.rmsnorm(x, w["norm"], c.rms_norm_eps), w["lm_head"],
                        out_dtype=torch.float32)

    def generate(self, prompt_ids: list, max_tokens: int, chunk: int = 512) -> list:
        """Greedy decoding with chunked prefill."""
        state, out, pos = self.new_state(), [], 0
        ids = torch.tensor(prompt_ids, device=self.device)
        logits = None
        for lo in range(0, len(prompt_ids), chunk):
            logits = self.forward(ids[lo:lo + chunk], state, pos)
            pos += min(chunk, len(prompt_ids) - lo)
        for _ in range(max_tokens):
            tok = int(logits[-1].argmax())
            out.append(tok)
            if tok == self.cfg.eos_token_id:
                break
            logits = self.forward(torch.tensor([tok], device=self.device), state, pos)
            pos += 1
        return out


def mrope_positions(input_ids, image_token_id: int, grids: list, merge: int, start: int = 0):
    """Rotary positions of a prompt with images: text tokens advance all three axes together;
    the merged patches of an image (t, h, w) keep the temporal value of the image's start and
    count rows / columns from it; the text after an image continues at start + max(h, w) / merge.
    Returns (positions [3, T], next position)."""
    ids = input_ids.tolist() if hasattr(input_ids, "tolist") else list(input_ids)
    cols, cur, i, g = [], start, 0, iter(grids)
    while i < len(ids):
        if ids[i] != image_token_id:
            cols.append(torch.tensor([[cur], [cur], [cur]]))
            cur += 1
            i += 1
            continue
        t, h, w = next(g)
        gh, gw = h // merge, w // merge
        n = t * gh * gw
        assert all(x == image_token_id for x in ids[i:i + n]), "placeholders do not cover the image"
        hh = torch.arange(cur, cur + gh).repeat_interleave(gw * t)
        ww = torch.arange(cur, cur + gw).repeat(gh * t)
        cols.append(torch.stack([torch.full((n,), cur), hh, ww]))
        cur += max(h, w) // merge
        i += n
    return torch.cat(cols, 1), cur


class Qwen35Multimodal:
    """The hybrid decoder with the vision tower in front: image rows replace the
    placeholder tokens of the prompt, positions are the three-axis ones, decoding continues
    on all axes from where the prompt ended (``Qwen3_5MoeForConditionalGeneration``)."""

    def __init__(self, text: Qwen35MoeModel, tower):
        self.text, self.tower = text, tower

    def prefill(self, prompt_ids: list, pixels, grids: list, state: list):
        """Returns (logits [T, vocab], next rotary position)."""
        c = self.text.cfg
        ids = torch.tensor(prompt_ids, device=self.text.device)
        emb = self.text.w["embed"][ids.long()]
        deep = None
        if pixels is not None:
            from .qwen3_vl_vision import splice
            rows, deep_rows = self.tower.forward(pixels, grids)
            emb = splice(emb, ids, c.image_token_id, rows)
            if deep_rows:
                deep = ((ids == c.image_token_id).nonzero(as_tuple=True)[0], deep_rows)
        pos3, nxt = mrope_positions(prompt_ids, c.image_token_id, grids or [],
                                    self.tower.cfg.spatial_merge_size)
        return self.text.forward(ids, state, 0, embeds=emb, positions3=pos3, deepstack=deep), nxt

    def generate(self, prompt_ids: list, pixels, grids: list, max_tokens: int) -> list:
        state = self.text.new_state()
        logits, pos = self.prefill(prompt_ids, pixels, grids, state)
        out = []
        for _ in range(max_tokens):
            tok = int(logits[-1].argmax())
            out.append(tok)
            if tok == self.text.cfg.eos_token_id:
                break
            p3 = torch.full((3, 1), pos)
            logits = self.text.forward(torch.tensor([tok], device=self.text.device), state, 0,
                                       positions3=p3)
            pos += 1
        return out


class HybridMtp:
    """Multi-token-prediction module of the hybrid family (``mtp.*``): one gated-attention
    decoder layer over ``fc([norm_e(embed(t_{p+1})) ; norm_h(h_p)])`` with a key / value stream
    of its own, the model's embedding and output matrices, and ``mtp.norm`` before the head.
    Reference behaviour: crates/models/src/qwen3/mtp.rs (reference project path)."""

    def __init__(self, model: Qwen35MoeModel):
        self.model, self.w = model, {}

    def init_random(self, seed: int = 0, std: float = 0.05) -> "HybridMtp":
        m, c = self.model, self.model.cfg
        g = torch.Generator().manual_seed(seed)
        rnd = lambda *sh: (torch.randn(*sh, generator=g) * std).to(m.device, m.dtype)
        ones = lambda n: torch.ones(n, dtype=torch.float32, device=m.device)
        H, D, I, S = c.hidden_size, c.head_dim, c.moe_intermediate_size, \
            c.shared_expert_intermediate_size
        L = {"kind": "full_attention", "in_norm": ones(H), "post_norm": ones(H),
             "q": rnd(c.num_attention_heads * 2 * D, H), "k": rnd(c.num_key_value_heads * D, H),
             "v": rnd(c.num_key_value_heads * D, H), "o": rnd(H, c.num_attention_heads * D),
             "q_norm": ones(D), "k_norm": ones(D)}
        if c.num_experts:
            L.update(router=rnd(c.num_experts, H), w13=rnd(c.num_experts, 2 * I, H),
                     w2=rnd(c.num_experts, H, I), s13=rnd(2 * S, H), s2=rnd(H, S),
                     sgate=rnd(1, H))
        else:
            L.update(d13=rnd(2 * c.intermediate_size, H), d2=rnd(H, c.intermediate_size))
        self.w = {"fc": rnd(H, 2 * H), "norm_e": ones(H), "norm_h": ones(H), "norm": ones(H),
                  "layer": L}
        return self

    def load_state(self, loader, prefix: str = "mtp.") -> "HybridMtp":
        m, c = self.model, self.model.cfg
        get = lambda n, dt=None: loader.get(prefix + n).to(device=m.device, dtype=dt or m.dtype)
        gain = lambda n: get(n, torch.float32) + 1.0
        p, I = "layers.0.", c.moe_intermediate_size
        L = {"kind": "full_attention", "in_norm": gain(p + "input_layernorm.weight"),
             "post_norm": gain(p + "post_attention_layernorm.weight"),
             "q_norm": gain(p + "self_attn.q_norm.weight"),
             "k_norm": gain(p + "self_attn.k_norm.weight")}
        for n in "qkvo":
            L[n] = get(p + f"self_attn.{n}_proj.weight")
        x = p + "mlp."
        if c.num_experts:
            gu = get(x + "experts.gate_up_proj")
            L.update(router=get(x + "gate.weight"),
                     w13=torch.cat([gu[:, I:], gu[:, :I]], 1).contiguous(),
                     w2=get(x + "experts.down_proj").contiguous(),
                     s13=torch.cat([get(x + "shared_expert.up_proj.weight"),
                                    get(x + "shared_expert.gate_proj.weight")], 0),
                     s2=get(x + "shared_expert.down_proj.weight"),
                     sgate=get(x + "shared_expert_gate.weight"))
        else:
            L.update(d13=torch.cat([get(x + "up_proj.weight"), get(x + "gate_proj.weight")], 0),
                     d2=get(x + "down_proj.weight"))
        self.w = {"fc": get("fc.weight"), "norm_e": gain("pre_fc_norm_embedding.weight"),
                  "norm_h": gain("pre_fc_norm_hidden.weight"), "norm": gain("norm.weight"),
                  "layer": L}
        return self

    def rows(self, hidden: torch.Tensor, next_ids: torch.Tensor, pos0: int, st: LayerState):
        """hidden [T, H] of positions pos0 .. with the token after each -> (the layer's output
        [T, H], logits [T, vocab]); ``st`` is the module's own key / value stream."""
        m, c, w = self.model, self.model.cfg, self.w
        e = m.w["embed"][next_ids.to(m.device).long()]
        x = F.linear(torch.cat([R.rmsnorm(e, w["norm_e"], c.rms_norm_eps),
                                R.rmsnorm(hidden.to(m.dtype), w["norm_h"], c.rms_norm_eps)], -1),
                     w["fc"])
        L = w["layer"]
        x = x + m._attention(L, R.rmsnorm(x, L["in_norm"], c.rms_norm_eps), st, pos0)
        x = x + m._mlp(L, R.rmsnorm(x, L["post_norm"], c.rms_norm_eps))
        return x, F.linear(R.rmsnorm(x, w["norm"], c.rms_norm_eps), m.w["lm_head"],
                           out_dtype=torch.float32)


class HybridMtpDrafter:
    """Drafts with ``HybridMtp`` inside the dense-state engine.  The module's key / value
    stream and the hidden row that still waits for its next token live in the sequence's state
    (``state.mtp``); every forward of the model extends them, ``propose_from_state`` runs the
    waiting row with the newest token, chains k - 1 further entries on the module's own outputs
    and cuts the stream back."""

    def __init__(self, mtp: HybridMtp, k: int = 2):
        self.mtp, self.k = mtp, k
        mtp.model.tap = self._tap

    def _tap(self, state, ids, hidden, pos0: int) -> None:
        if not isinstance(state, SequenceState):
            return
        ms = state.mtp
        if ms is None:
            ms = state.mtp = {"kv": LayerState(), "h": None, "pos": 0}
        rows = hidden[:-1] if ms["h"] is None else torch.cat([ms["h"], hidden[:-1]])
        nxt = ids[1:] if ms["h"] is None else ids
        if rows.shape[0]:
            self.mtp.rows(rows, nxt, ms["pos"], ms["kv"])
            ms["pos"] += rows.shape[0]
        ms["h"] = hidden[-1:].clone()

    def propose(self, token_ids) -> list:
        return []

    def propose_from_state(self, token_ids, state) -> list:
        ms = getattr(state, "mtp", None)
        if ms is None or ms["h"] is None or ms["pos"] != len(token_ids) - 2:
            return []                    # the stream does not cover the sequence: no drafts
        kv = ms["kv"]
        kept = 0 if kv.k is None else kv.k.shape[0]
        h, tok, out = ms["h"], int(token_ids[-1]), []
        for j in range(self.k):
            h, logits = self.mtp.rows(h, torch.tensor([tok]), ms["pos"] + j, kv)
            tok = int(logits[-1].argmax())
            out.append(tok)
        kv.k, kv.v = (None, None) if kept == 0 else (kv.k[:kept], kv.v[:kept])
        return out
