"""Qwen3-VL language model (Qwen3 decoder, dense or with experts, with three-axis rotary
positions and deep-stack inputs) on a dense per-sequence state.

Differences from the text-only Qwen3 decoder: the rotary embedding covers the whole head
and its frequencies are shared out between the temporal, row and column position
(interleaved sections, 24 / 20 / 20 of 64 by default); the vision tower's deep-stack rows
are *added* to the hidden states of the image positions after each of the first few
layers.  The class has the interface of ``Qwen35MoeModel`` (``new_state`` /
``forward(ids, state, pos0, embeds, positions3, deepstack)``), so the dense-state engine
and ``Qwen35Multimodal`` drive it unchanged.

Hugging Face names (``Qwen3VLForConditionalGeneration``, ``Qwen3VLMoeForConditionalGeneration``): ``model.language_model.*``,
``model.visual.*``, ``lm_head.weight``.

Reference behaviour: crates/models/src/qwen3/vl.rs, crates/models/src/qwen3/positions.rs
(reference project paths).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..ops import functional as F
from ..ops import reference as R
from .qwen3_5 import LayerState, norm_mrope


@dataclass
class Qwen3VLTextConfig:
    vocab_size: int = 151936
    hidden_size: int = 4096
    intermediate_size: int = 12288
    num_hidden_layers: int = 36
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    rope_theta: float = 5e6
    rms_norm_eps: float = 1e-6
    mrope_section: tuple = (24, 20, 20)
    eos_token_id: int = 151645
    image_token_id: int = 151655
    video_token_id: int = 151656
    tie_word_embeddings: bool = False
    num_experts: int = 0                 # > 0: Qwen3-VL-MoE (experts in every sparse layer)
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 768
    decoder_sparse_step: int = 1
    mlp_only_layers: tuple = ()

    def is_moe_layer(self, i: int) -> bool:
        return (self.num_experts > 0 and i not in self.mlp_only_layers
                and (i + 1) % self.decoder_sparse_step == 0)

    @classmethod
    def from_hf(cls, d: dict) -> "Qwen3VLTextConfig":
        outer, d = d, d.get("text_config", d)
        rp = d.get("rope_parameters") or d.get("rope_scaling") or {}
        kw = {k: v for k, v in d.items() if k in cls.__dataclass_fields__ and v is not None}
        kw["rope_theta"] = float(rp.get("rope_theta", d.get("rope_theta", 5e6)))
        kw["mrope_section"] = tuple(rp.get("mrope_section", (24, 20, 20)))
        kw.setdefault("head_dim", d["hidden_size"] // d["num_attention_heads"])
        kw["mlp_only_layers"] = tuple(kw.get("mlp_only_layers") or ())
        if not kw.get("num_experts") and d.get("num_local_experts"):    # newer config key
            kw["num_experts"] = int(d["num_local_experts"])
        for k in ("image_token_id", "video_token_id", "tie_word_embeddings"):
            if outer.get(k) is not None:
                kw[k] = outer[k]
        if isinstance(kw.get("eos_token_id"), (list, tuple)):
            kw["eos_token_id"] = int(kw["eos_token_id"][0])
        return cls(**kw)


class Qwen3VLDenseModel:
    def __init__(self, cfg: Qwen3VLTextConfig, device="cpu", dtype=torch.bfloat16):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.rot = cfg.head_dim
        self.inv_freq = R.rope_inv_freq(self.rot, cfg.rope_theta, self.device)
        self.w: dict = {}

    def load_state(self, loader) -> "Qwen3VLDenseModel":
        c, w = self.cfg, self.w
        names = set(loader.names())
        prefix = "model.language_model." if any(n.startswith("model.language_model.")
                                                for n in names) else "model."

        def get(n, dtype=None):
            return loader.get(n).to(device=self.device, dtype=dtype or self.dtype)
        w["embed"] = get(prefix + "embed_tokens.weight")
        w["norm"] = get(prefix + "norm.weight", torch.float32)
        w["lm_head"] = get("lm_head.weight") if "lm_head.weight" in names else w["embed"]
        for i in range(c.num_hidden_layers):
            p, a = f"{prefix}layers.{i}.", f"{prefix}layers.{i}.self_attn."
            w[i] = {"in_norm": get(p + "input_layernorm.weight", torch.float32),
                    "post_norm": get(p + "post_attention_layernorm.weight", torch.float32),
                    "qkv": torch.cat([get(a + f"{n}_proj.weight") for n in "qkv"], 0),
                    "o": get(a + "o_proj.weight"),
                    "q_norm": get(a + "q_norm.weight", torch.float32),
                    "k_norm": get(a + "k_norm.weight", torch.float32)}
            if c.is_moe_layer(i):
                I = c.moe_intermediate_size
                gu = get(p + "mlp.experts.gate_up_proj")             # [E, 2I, H]: gate, then up
                w[i]["router"] = get(p + "mlp.gate.weight")
                w[i]["w13"] = torch.cat([gu[:, I:], gu[:, :I]], 1).contiguous()
                w[i]["w2"] = get(p + "mlp.experts.down_proj").contiguous()
            else:
                w[i]["w13"] = torch.cat([get(p + "mlp.up_proj.weight"),
                                         get(p + "mlp.gate_proj.weight")], 0)
                w[i]["w2"] = get(p + "mlp.down_proj.weight")
        return self

    def new_state(self) -> list:
        return [LayerState() for _ in range(self.cfg.num_hidden_layers)]

    def _attention(self, L, n, st: LayerState, pos3):
        c, D = self.cfg, self.cfg.head_dim
        T, Hq, Hkv = n.shape[0], c.num_attention_heads, c.num_key_value_heads
        qkv = F.linear(n, L["qkv"]).view(T, Hq + 2 * Hkv, D)
        q = norm_mrope(qkv[:, :Hq], L["q_norm"], pos3, self.inv_freq, self.rot, c.mrope_section,
                       c.rms_norm_eps)
        k = norm_mrope(qkv[:, Hq:Hq + Hkv], L["k_norm"], pos3, self.inv_freq, self.rot,
                       c.mrope_section, c.rms_norm_eps)
        v = qkv[:, Hq + Hkv:]
        st.k = k if st.k is None else torch.cat([st.k, k], 0)
        st.v = v if st.v is None else torch.cat([st.v, v], 0)
        from ..ops.attention import cached_causal_attention
        att = cached_causal_attention(q, st.k, st.v, 1.0 / math.sqrt(D)) \
            .reshape(T, Hq * D).to(n.dtype)
        return F.linear(att, L["o"])

    def forward(self, ids: torch.Tensor, state: list, pos0: int = 0, embeds=None,
                positions3=None, deepstack=None) -> torch.Tensor:
        """``deepstack``: (row indices of the image positions inside this call, list of
        [n, hidden] rows) - rows k are added after layer k."""
        c, w = self.cfg, self.w
        x = w["embed"][ids.to(self.device).long()] if embeds is None else \
            embeds.to(device=self.device, dtype=self.dtype)
        T = x.shape[0]
        if positions3 is None:
            positions3 = torch.arange(pos0, pos0 + T)[None].expand(3, -1)
        for i in range(c.num_hidden_layers):
            L = w[i]
            x = x + self._attention(L, R.rmsnorm(x, L["in_norm"], c.rms_norm_eps), state[i],
                                    positions3)
            n = R.rmsnorm(x, L["post_norm"], c.rms_norm_eps)
            if "router" in L:
                logits = F.linear(n, L["router"], out_dtype=torch.float32)
                ids_, wts = F.topk_softmax(logits, c.num_experts_per_tok, True)
                x = x + F.moe_experts(n, ids_, wts, L["w13"], L["w2"])
            else:
                x = x + F.linear(F.linear_gated(n, L["w13"]), L["w2"])
            if deepstack is not None and i < len(deepstack[1]) and deepstack[0].numel():
                x = x.clone()
                x[deepstack[0]] += deepstack[1][i].to(x.dtype)
        return F.linear(R.rmsnorm(x, w["norm"], c.rms_norm_eps), w["lm_head"],
                        out_dtype=torch.float32)
