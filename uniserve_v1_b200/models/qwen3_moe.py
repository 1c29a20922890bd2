"""Qwen3 / Qwen3-MoE decoder (vLLM residual form) over the fused operators.

Layer (reference: crates/models/src/qwen3/decoder.rs:1-24, :242-361, reference
project path)::

    x, residual = add_rmsnorm(hidden, residual)           # FP32 residual stream
    mixed       = attention(x)                            # QKV GEMM -> q/k norm + rope + kv write
                                                          #  -> paged / varlen attention -> o_proj
    x, residual = add_rmsnorm(mixed, residual)
    hidden      = experts(x)  |  mlp(x)                   # router -> top-k -> grouped FC1/FC2

Weights are fused at load time: ``qkv`` stacks q, k, v rows; ``w13`` stacks each
expert's up rows *before* its gate rows ([E, 2I, H]); ``w2`` is [E, H, I].

Parallel layouts (crates/nn/src/modules/linear.rs:27-41, moe.rs:50-55, reference
paths): attention heads and the dense MLP are split column/row-wise over the
tensor group; with ``expert_parallel`` every rank of the group holds E/P whole
experts, runs all rows, foreign routes contribute zero and the group all-reduce
sums the partial outputs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch

from ..ops import functional as F
from ..ops import reference as R
from ..parallel.context import ParallelContext


@dataclass
class Qwen3MoeConfig:
    vocab_size: int = 151936
    hidden_size: int = 2048
    num_hidden_layers: int = 48
    num_attention_heads: int = 32
    num_key_value_heads: int = 4
    head_dim: int = 128
    rope_theta: float = 1e6
    rms_norm_eps: float = 1e-6
    num_experts: int = 128
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 768
    intermediate_size: int = 6144          # dense MLP layers (mlp_only_layers)
    norm_topk_prob: bool = True
    mlp_only_layers: tuple = ()
    decoder_sparse_step: int = 1
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 40960
    sliding_window: int = 0
    eos_token_id: int = 151645
    architectures: tuple = ("Qwen3MoeForCausalLM",)

    @classmethod
    def from_hf(cls, d: dict) -> "Qwen3MoeConfig":
        keys = {f for f in cls.__dataclass_fields__}
        d = dict(d)
        # newer transformers write `num_local_experts` and nest the rotary base
        if "num_experts" not in d and d.get("num_local_experts"):
            d["num_experts"] = d["num_local_experts"]
        if "rope_theta" not in d and isinstance(d.get("rope_parameters"), dict):
            d["rope_theta"] = d["rope_parameters"].get("rope_theta", 10000.0)
        kw = {k: v for k, v in d.items() if k in keys}
        if "head_dim" not in kw:
            kw["head_dim"] = d["hidden_size"] // d["num_attention_heads"]
        for k in ("mlp_only_layers", "architectures"):
            if k in kw and kw[k] is not None:
                kw[k] = tuple(kw[k])
        if kw.get("sliding_window") is None:
            kw["sliding_window"] = 0
        if isinstance(kw.get("eos_token_id"), list):
            kw["eos_token_id"] = kw["eos_token_id"][0]
        if "num_experts" not in d:          # dense Qwen3
            kw["num_experts"] = 0
        return cls(**kw)

    def is_moe_layer(self, i: int) -> bool:
        return (self.num_experts > 0 and i not in self.mlp_only_layers
                and (i + 1) % self.decoder_sparse_step == 0)

    # Named shapes -----------------------------------------------------------
    @classmethod
    def tiny(cls) -> "Qwen3MoeConfig":
        """2 layers, hidden 256, 4 q / 2 kv heads x 64, 8 experts top-2, inter 128, vocab 1024."""
        return cls(vocab_size=1024, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=64, num_experts=8, num_experts_per_tok=2,
                   moe_intermediate_size=128, intermediate_size=512, eos_token_id=1023,
                   max_position_embeddings=4096)

    @classmethod
    def qwen3_30b_a3b(cls) -> "Qwen3MoeConfig":
        return cls()

    @classmethod
    def qwen3_235b_a22b(cls) -> "Qwen3MoeConfig":
        return cls(hidden_size=4096, num_hidden_layers=94, num_attention_heads=64,
                   num_key_value_heads=4, head_dim=128, num_experts=128, num_experts_per_tok=8,
                   moe_intermediate_size=1536, intermediate_size=12288)


import os as _os

# Routing and route sort in one launch by one CTA: measured 8 us per layer slower than the
# two kernels at 64 tokens (one CTA routes every token), so it is opt-in.
FUSED_ROUTE_SORT = _os.environ.get("US_ROUTE_SORT", "0") == "1"
# Routing, route sort and row gather in one launch over many CTAs (decode-size batches):
# its two grid-wide waits cost more than the two launches they save behind programmatic
# dependent launch (measured +5 us per layer at 64 tokens), so it is opt-in (US_ROUTE_FUSED=1).
# The weighted un-permute is folded into the norm (or the fused all-reduce) that follows the
# experts; US_UNPERMUTE_FUSED=0 is the A/B switch.
FUSED_ROUTE_GATHER = _os.environ.get("US_ROUTE_FUSED", "0") == "1"
FUSED_UNPERMUTE = _os.environ.get("US_UNPERMUTE_FUSED", "1") == "1"
# Tensor-parallel prefill above this many rows takes the fused reduce-scatter / all-gather path
# when a FusedTP heap is attached (US_TP_FUSED=0: library all-reduce instead).
TP_FUSED_MIN_ROWS = 256 if _os.environ.get("US_TP_FUSED", "1") == "1" else 1 << 30


@dataclass
class LayerWeights:
    input_norm: torch.Tensor
    post_norm: torch.Tensor
    qkv: torch.Tensor            # [(Hq_l + 2 Hkv_l) * D, H]
    q_norm: Optional[torch.Tensor]
    k_norm: Optional[torch.Tensor]
    o_proj: torch.Tensor         # [H, Hq_l * D]
    router: Optional[torch.Tensor] = None   # [E, H]
    w13: Optional[torch.Tensor] = None      # [E_l, 2I, H] (or [1, 2I_l, H] dense MLP)
    w2: Optional[torch.Tensor] = None       # [E_l, H, I]
    fp8: Optional[object] = None            # ops.fp8.Fp8Experts replacing w13 / w2
    dense: bool = False


@dataclass
class AttnMeta:
    """What attention needs besides q/k/v.  ``decode``: one row per sequence."""
    kind: str                                   # "decode" | "prefill"
    slots: torch.Tensor                         # [T] int32 cache slot per row, -1 skips
    page_table: Optional[torch.Tensor] = None   # [B, max_pages] int32
    seq_lens: Optional[torch.Tensor] = None     # [B] int32 keys to attend (incl. this step)
    splits: int = 1
    scratch: Optional[torch.Tensor] = None
    counters: Optional[torch.Tensor] = None     # arrival counters: splits merged in-kernel
    cu_q: Optional[torch.Tensor] = None         # [n+1] int32
    cu_k: Optional[torch.Tensor] = None
    max_q: int = 0
    max_k: int = 0
    context_lens: Optional[list] = None         # per sequence keys already in the cache
    logits_rows: Optional[torch.Tensor] = None  # rows whose logits are needed (int32)
    live: Optional[torch.Tensor] = None         # device word: rows that are real (padding after)
    rows_real: Optional[int] = None             # prefill padded to a capacity: rows before the padding
    ctx_tables: Optional[tuple] = None          # ops.attention.context_tables(...) when sequences
                                                # have cached context (GPU: no host sync in prefill)


class Qwen3MoeModel:
    def __init__(self, cfg: Qwen3MoeConfig, device="cpu", dtype=torch.bfloat16,
                 ctx: Optional[ParallelContext] = None, expert_quant: Optional[str] = None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype
        assert expert_quant in (None, "fp8_block")
        self.expert_quant = expert_quant
        self.kv_dtype = None            # "fp8": E4M3 pages with per-page scales (set before the
                                        # engine allocates the cache)
        self.ctx = ctx or ParallelContext.single()
        tp = self.ctx.tp_size
        self.Hq = cfg.num_attention_heads // tp
        assert cfg.num_attention_heads % tp == 0
        # KV heads are replicated when the tensor group is wider than their count.
        self.Hkv = max(1, cfg.num_key_value_heads // tp)
        self.kv_rep = max(1, tp // cfg.num_key_value_heads)
        self.D = cfg.head_dim
        self.E_local = cfg.num_experts // self.ctx.ep_size if cfg.num_experts else 0
        self.e_lo = self.E_local * self.ctx.ep_rank
        # Exchange layout (data-parallel attention + expert parallelism, or attention-FFN
        # disaggregation): experts live whole on the expert ranks, attention is not split.
        self.expert_ranks = getattr(self.ctx, "expert_ranks", None)
        self.source_ranks = getattr(self.ctx, "source_ranks", None)
        self.exchange = None
        self.micro_exchanges: list = []  # two exchanges: decode steps as interleaved half-batches
        self.microbatch_now = False      # set per agreed step (every member decides alike)
        self.tp_fused = None            # parallel.tp_fused.FusedTP: prefill with fused collectives
        self.weight_peers = None        # parallel.dwdp: experts read from the peers' shards
        self.moe_layer_order: list = []
        if self.expert_ranks is not None:
            r = self.ctx.world_rank
            n = len(self.expert_ranks)
            self.E_local = cfg.num_experts // n if r in self.expert_ranks else 0
            self.e_lo = (r - self.expert_ranks[0]) * (cfg.num_experts // n) \
                if r in self.expert_ranks else 0
        self.is_source = self.source_ranks is None or self.ctx.world_rank in self.source_ranks
        self.inv_freq = R.rope_inv_freq(self.D, cfg.rope_theta, self.device)
        self.scale = 1.0 / math.sqrt(self.D)
        self.layers: list[LayerWeights] = []
        # Pipeline stages: contiguous shares of the layers along the "layer" axis; layers
        # of other stages are kept as None (their KV caches too).
        ax = self.ctx.axis("layer")
        self.pp, self.pp_rank, self.pp_axis = ax.size, ax.rank, ax
        L = cfg.num_hidden_layers
        per = (L + self.pp - 1) // self.pp
        self.layer_lo, self.layer_hi = min(L, self.pp_rank * per), min(L, (self.pp_rank + 1) * per)
        self.embed: Optional[torch.Tensor] = None
        self.final_norm: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None
        self.vocab_lo = 0
        self.vocab_hi = cfg.vocab_size
        self._moe_ws: dict = {}
        # expert load: per routed layer an [experts] int64 counter of the tokens each expert
        # took, added to by every forward while it is lent (None: nothing is counted)
        self.expert_load: Optional[dict] = None

    # ------------------------------------------------------------- weights --
    def init_random(self, seed: int = 0, std: float = 0.02) -> "Qwen3MoeModel":
        """Random N(0, std) weights of the architecture, generated per tensor on
        the target device.  Every rank draws the full tensor from the same
        generator state and keeps its shard, so a sharded model equals the
        unsharded one."""
        cfg, dev, dt = self.cfg, self.device, self.dtype
        g = torch.Generator(device=dev)
        g.manual_seed(seed)
        tp, tr = self.ctx.tp_size, self.ctx.tp_rank

        def rnd(*shape):
            return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * std).to(dt)

        def ones(n):
            return torch.ones(n, device=dev, dtype=dt)

        H, D = cfg.hidden_size, self.D
        self.embed = rnd(cfg.vocab_size, H)
        for i in range(cfg.num_hidden_layers):
            q = rnd(cfg.num_attention_heads * D, H)
            k = rnd(cfg.num_key_value_heads * D, H)
            v = rnd(cfg.num_key_value_heads * D, H)
            o = rnd(H, cfg.num_attention_heads * D)
            lw = LayerWeights(input_norm=ones(H), post_norm=ones(H),
                              qkv=self._shard_qkv(q, k, v), q_norm=ones(D), k_norm=ones(D),
                              o_proj=o[:, tr * self.Hq * D:(tr + 1) * self.Hq * D].contiguous())
            if cfg.is_moe_layer(i):
                lw.router = rnd(cfg.num_experts, H)
                I = cfg.moe_intermediate_size
                w13 = torch.empty(self.E_local, 2 * I, H, device=dev, dtype=dt)
                w2 = torch.empty(self.E_local, H, I, device=dev, dtype=dt)
                for e in range(cfg.num_experts):
                    gate, up, down = rnd(I, H), rnd(I, H), rnd(H, I)
                    if self.e_lo <= e < self.e_lo + self.E_local:
                        w13[e - self.e_lo, :I] = up
                        w13[e - self.e_lo, I:] = gate
                        w2[e - self.e_lo] = down
                lw.w13, lw.w2 = w13, w2
                self._quantize_experts(lw)
            else:
                I = cfg.intermediate_size
                gate, up, down = rnd(I, H), rnd(I, H), rnd(H, I)
                Il = I // tp
                sl = slice(tr * Il, (tr + 1) * Il)
                lw.w13 = torch.cat([up[sl], gate[sl]], 0).unsqueeze(0).contiguous()
                lw.w2 = down[:, sl].contiguous().unsqueeze(0)
                lw.dense = True
            self.layers.append(lw if self.layer_lo <= i < self.layer_hi else None)
        self.final_norm = ones(H)
        self.lm_head = self.embed if cfg.tie_word_embeddings else rnd(cfg.vocab_size, H)
        self._shard_vocab()
        return self

    def _shard_qkv(self, q, k, v):
        tr, D = self.ctx.tp_rank, self.D
        qs = q[tr * self.Hq * D:(tr + 1) * self.Hq * D]
        kv_idx = tr // self.kv_rep if self.kv_rep > 1 else tr
        ks = k[kv_idx * self.Hkv * D:(kv_idx + 1) * self.Hkv * D]
        vs = v[kv_idx * self.Hkv * D:(kv_idx + 1) * self.Hkv * D]
        return torch.cat([qs, ks, vs], 0).contiguous()

    def _shard_vocab(self):
        """LM head rows are split over the tensor group (all-gather of logits)."""
        tp, tr = self.ctx.tp_size, self.ctx.tp_rank
        if tp == 1:
            return
        V = self.cfg.vocab_size
        per = (V + tp - 1) // tp
        self.vocab_lo, self.vocab_hi = tr * per, min(V, (tr + 1) * per)
        head = self.lm_head[self.vocab_lo:self.vocab_hi]
        if head.shape[0] < per:      # pad so every rank gathers equal blocks
            pad = torch.zeros(per - head.shape[0], head.shape[1], dtype=head.dtype,
                              device=head.device)
            head = torch.cat([head, pad], 0)
        self.lm_head = head.contiguous()

    def export_state(self) -> dict:
        """Hugging Face tensor names -> tensors of an unsharded model (the inverse of
        ``load_state``; per-expert names)."""
        cfg, D = self.cfg, self.D
        assert self.ctx.tp_size == 1 and self.layer_lo == 0 and self.layer_hi == cfg.num_hidden_layers
        Hq, Hkv, I = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.moe_intermediate_size
        out = {"model.embed_tokens.weight": self.embed, "model.norm.weight": self.final_norm,
               "lm_head.weight": self.lm_head}
        for i, lw in enumerate(self.layers):
            p = f"model.layers.{i}."
            out[p + "input_layernorm.weight"] = lw.input_norm
            out[p + "post_attention_layernorm.weight"] = lw.post_norm
            out[p + "self_attn.q_proj.weight"] = lw.qkv[:Hq * D]
            out[p + "self_attn.k_proj.weight"] = lw.qkv[Hq * D:(Hq + Hkv) * D]
            out[p + "self_attn.v_proj.weight"] = lw.qkv[(Hq + Hkv) * D:]
            out[p + "self_attn.o_proj.weight"] = lw.o_proj
            if lw.q_norm is not None:
                out[p + "self_attn.q_norm.weight"] = lw.q_norm
                out[p + "self_attn.k_norm.weight"] = lw.k_norm
            if cfg.is_moe_layer(i):
                out[p + "mlp.gate.weight"] = lw.router
                for e in range(cfg.num_experts):
                    out[p + f"mlp.experts.{e}.up_proj.weight"] = lw.w13[e, :I]
                    out[p + f"mlp.experts.{e}.gate_proj.weight"] = lw.w13[e, I:]
                    out[p + f"mlp.experts.{e}.down_proj.weight"] = lw.w2[e]
            else:
                J = lw.w13.shape[-2] // 2
                out[p + "mlp.up_proj.weight"] = lw.w13[..., :J, :].reshape(J, -1)
                out[p + "mlp.gate_proj.weight"] = lw.w13[..., J:, :].reshape(J, -1)
                out[p + "mlp.down_proj.weight"] = lw.w2.reshape(lw.w2.shape[-2], lw.w2.shape[-1])
        return {k: v.detach().contiguous() for k, v in out.items()}

    def load_state(self, loader) -> "Qwen3MoeModel":
        """Loads Hugging Face tensor names through ``loader.get(name)``."""
        cfg, dev, dt, D = self.cfg, self.device, self.dtype, self.D
        tp, tr = self.ctx.tp_size, self.ctx.tp_rank

        def get(name):
            return loader.get(name).to(device=dev, dtype=dt)

        self.embed = get("model.embed_tokens.weight")
        for i in range(cfg.num_hidden_layers):
            if not (self.layer_lo <= i < self.layer_hi):     # another pipeline stage's layer
                self.layers.append(None)
                continue
            p = f"model.layers.{i}."
            q, k, v = (get(p + f"self_attn.{n}_proj.weight") for n in "qkv")
            o = get(p + "self_attn.o_proj.weight")
            lw = LayerWeights(
                input_norm=get(p + "input_layernorm.weight"),
                post_norm=get(p + "post_attention_layernorm.weight"),
                qkv=self._shard_qkv(q, k, v),
                q_norm=get(p + "self_attn.q_norm.weight") if loader.has(p + "self_attn.q_norm.weight") else None,
                k_norm=get(p + "self_attn.k_norm.weight") if loader.has(p + "self_attn.k_norm.weight") else None,
                o_proj=o[:, tr * self.Hq * D:(tr + 1) * self.Hq * D].contiguous())
            if cfg.is_moe_layer(i):
                lw.router = get(p + "mlp.gate.weight")
                I = cfg.moe_intermediate_size
                w13 = torch.empty(self.E_local, 2 * I, cfg.hidden_size, device=dev, dtype=dt)
                w2 = torch.empty(self.E_local, cfg.hidden_size, I, device=dev, dtype=dt)
                if loader.has(p + "mlp.experts.gate_up_proj"):
                    # stacked form: [E, 2I, H] gate rows then up rows; [E, H, I]
                    gu = get(p + "mlp.experts.gate_up_proj")[self.e_lo:self.e_lo + self.E_local]
                    w13[:, :I] = gu[:, I:]
                    w13[:, I:] = gu[:, :I]
                    w2.copy_(get(p + "mlp.experts.down_proj")[self.e_lo:self.e_lo + self.E_local])
                else:
                    for e in range(self.e_lo, self.e_lo + self.E_local):
                        pe = p + f"mlp.experts.{e}."
                        w13[e - self.e_lo, :I] = get(pe + "up_proj.weight")
                        w13[e - self.e_lo, I:] = get(pe + "gate_proj.weight")
                        w2[e - self.e_lo] = get(pe + "down_proj.weight")
                lw.w13, lw.w2 = w13, w2
                self._quantize_experts(lw)
            else:
                gate, up, down = (get(p + f"mlp.{n}_proj.weight") for n in ("gate", "up", "down"))
                Il = gate.shape[0] // tp
                sl = slice(tr * Il, (tr + 1) * Il)
                lw.w13 = torch.cat([up[sl], gate[sl]], 0).unsqueeze(0).contiguous()
                lw.w2 = down[:, sl].contiguous().unsqueeze(0)
                lw.dense = True
            self.layers.append(lw)
        self.final_norm = get("model.norm.weight")
        self.lm_head = (self.embed if cfg.tie_word_embeddings or not loader.has("lm_head.weight")
                        else get("lm_head.weight"))
        self._shard_vocab()
        return self

    # -------------------------------------------------------------- forward --
    def _fused(self, T: int, on_cuda: bool):
        """The peer-memory path serves small row counts (decode); larger batches
        take the library collective."""
        fc = self.ctx.fused
        if fc is not None and on_cuda and self.ctx.tp_size > 1 and self.pp == 1 and \
                fc.fits(T, self.cfg.hidden_size):
            return fc
        return None

    def _reduce_norm(self, fc, h, pending, residual, w):
        """residual += sum over ranks of h;  returns (rmsnorm(residual) * w, residual).
        ``pending`` says what is still owed to ``h``: nothing (None), the tensor group's sum
        ("sum": push-form all-reduce, residual add and norm in one kernel), the expert
        exchange's combine ("ep"), or the weighted un-permute of the local expert rows
        ("routed": folded into the norm kernel, or into the fused all-reduce when the
        experts are spread over the group)."""
        eps = self.cfg.rms_norm_eps
        if pending is None:
            return F.add_rmsnorm(h, residual, w, eps)
        kind = pending[0]
        if kind == "ep":            # pending expert-parallel combine
            return self.exchange.combine_add_rmsnorm(pending[1], getattr(self, "_live", None),
                                                     residual, w, eps)
        if kind == "routed":
            _, y_perm, perm, weights, reduce = pending
            if reduce:
                return fc.allreduce_add_rmsnorm(None, residual, w, eps,
                                                routed=(y_perm, perm, weights))
            return F.unpermute_add_rmsnorm(y_perm, perm, weights, residual, w, eps)
        return fc.allreduce_add_rmsnorm(h, residual, w, eps)

    def _attention(self, fc, lw: LayerWeights, x, positions, meta: AttnMeta, kcache, vcache,
                   project: bool = True):
        """``project=False`` returns the heads' output [T, Hq_l * D] before the output
        projection (the caller runs it as a GEMM whose epilogue reduce-scatters)."""
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        T = x.shape[0]
        qkv = F.linear(x, lw.qkv)
        k_scale = getattr(kcache, "page_scale", None)      # E4M3 pages: one scale per page
        v_scale = getattr(vcache, "page_scale", None)
        if k_scale is None:
            F.qk_norm_rope_kv_(qkv, lw.q_norm, lw.k_norm, positions, self.inv_freq, meta.slots,
                               kcache, vcache, Hq, Hkv, D, eps=self.cfg.rms_norm_eps)
        else:
            # norm + rotary in place, then the scaled page write derives the pages' scales
            F.qk_norm_rope_kv_(qkv, lw.q_norm, lw.k_norm, positions, self.inv_freq, None,
                               None, None, Hq, Hkv, D, eps=self.cfg.rms_norm_eps)
            v3 = qkv.view(T, Hq + 2 * Hkv, D)
            F.kv_write_scaled(v3[:, Hq:Hq + Hkv], v3[:, Hq + Hkv:], meta.slots, kcache, vcache,
                              k_scale, v_scale)
        if meta.kind == "decode":
            q = qkv[:, :Hq * D] if qkv.is_cuda else qkv[:, :Hq * D].reshape(T, Hq, D)
            att = F.paged_decode_attention(q, kcache, vcache, meta.page_table, meta.seq_lens,
                                           self.scale, meta.splits, self.cfg.sliding_window,
                                           scratch=meta.scratch, Hq=Hq, D=D,
                                           counters=meta.counters, k_scale=k_scale,
                                           v_scale=v_scale)
        else:
            from ..ops.attention import prefill_attention
            att = prefill_attention(qkv, Hq, Hkv, D, meta, kcache, vcache, self.scale)
        if not project:
            return att.reshape(T, Hq * D), None
        out = F.linear(att.reshape(T, Hq * D), lw.o_proj)
        if fc is not None:
            return out, ("sum",)
        return self.ctx.all_reduce_tp(out), None

    def _quantize_experts(self, lw: LayerWeights) -> None:
        """``expert_quant == "fp8_block"``: the stacked expert weights are replaced by
        E4M3 bytes with one FP32 scale per 128 x 128 block."""
        if self.expert_quant != "fp8_block" or lw.w13 is None or lw.w13.shape[0] == 0:
            return
        from ..ops.fp8 import Fp8Experts
        lw.fp8 = Fp8Experts.from_bf16(lw.w13, lw.w2)
        lw.w13 = lw.w2 = None

    def _mlp(self, fc, lw: LayerWeights, x, defer: bool = True, reduce_out: bool = True):
        """Returns (hidden, pending); see ``_reduce_norm``.  ``defer=False`` returns finished
        rows (no pending un-permute) for callers that use them without a norm;
        ``reduce_out=False`` returns this rank's partial sum (the caller reduce-scatters it)."""
        cfg = self.cfg
        T = x.shape[0]
        if lw.dense:
            h = F.linear_gated(x, lw.w13[0])
            if not reduce_out:
                return h, ("down", lw.w2[0])       # the caller's GEMM reduce-scatters
            out = F.linear(h, lw.w2[0])
            if fc is not None:
                return out, ("sum",)
            return self.ctx.all_reduce_tp(out), None
        logits = F.linear(x, lw.router, out_dtype=torch.float32)
        if self.exchange is not None and (x.is_cuda or getattr(self.exchange, "host", False)):
            live = getattr(self, "_live", None)
            ids, weights = F.topk_softmax(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob,
                                          live=live)
            self._count_experts(lw, ids, live)
            self.exchange.dispatch(x, ids, weights, live)
            if self.exchange.is_expert:
                if lw.fp8 is not None:
                    self.exchange.experts_fp8(lw.fp8, T)
                else:
                    self.exchange.experts(lw.w13, lw.w2, T)
            return x, ("ep", ids)
        ws = None
        if x.is_cuda:
            key = (T, x.device)
            ws = self._moe_ws.get(key)
            if ws is None:
                ws = F.MoeWorkspace.create(T, cfg.num_experts_per_tok, self.E_local,
                                           cfg.hidden_size, cfg.moe_intermediate_size, x.device,
                                           E_total=cfg.num_experts)
                self._moe_ws[key] = ws
        # distributed weight data parallelism: every expert runs here, on weights read from the
        # peers' resident shards; tokens stay, so nothing is reduced across ranks
        peers = self.weight_peers
        w13, w2 = lw.w13, lw.w2
        if peers is not None:
            order = self.moe_layer_order
            nxt = order[(order.index(lw.index) + 1) % len(order)]
            w13, w2 = peers.layer_weights(lw.index, nxt if len(order) > 1 else None)
        reduce = self.ctx.ep_size > 1 and peers is None and reduce_out
        small = x.is_cuda and T <= 512 and lw.fp8 is None
        # decode-size batches: route, sort and gather in one launch; the un-permute rides on
        # the norm (or the fused all-reduce) that follows
        fused_route = small and FUSED_ROUTE_GATHER and self.E_local > 0
        presorted = small and FUSED_ROUTE_SORT and not fused_route
        if fused_route:
            ids, weights = F.route_sort_gather(logits, x, cfg.num_experts_per_tok,
                                               cfg.norm_topk_prob, ws, self.e_lo, self.E_local,
                                               live=getattr(self, "_live", None))
        elif presorted:
            ids, weights = F.route_and_sort(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob,
                                            ws, self.e_lo, self.E_local)
        else:
            ids, weights = F.topk_softmax(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob)
        self._count_experts(lw, ids, getattr(self, "_live", None) if fused_route else None)
        if lw.fp8 is not None:
            from ..ops.fp8 import moe_experts_fp8
            if ws is not None and ws.block_n > 64:
                ws = self._moe_ws[key] = F.MoeWorkspace.create(
                    T, cfg.num_experts_per_tok, self.E_local, cfg.hidden_size,
                    cfg.moe_intermediate_size, x.device, block_n=64)
            out = moe_experts_fp8(x, ids, weights, lw.fp8, e_lo=self.e_lo, ws=ws)
        else:
            later = defer and small and FUSED_UNPERMUTE and (fc is not None or not reduce)
            out = F.moe_experts(x, ids, weights, w13, w2, e_lo=self.e_lo, ws=ws,
                                presorted=presorted, pregathered=fused_route,
                                defer_unpermute=later)
            if peers is not None:
                peers.release(lw.index)
            if later:
                y_perm, perm = out
                return y_perm, ("routed", y_perm, perm, weights, reduce and fc is not None)
        if reduce:
            if fc is not None:
                return out, ("sum",)
            out = self.ctx.all_reduce_tp(out)
        return out, None

    def forward(self, input_ids, positions, meta: AttnMeta, kv_caches) -> torch.Tensor:
        """Returns the final-normed hidden rows [T, H] (bf16).
        ``kv_caches[layer] = (k, v)`` each [pages, page_size, Hkv_local, D]."""
        self._live = meta.live
        T = input_ids.shape[0]
        ft = self.tp_fused
        if ft is not None and meta.kind == "prefill" and input_ids.is_cuda and self.pp == 1 \
                and self.exchange is None and self.weight_peers is None and meta.rows_real is None \
                and T > TP_FUSED_MIN_ROWS and ft.padded(T, ft.P) <= ft.rows_max:
            return self._forward_tp_fused(ft, input_ids, positions, meta, kv_caches)
        if self.micro_exchanges and self.microbatch_now and meta.kind == "decode" \
                and T >= 2 and T % 2 == 0 and self.pp == 1:
            return self._forward_microbatched(input_ids, positions, meta, kv_caches)
        fc = self._fused(T, input_ids.is_cuda)
        if fc is not None:
            fc.begin_forward()
        residual, site = None, None
        if self.pp == 1 or self.pp_rank == 0:
            hidden = F.embedding(input_ids, self.embed)
        else:
            hidden, residual = self._stage_recv(T)
        for i in range(self.layer_lo, self.layer_hi):
            lw = self.layers[i]
            x, residual = self._reduce_norm(fc, hidden, site, residual, lw.input_norm)
            kc, vc = kv_caches[i]
            mixed, site = self._attention(fc, lw, x, positions, meta, kc, vc)
            x, residual = self._reduce_norm(fc, mixed, site, residual, lw.post_norm)
            hidden, site = self._mlp(fc, lw, x, defer=self.pp == 1)
        if self.pp == 1:
            x, _ = self._reduce_norm(fc, hidden, site, residual, self.final_norm)
            return x
        last = self.pp - 1
        if self.pp_rank != last:
            assert site is None      # stages reduce with plain collectives (see _fused)
            self._stage_send(hidden, residual)
            x = torch.empty(T, self.cfg.hidden_size, dtype=self.dtype, device=self.device)
        else:
            x, _ = self._reduce_norm(fc, hidden, site, residual, self.final_norm)
        # every stage samples the same tokens from the last stage's rows
        return self.ctx.broadcast(x.contiguous(), last, "layer")

    def _forward_microbatched(self, input_ids, positions, meta: AttnMeta, kv_caches):
        """A decode step of an expert union as two half-batches, each with an exchange of its
        own, interleaved layer by layer: while the experts (this rank's share, or the expert
        ranks of the disaggregated layout) work on half A of layer l, this rank runs the
        attention of half B; A's combine is waited for only when A's next layer starts.
        Expert ranks serve the two windows of a layer in the same order
        (``forward_experts_only``)."""
        import copy
        T = input_ids.shape[0]
        h = T // 2
        live = meta.live
        halves = []
        for j, (lo, hi) in enumerate(((0, h), (h, T))):
            m = copy.copy(meta)
            m.slots = meta.slots[lo:hi]
            m.page_table = meta.page_table[lo:hi] if meta.page_table is not None else None
            m.seq_lens = meta.seq_lens[lo:hi] if meta.seq_lens is not None else None
            m.live = None if live is None else (live - lo).clamp(0, hi - lo).to(torch.int32)
            halves.append({"meta": m, "ids": input_ids[lo:hi], "pos": positions[lo:hi],
                           "hidden": None, "residual": None, "site": None})
        saved, saved_live = self.exchange, getattr(self, "_live", None)
        try:
            for st in halves:
                st["hidden"] = F.embedding(st["ids"], self.embed)
            for i in range(self.layer_lo, self.layer_hi):
                lw = self.layers[i]
                kc, vc = kv_caches[i]
                for j, st in enumerate(halves):
                    self.exchange, self._live = self.micro_exchanges[j], st["meta"].live
                    x, st["residual"] = self._reduce_norm(None, st["hidden"], st["site"],
                                                          st["residual"], lw.input_norm)
                    mixed, _ = self._attention(None, lw, x, st["pos"], st["meta"], kc, vc)
                    x, st["residual"] = self._reduce_norm(None, mixed, None, st["residual"],
                                                          lw.post_norm)
                    st["hidden"], st["site"] = self._mlp(None, lw, x)
            outs = []
            for j, st in enumerate(halves):
                self.exchange, self._live = self.micro_exchanges[j], st["meta"].live
                x, _ = self._reduce_norm(None, st["hidden"], st["site"], st["residual"],
                                         self.final_norm)
                outs.append(x)
        finally:
            self.exchange, self._live = saved, saved_live
        return torch.cat(outs, 0)

    def _forward_tp_fused(self, ft, input_ids, positions, meta: AttnMeta, kv_caches):
        """Tensor-parallel prefill with the collectives inside the kernels: the residual stream
        is row-sharded (rank r owns rows [r * ro, (r + 1) * ro) in FP32), every row-parallel
        product leaves as a reduce-scatter (the output projection's GEMM epilogue, or a row
        push for the un-permuted expert output), and the slot sum + residual add + RMSNorm
        kernel stores the normalised rows into every rank's gathered buffer, so the next
        column-parallel GEMM is local.  No library collective runs in the layer loop."""
        from ..parallel.tp_fused import SITE_NORM_A, SITE_NORM_B
        cfg, eps = self.cfg, self.cfg.rms_norm_eps
        T, H = input_ids.shape[0], cfg.hidden_size
        P, r = ft.P, ft.rank
        ft.set_rows(ft.padded(T, P))
        Tp, ro = ft.rows, ft.ro

        def padded(t):                       # [T, n] -> [Tp, n], zero rows behind
            if t.shape[0] == Tp:
                return t
            out = torch.zeros(Tp, t.shape[1], dtype=t.dtype, device=t.device)
            out[:T] = t
            return out
        hidden = F.embedding(input_ids, self.embed)
        lo, hi = r * ro, min((r + 1) * ro, T)
        residual = torch.zeros(ro, H, dtype=torch.float32, device=self.device)
        if hi > lo:
            residual[:hi - lo] = hidden[lo:hi].float()
        site_in, site_out = SITE_NORM_A, SITE_NORM_B
        ft.barrier()                         # every rank has left its previous use of the sites
        xa = ft.gathered(site_in)
        xa[:T] = F.rmsnorm(hidden, self.layers[self.layer_lo].input_norm, eps)
        if Tp > T:
            xa[T:].zero_()
        for i in range(self.layer_lo, self.layer_hi):
            lw = self.layers[i]
            kc, vc = kv_caches[i]
            att, _ = self._attention(None, lw, ft.gathered(site_in)[:T], positions, meta, kc, vc,
                                     project=False)
            ft.reduce_scatter_linear(lw.o_proj, padded(att))
            ft.barrier()                     # every partial row has landed in its owner's slots
            ft.reduce_add_rmsnorm(residual, lw.post_norm, site_out, eps)
            ft.barrier()                     # every normalised row has landed everywhere
            out, pending = self._mlp(None, lw, ft.gathered(site_out)[:T], defer=False,
                                     reduce_out=False)
            if pending is not None and pending[0] == "down":
                ft.reduce_scatter_linear(pending[1], padded(out))
            else:
                ft.push_rows(padded(out))
            ft.barrier()
            nxt = self.layers[i + 1].input_norm if i + 1 < self.layer_hi else self.final_norm
            ft.reduce_add_rmsnorm(residual, nxt, site_in, eps)
            ft.barrier()
        return ft.gathered(site_in)[:T].clone()

    def encode(self, input_ids, num_layers: Optional[int] = None) -> torch.Tensor:
        """Encoder use of the decoder (text conditioning of the video family): one causal
        pass over ``input_ids`` [T] without a KV cache; returns the residual stream after
        ``num_layers`` blocks (all of them by default), FP32 [T, hidden] - what
        ``transformers`` calls ``hidden_states[num_layers]``."""
        assert self.pp == 1, "the encoder pass runs on one pipeline stage"
        ids = torch.as_tensor(input_ids, dtype=torch.int32, device=self.device)
        T = ids.shape[0]
        L = self.cfg.num_hidden_layers if num_layers is None else int(num_layers)
        i32 = torch.int32
        cu = torch.tensor([0, T], dtype=i32, device=self.device)
        meta = AttnMeta(kind="prefill", slots=torch.full((T,), -1, dtype=i32, device=self.device),
                        cu_q=cu, cu_k=cu, max_q=T, max_k=T, context_lens=[0])
        pos = torch.arange(T, dtype=i32, device=self.device)
        kc = torch.zeros(1, 16, self.Hkv, self.D, dtype=self.dtype, device=self.device)
        hidden, residual = F.embedding(ids, self.embed), None
        if L == 0:
            return hidden.float()
        for i in range(L):
            lw = self.layers[i]
            x, residual = self._reduce_norm(None, hidden, None, residual, lw.input_norm)
            mixed, _ = self._attention(None, lw, x, pos, meta, kc, kc)
            x, residual = self._reduce_norm(None, mixed, None, residual, lw.post_norm)
            hidden, _ = self._mlp(None, lw, x, defer=False)
        return residual.float() + hidden.float()

    # ------------------------------------------------------------ pipeline --
    def _stage_send(self, hidden, residual) -> None:
        """Hand-off to the next stage: the block output and the FP32 residual stream
        (point-to-point on the layer axis)."""
        import torch.distributed as dist
        nxt = self.pp_axis.ranks[self.pp_rank + 1]
        ops = [dist.P2POp(dist.isend, hidden.contiguous(), nxt, self.pp_axis.group),
               dist.P2POp(dist.isend, residual.contiguous(), nxt, self.pp_axis.group)]
        for r in dist.batch_isend_irecv(ops):
            r.wait()

    def _stage_recv(self, T: int):
        import torch.distributed as dist
        prev = self.pp_axis.ranks[self.pp_rank - 1]
        H = self.cfg.hidden_size
        hidden = torch.empty(T, H, dtype=self.dtype, device=self.device)
        residual = torch.empty(T, H, dtype=torch.float32, device=self.device)
        ops = [dist.P2POp(dist.irecv, hidden, prev, self.pp_axis.group),
               dist.P2POp(dist.irecv, residual, prev, self.pp_axis.group)]
        for r in dist.batch_isend_irecv(ops):
            r.wait()
        return hidden, residual

    def forward_experts_only(self, t_step: int, micro: bool = False) -> None:
        """An expert rank of the disaggregated layout: every forward is the join - per
        layer it waits for the attention ranks' rows, runs its experts and pushes back.
        ``micro``: the step runs as two half-batches, each through its own exchange."""
        windows = [(self.exchange, t_step)]
        if micro and self.micro_exchanges and t_step >= 2 and t_step % 2 == 0:
            windows = [(ex, t_step // 2) for ex in self.micro_exchanges]
        for lw in self.layers:
            if lw is None or lw.dense:
                continue
            for ex, t in windows:
                if lw.fp8 is not None:
                    ex.experts_fp8(lw.fp8, t)
                else:
                    ex.experts(lw.w13, lw.w2, t)
        for ex, _ in windows:               # host exchanges hold a layer's last collective back
            if hasattr(ex, "flush"):
                ex.flush()

    def greedy_tokens(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        """arg-max token of every row, int32 [rows], the same on every rank.  With a
        vocabulary-sharded head and a peer heap only (value, column) pairs cross NVLink
        (one kernel: local arg-max, push, pick); the logits are never gathered."""
        lg = F.linear(hidden_rows, self.lm_head, out_dtype=torch.float32)
        if self.ctx.tp_size > 1:
            fc = self.ctx.fused
            if fc is not None and lg.is_cuda and lg.shape[0] <= fc.max_rows:
                return fc.argmax(lg, self.vocab_hi - self.vocab_lo, self.vocab_lo)
            lg = self.ctx.all_gather_tp_cols(lg)[:, :self.cfg.vocab_size]
        return F.argmax(lg)

    def logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        """FP32 logits [rows, vocab]; vocab-sharded heads are all-gathered and un-padded."""
        lg = F.linear(hidden_rows, self.lm_head, out_dtype=torch.float32)
        if self.ctx.tp_size > 1:
            lg = self.ctx.all_gather_tp_cols(lg)[:, :self.cfg.vocab_size]
        return lg

    # ------------------------------------------------------------- caches --
    def new_kv_caches(self, num_pages: int, page_size: int = 16):
        """One (key, value) plane pair per layer this rank owns.  ``kv_dtype == "fp8"``: the
        planes hold E4M3 bytes and carry their per-page FP32 scales as ``page_scale``."""
        shape = (num_pages, page_size, self.Hkv, self.D)
        fp8 = self.kv_dtype == "fp8"

        def plane():
            t = torch.zeros(shape, dtype=torch.uint8 if fp8 else self.dtype, device=self.device)
            if fp8:
                t.page_scale = torch.zeros(num_pages, dtype=torch.float32, device=self.device)
            return t
        return [(plane(), plane()) if self.layer_lo <= i < self.layer_hi else (None, None)
                for i in range(self.cfg.num_hidden_layers)]

    # ------------------------------------------------------------ expert load --
    def enable_expert_load(self, on: bool = True) -> None:
        """Lends (or takes back) the expert load counters: one ``[experts]`` int64 tensor per
        routed layer, indexed by the model's own expert id, to which every forward adds each
        live token's routes.  On a GPU this is a few small launches per routed layer and
        forward, so a deployment counts only while something reads the counters.
        Reference behaviour: crates/ops/src/moe/load.rs (reference project path)."""
        self._load_of: dict = {}
        if not on:
            self.expert_load = None
            return
        self.expert_load = {
            i: torch.zeros(self.cfg.num_experts, dtype=torch.int64, device=self.device)
            for i, lw in enumerate(self.layers) if lw is not None and not getattr(lw, "dense", False)}
        self._load_of = {id(self.layers[i]): t for i, t in self.expert_load.items()}

    def _count_experts(self, lw, ids, live=None) -> None:
        load = self.expert_load
        if load is None or ids is None:
            return
        counter = self._load_of.get(id(lw))
        if counter is None:
            return
        flat = ids.reshape(-1).to(torch.int64)
        if live is not None:                       # rows past the live count are padding
            k = ids.shape[-1]
            rows = torch.arange(ids.shape[0], device=ids.device).repeat_interleave(k)
            ones = (rows < live.to(torch.int64)).to(torch.int64)
        else:
            ones = torch.ones_like(flat)
        counter.index_add_(0, flat.clamp_(0, counter.numel() - 1), ones)

    def expert_load_snapshot(self) -> dict:
        """{layer index: tokens per expert} read back from the device (empty when nothing is
        counted)."""
        if not self.expert_load:
            return {}
        return {i: t.tolist() for i, t in sorted(self.expert_load.items())}

    def kv_bytes_per_page(self, page_size: int = 16) -> int:
        elem = 1 if self.kv_dtype == "fp8" else 2
        per_layer = 2 * (page_size * self.Hkv * self.D * elem + (4 if elem == 1 else 0))
        return per_layer * (self.layer_hi - self.layer_lo)

    def weight_bytes(self) -> int:
        n = self.embed.numel() + self.final_norm.numel()
        if self.lm_head is not self.embed:
            n += self.lm_head.numel()
        for lw in self.layers:
            if lw is None:
                continue
            for t in (lw.input_norm, lw.post_norm, lw.qkv, lw.q_norm, lw.k_norm, lw.o_proj,
                      lw.router, lw.w13, lw.w2):
                if t is not None:
                    n += t.numel()
        return n * 2
