"""Qwen3-VL vision tower: patches -> vision rows for the language model.

Input is what the image processor emits: ``pixels`` [patches, C * T * P * P] (patches
ordered merge-block by merge-block) and one (t, h, w) patch grid per image or video.

    embed   linear over the flattened patch (the Conv3d with stride = kernel) + bias
    + pos   learned grid embedding, bilinearly interpolated to (h, w), merge-block order
    blocks  LayerNorm -> attention (fused QKV + bias, 2-D rotary over (row, col),
            bidirectional inside each frame) -> LayerNorm -> GELU-tanh MLP
    merger  LayerNorm -> concat of merge^2 neighbours -> MLP (GELU) -> out width
    deepstack  the same merger (norm after the concat) applied to chosen blocks'
            outputs; the language model adds those rows to its first layers' states

``splice`` puts the merged rows at the placeholder tokens of the text embedding.
Linears, norms and attention go through the package's operators (the tensor-core GEMM
and flash kernels on a GPU; 64-wide heads run the two-tile kernel).

Reference behaviour: crates/models/src/qwen3/vision.rs, crates/models/src/qwen3/vl.rs,
crates/nn/src/capability.rs (Vision, Splicer) - reference project paths.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from ..ops import functional as F
from ..ops.attention import varlen_attention


@dataclass
class VisionConfig:
    depth: int = 27
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 3584
    num_position_embeddings: int = 2304
    deepstack_visual_indexes: list = field(default_factory=lambda: [8, 16, 24])
    hidden_act: str = "gelu_pytorch_tanh"

    @classmethod
    def from_hf(cls, d: dict) -> "VisionConfig":
        d = d.get("vision_config", d)
        kw = {k: v for k, v in d.items() if k in cls.__dataclass_fields__ and v is not None}
        kw.setdefault("deepstack_visual_indexes", [])      # absent: a tower without deep stack
        return cls(**kw)


def _gelu(x, tanh: bool):
    return torch.nn.functional.gelu(x.float(), approximate="tanh" if tanh else "none").to(x.dtype)


class Qwen3VLVisionTower:
    def __init__(self, cfg: VisionConfig, device="cpu", dtype=torch.bfloat16):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.head_dim = cfg.hidden_size // cfg.num_heads
        quarter = self.head_dim // 2
        self.inv_freq = 1.0 / (10000.0 ** (torch.arange(0, quarter, 2, dtype=torch.float32,
                                                        device=self.device) / quarter))
        self.w: dict = {}

    def load_state(self, loader, prefix: str = "model.visual.") -> "Qwen3VLVisionTower":
        names = set(loader.names())
        if not any(n.startswith(prefix) for n in names):
            prefix = next((p for p in ("visual.", "") if any(n.startswith(p + "patch_embed.")
                                                              for n in names)), prefix)

        def get(n):
            return loader.get(prefix + n).to(device=self.device, dtype=self.dtype)
        c, w = self.cfg, self.w
        w["patch_w"] = get("patch_embed.proj.weight").reshape(c.hidden_size, -1).contiguous()
        w["patch_b"] = get("patch_embed.proj.bias")
        w["pos"] = get("pos_embed.weight")

        def merger(p):
            return {k: get(p + k) for k in ("norm.weight", "norm.bias", "linear_fc1.weight",
                                            "linear_fc1.bias", "linear_fc2.weight",
                                            "linear_fc2.bias")}
        for i in range(c.depth):
            b = f"blocks.{i}."
            w[i] = {k: get(b + k) for k in (
                "norm1.weight", "norm1.bias", "norm2.weight", "norm2.bias", "attn.qkv.weight",
                "attn.qkv.bias", "attn.proj.weight", "attn.proj.bias", "mlp.linear_fc1.weight",
                "mlp.linear_fc1.bias", "mlp.linear_fc2.weight", "mlp.linear_fc2.bias")}
        w["merger"] = merger("merger.")
        w["deepstack"] = [merger(f"deepstack_merger_list.{j}.")
                          for j in range(len(c.deepstack_visual_indexes))]
        return self

    # ------------------------------------------------------------ positions --
    def _block_order(self, h: int, w: int):
        """(row, col) of every patch of an h x w grid in merge-block order."""
        m = self.cfg.spatial_merge_size
        rows = torch.arange(h).view(h // m, m)[:, None, :, None].expand(h // m, w // m, m, m)
        cols = torch.arange(w).view(w // m, m)[None, :, None, :].expand(h // m, w // m, m, m)
        return rows.reshape(-1), cols.reshape(-1)

    def position_embedding(self, grids: list) -> torch.Tensor:
        side = int(math.isqrt(self.cfg.num_position_embeddings))
        pos = self.w["pos"].float()
        out = []
        for t, h, w in grids:
            ys, xs = torch.linspace(0, side - 1, h), torch.linspace(0, side - 1, w)
            y0, x0 = ys.int(), xs.int()
            y1, x1 = (y0 + 1).clip(max=side - 1), (x0 + 1).clip(max=side - 1)
            dy, dx = (ys - y0)[:, None], (xs - x0)[None, :]

            def at(yy, xx):
                return pos[(yy[:, None] * side + xx[None, :]).long().to(pos.device)]
            dy, dx = dy.to(pos.device)[..., None], dx.to(pos.device)[..., None]
            grid = at(y0, x0) * (1 - dy) * (1 - dx) + at(y0, x1) * (1 - dy) * dx + \
                at(y1, x0) * dy * (1 - dx) + at(y1, x1) * dy * dx           # [h, w, C]
            r, c_ = self._block_order(h, w)
            out.append(grid[r.to(pos.device), c_.to(pos.device)].repeat(t, 1))
        return torch.cat(out).to(self.dtype)

    def rotary(self, grids: list):
        parts = []
        for t, h, w in grids:
            r, c_ = self._block_order(h, w)
            ang = torch.cat([r.to(self.device).float()[:, None] * self.inv_freq,
                             c_.to(self.device).float()[:, None] * self.inv_freq], -1)
            parts.append(ang.repeat(t, 1))
        ang = torch.cat(parts)                                   # [N, head_dim / 2]
        emb = torch.cat([ang, ang], -1)
        return emb.cos()[:, None, :], emb.sin()[:, None, :]

    # -------------------------------------------------------------- forward --
    def _merge(self, mw, x, post_shuffle: bool):
        c = self.cfg
        wide = c.hidden_size * c.spatial_merge_size ** 2
        if post_shuffle:
            x = F.layer_norm(x.reshape(-1, wide), mw["norm.weight"], mw["norm.bias"], 1e-6)
        else:
            x = F.layer_norm(x, mw["norm.weight"], mw["norm.bias"], 1e-6).reshape(-1, wide)
        x = _gelu(F.linear(x.contiguous(), mw["linear_fc1.weight"], mw["linear_fc1.bias"]), False)
        return F.linear(x, mw["linear_fc2.weight"], mw["linear_fc2.bias"])

    def forward(self, pixels: torch.Tensor, grids: list):
        """Returns (vision rows [patches / merge^2, out width], deepstack rows list)."""
        c, w, D, H = self.cfg, self.w, self.head_dim, self.cfg.num_heads
        x = F.linear(pixels.to(device=self.device, dtype=self.dtype).contiguous(), w["patch_w"],
                     w["patch_b"])
        x = x + self.position_embedding(grids)
        cos, sin = self.rotary(grids)
        lens = [h * wd for t, h, wd in grids for _ in range(t)]
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32,
                          device=self.device)
        N_, tanh = x.shape[0], c.hidden_act == "gelu_pytorch_tanh"

        def rot(t):
            tf = t.float()
            half = D // 2
            turned = torch.cat([-tf[..., half:], tf[..., :half]], -1)
            return (tf * cos + turned * sin).to(t.dtype)
        deep = []
        for i in range(c.depth):
            b = w[i]
            n = F.layer_norm(x, b["norm1.weight"], b["norm1.bias"], 1e-6)
            qkv = F.linear(n, b["attn.qkv.weight"], b["attn.qkv.bias"]).view(N_, 3, H, D)
            q, k, v = rot(qkv[:, 0]).contiguous(), rot(qkv[:, 1]).contiguous(), \
                qkv[:, 2].contiguous()
            if q.is_cuda and D not in (64, 128):      # e.g. 72-wide heads: zero-pad to 128
                pad = lambda t_: torch.nn.functional.pad(t_, (0, 128 - D))
                att = varlen_attention(pad(q), pad(k), pad(v), cu, cu, max(lens), max(lens),
                                       D ** -0.5, False)[..., :D]
            else:
                att = varlen_attention(q, k, v, cu, cu, max(lens), max(lens), D ** -0.5, False)
            x = x + F.linear(att.reshape(N_, H * D), b["attn.proj.weight"], b["attn.proj.bias"])
            n = F.layer_norm(x, b["norm2.weight"], b["norm2.bias"], 1e-6)
            hmid = _gelu(F.linear(n, b["mlp.linear_fc1.weight"], b["mlp.linear_fc1.bias"]), tanh)
            x = x + F.linear(hmid, b["mlp.linear_fc2.weight"], b["mlp.linear_fc2.bias"])
            if i in c.deepstack_visual_indexes:
                deep.append(self._merge(w["deepstack"][c.deepstack_visual_indexes.index(i)], x,
                                        True))
        return self._merge(w["merger"], x, False), deep


def splice(embeds: torch.Tensor, input_ids: torch.Tensor, placeholder_id: int,
           vision_rows: torch.Tensor) -> torch.Tensor:
    """Text embedding rows [T, H] with the rows at ``placeholder_id`` tokens replaced, in
    order, by ``vision_rows``; the counts must agree."""
    at = (input_ids == placeholder_id).nonzero(as_tuple=True)[0]
    if at.numel() != vision_rows.shape[0]:
        raise ValueError(f"{at.numel()} placeholder tokens for {vision_rows.shape[0]} vision rows")
    out = embeds.clone()
    out[at.to(out.device)] = vision_rows.to(out.dtype)
    return out
