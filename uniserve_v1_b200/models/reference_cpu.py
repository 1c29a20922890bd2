"""Independent FP32 CPU implementation of the Qwen3-MoE decoder.

It shares no code with the fused operators: plain ``torch`` matmuls, a
contiguous KV cache, a Python loop over experts.  It is the numerics gate for
the engine (tiny shape: 2 layers, hidden 256, 4 q / 2 kv heads x 64, 8 experts
top-2, vocab 1024, greedy decode of 16 tokens from 32 random prompt ids) in the
way the reference checks its Rust model against a transformers forward
(crates/models/python/src/model_fixtures/qwen3.py:180-196, reference project
path).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


class ReferenceQwen3Moe:
    def __init__(self, model):
        """Takes the (unsharded) weights of a ``Qwen3MoeModel`` as FP32 copies."""
        self.cfg = model.cfg
        self.m = model
        f = lambda t: None if t is None else t.detach().float().cpu()
        self.embed = f(model.embed)
        self.final_norm = f(model.final_norm)
        self.lm_head = f(model.lm_head)
        self.layers = [{k: f(getattr(lw, k)) for k in
                        ("input_norm", "post_norm", "qkv", "q_norm", "k_norm", "o_proj",
                         "router", "w13", "w2")} | {"dense": lw.dense} for lw in model.layers]

    @staticmethod
    def _norm(x, w, eps):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w

    def _rope(self, x, pos):
        D = x.shape[-1]
        inv = 1.0 / (self.cfg.rope_theta ** (torch.arange(0, D, 2).float() / D))
        ang = pos.float()[:, None] * inv[None]
        cos, sin = ang.cos()[:, None], ang.sin()[:, None]
        x1, x2 = x[..., :D // 2], x[..., D // 2:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

    def forward(self, ids: torch.Tensor, past=None):
        """ids [T] for ONE sequence appended after ``past``; returns (logits [T,V], past)."""
        cfg = self.cfg
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        T = ids.shape[0]
        start = 0 if past is None else past[0][0].shape[0]
        pos = torch.arange(start, start + T)
        h = self.embed[ids.long()]
        new_past = []
        for li, lw in enumerate(self.layers):
            x = self._norm(h, lw["input_norm"], cfg.rms_norm_eps)
            qkv = x @ lw["qkv"].t()
            q = qkv[:, :Hq * D].view(T, Hq, D)
            k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
            v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
            if lw["q_norm"] is not None:
                q = self._norm(q, lw["q_norm"], cfg.rms_norm_eps)
                k = self._norm(k, lw["k_norm"], cfg.rms_norm_eps)
            q, k = self._rope(q, pos), self._rope(k, pos)
            if past is not None:
                k = torch.cat([past[li][0], k], 0)
                v = torch.cat([past[li][1], v], 0)
            new_past.append((k, v))
            G = Hq // Hkv
            kk = k.repeat_interleave(G, 1)
            vv = v.repeat_interleave(G, 1)
            s = torch.einsum("qhd,khd->hqk", q, kk) / math.sqrt(D)
            qi = pos[:, None]
            ki = torch.arange(k.shape[0])[None]
            s = s.masked_fill(ki > qi, float("-inf"))
            a = torch.einsum("hqk,khd->qhd", s.softmax(-1), vv).reshape(T, Hq * D)
            h = h + a @ lw["o_proj"].t()
            x = self._norm(h, lw["post_norm"], cfg.rms_norm_eps)
            if lw["dense"]:
                y = x @ lw["w13"][0].t()
                I = y.shape[1] // 2
                h = h + (y[:, :I] * F.silu(y[:, I:])) @ lw["w2"][0].t()
                continue
            p = (x @ lw["router"].t()).softmax(-1)
            w, e = torch.topk(p, cfg.num_experts_per_tok, dim=-1)
            if cfg.norm_topk_prob:
                w = w / w.sum(-1, keepdim=True)
            out = torch.zeros_like(h)
            I = cfg.moe_intermediate_size
            for t in range(T):
                for j in range(cfg.num_experts_per_tok):
                    ei = int(e[t, j])
                    y = lw["w13"][ei] @ x[t]
                    out[t] += w[t, j] * (lw["w2"][ei] @ (y[:I] * F.silu(y[I:])))
            h = h + out
        h = self._norm(h, self.final_norm, cfg.rms_norm_eps)
        return h @ self.lm_head.t(), new_past

    def greedy(self, prompt: torch.Tensor, max_new: int):
        logits, past = self.forward(prompt)
        out = []
        tok = int(logits[-1].argmax())
        out.append(tok)
        for _ in range(max_new - 1):
            logits, past = self.forward(torch.tensor([tok]), past)
            tok = int(logits[-1].argmax())
            out.append(tok)
        return out
