"""Decoders of the video pipeline: the video VAE decoder (a non-causal ViT over
latent voxels) and the audio VAE decoder (BigVGAN-style transposed-convolution
stack with anti-aliased snake activations).

Video: ``post_quant`` (per-voxel channel mix) -> ``proj_in`` (one token per latent
voxel) + register tokens -> pre-norm blocks (LayerNorm, attention with 64-wide
heads and a three-axis rotary, GELU MLP x4) -> ``proj_out`` writes 3 x 4 x 16 x 16
values per token, the voxel's pixel block.  A temporal unit is 5 latent frames ->
17 frames (the first latent frame yields one frame, the rest four each); the
2-latent-frame tail of the 17n + 5 rule yields 5 frames.  Units are independent
and are dealt round-robin over ranks ("temporal_units" distribution).

Audio: conv_pre -> for each rate in [5,5,2,2,2,2,2]: transposed conv (upsample)
then three residual blocks (kernels 3/7/11, dilations 1/3/5) with the
anti-aliased activation -> conv_post -> tanh.  32 latent channels at 40 Hz become
32 kHz samples; stereo channels ride the batch dimension.  FP32 throughout.

Reference behaviour: crates/models/src/minimax_h3/video_vae.rs:1-55, splice.rs:1-10,
audio_vae.rs:1-30, fixtures.rs:73-119 (reference project paths).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from ..ops import functional as F
from ..ops import media as M
from ..ops import reference as R
from ..ops.attention import varlen_attention


@dataclass
class VideoVaeConfig:
    latent_channels: int = 24
    width: int = 2048
    heads: int = 32
    head_dim: int = 64
    layers: int = 36
    registers: int = 4
    mlp_ratio: int = 4
    spatial: int = 16
    temporal: int = 4
    rope_theta: float = 100.0
    rope_freqs_per_axis: int = 8
    eps: float = 1e-6

    @classmethod
    def tiny(cls):
        return cls(latent_channels=4, width=128, heads=2, head_dim=64, layers=2, registers=2,
                   spatial=4, temporal=4)


class VideoVaeDecoder:
    def __init__(self, cfg: VideoVaeConfig, device="cpu", dtype=torch.bfloat16):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.inv_freq = R.rope_inv_freq(2 * cfg.rope_freqs_per_axis, cfg.rope_theta, self.device)

    def init_random(self, seed=0, std=0.02):
        c, dev, dt = self.cfg, self.device, self.dtype
        g = torch.Generator(device=dev)
        g.manual_seed(seed)
        rnd = lambda *s: (torch.randn(*s, generator=g, device=dev) * std).to(dt)
        ones = lambda n: torch.ones(n, device=dev, dtype=dt)
        zeros = lambda n: torch.zeros(n, device=dev, dtype=dt)
        W = c.width
        self.post_quant = rnd(c.latent_channels, c.latent_channels) + \
            torch.eye(c.latent_channels, device=dev, dtype=dt)
        self.proj_in = rnd(W, c.latent_channels)
        self.registers = rnd(c.registers, W)
        self.blocks = []
        for _ in range(c.layers):
            self.blocks.append(dict(n1w=ones(W), n1b=zeros(W), qkv=rnd(3 * W, W), out=rnd(W, W),
                                    n2w=ones(W), n2b=zeros(W), fc1=rnd(c.mlp_ratio * W, W),
                                    fc2=rnd(W, c.mlp_ratio * W)))
        self.norm_w, self.norm_b = ones(W), zeros(W)
        self.proj_out = rnd(3 * c.temporal * c.spatial * c.spatial, W)
        return self

    def _attention(self, q, k, v, n):
        """Dense bidirectional attention over the unit's tokens; 64- and 128-wide heads run
        the tensor-core flash kernel directly."""
        c = self.cfg
        D = c.head_dim
        cu = torch.tensor([0, n], dtype=torch.int32, device=q.device)
        scale = 1.0 / math.sqrt(D)
        if q.is_cuda and D not in (64, 128):
            pad = lambda t: torch.nn.functional.pad(t, (0, 128 - D))
            o = varlen_attention(pad(q), pad(k), pad(v), cu, cu, n, n, scale, False)
            return o[..., :D]
        return varlen_attention(q, k, v, cu, cu, n, n, scale, False)

    def decode_unit(self, latent: torch.Tensor) -> torch.Tensor:
        """latent [C, f, h, w] fp32 (f latent frames) -> frames [1 + 4 (f - 1), 3, 16h, 16w]."""
        c = self.cfg
        C, f, h, w = latent.shape
        x = latent.permute(1, 2, 3, 0).reshape(f * h * w, C).to(self.dtype)
        x = F.linear(x, self.post_quant)
        x = F.linear(x, self.proj_in)
        x = torch.cat([self.registers, x], 0).contiguous()
        n = x.shape[0]
        grid = torch.stack(torch.meshgrid(torch.arange(f), torch.arange(h), torch.arange(w),
                                          indexing="ij"), 0).reshape(3, -1).float()
        coords = torch.cat([torch.zeros(3, c.registers), grid], 1).to(x.device)
        H, D = c.heads, c.head_dim
        for b in self.blocks:
            y = F.layer_norm(x, b["n1w"], b["n1b"], c.eps)
            qkv = F.linear(y, b["qkv"])
            q, k, v = qkv[:, :H * D], qkv[:, H * D:2 * H * D], qkv[:, 2 * H * D:]
            F.qk_norm_rope3_(q, k, None, None, coords, self.inv_freq, H, H, D,
                             c.rope_freqs_per_axis, c.eps)
            a = self._attention(q.reshape(n, H, D), k.reshape(n, H, D), v.reshape(n, H, D), n)
            x = x + F.linear(a.reshape(n, H * D).contiguous(), b["out"])
            y = F.layer_norm(x, b["n2w"], b["n2b"], c.eps)
            hdn = torch.nn.functional.gelu(F.linear(y, b["fc1"]).float(), approximate="tanh")
            x = x + F.linear(hdn.to(self.dtype), b["fc2"])
        x = F.layer_norm(x, self.norm_w, self.norm_b, c.eps)[c.registers:]
        px = F.linear(x, self.proj_out).float()            # [f*h*w, 3 * 4 * S * S]
        S, T = c.spatial, c.temporal
        px = px.view(f, h, w, 3, T, S, S).permute(0, 4, 3, 1, 5, 2, 6)   # f,T,3,h,S,w,S
        frames = px.reshape(f * T, 3, h * S, w * S)
        return frames[T - 1:].contiguous()                  # first latent frame -> one frame

    def decode(self, latent: torch.Tensor, rank: int = 0, world: int = 1, unit: int = 5):
        """All temporal units this rank owns, in order: list of (unit index, frames)."""
        C, Fl, h, w = latent.shape
        units = []
        k = 0
        for f0 in range(0, Fl, unit):
            if k % world == rank:
                units.append((k, self.decode_unit(latent[:, f0:f0 + unit])))
            k += 1
        return units


@dataclass
class AudioVaeConfig:
    latent_channels: int = 32
    decoder_dim: int = 1024
    rates: tuple = (5, 5, 2, 2, 2, 2, 2)
    kernels: tuple = (9, 9, 4, 4, 4, 4, 4)
    res_kernels: tuple = (3, 7, 11)
    res_dilations: tuple = (1, 3, 5)
    sample_rate: int = 32000

    @classmethod
    def tiny(cls):
        return cls(latent_channels=8, decoder_dim=32, rates=(5, 2), kernels=(9, 4),
                   res_kernels=(3,), res_dilations=(1, 3))

    @property
    def upsample(self) -> int:
        r = 1
        for x in self.rates:
            r *= x
        return r


class AudioVaeDecoder:
    def __init__(self, cfg: AudioVaeConfig, device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        self.taps = M.kaiser_sinc_taps(12).to(self.device)

    def init_random(self, seed=0, std=0.02):
        c, dev = self.cfg, self.device
        g = torch.Generator(device=dev)
        g.manual_seed(seed)
        rnd = lambda *s: torch.randn(*s, generator=g, device=dev) * std
        zeros = lambda n: torch.zeros(n, device=dev)
        self.conv_pre = (rnd(c.decoder_dim, c.latent_channels, 7), zeros(c.decoder_dim))
        self.stages = []
        ch = c.decoder_dim
        for r, k in zip(c.rates, c.kernels):
            out = ch // 2
            st = dict(up=(rnd(ch, out, k), zeros(out)), rate=r, k=k, res=[])
            for rk in c.res_kernels:
                convs = []
                for d in c.res_dilations:
                    convs.append(dict(a1=(zeros(out), zeros(out)), c1=(rnd(out, out, rk), zeros(out)),
                                      a2=(zeros(out), zeros(out)), c2=(rnd(out, out, rk), zeros(out)),
                                      d=d, k=rk))
                st["res"].append(convs)
            self.stages.append(st)
            ch = out
        self.act_post = (zeros(ch), zeros(ch))
        self.conv_post = (rnd(1, ch, 7), zeros(1))
        return self

    def decode(self, latents: torch.Tensor) -> torch.Tensor:
        """latents [channels(batch), latent_channels, T] fp32 -> audio [channels, T * upsample]."""
        x = M.conv1d(latents.float(), *self.conv_pre, padding=3)
        for st in self.stages:
            r, k = st["rate"], st["k"]
            pad = (k - r) // 2
            x = M.conv_transpose1d(x, *st["up"], stride=r, padding=pad)
            if (k - r) % 2:                       # odd kernel surplus: trim the extra sample
                x = x[..., :x.shape[-1] - ((k - r) % 2)].contiguous()
            acc = None
            for convs in st["res"]:
                y = x
                for cv in convs:
                    t = M.activation1d(y, self.taps, *cv["a1"])
                    t = M.conv1d(t, *cv["c1"], padding=cv["d"] * (cv["k"] - 1) // 2, dilation=cv["d"])
                    t = M.activation1d(t, self.taps, *cv["a2"])
                    t = M.conv1d(t, *cv["c2"], padding=(cv["k"] - 1) // 2)
                    y = y + t
                acc = y if acc is None else acc + y
            x = acc / len(st["res"])
        x = M.activation1d(x, self.taps, *self.act_post)
        x = M.conv1d(x, *self.conv_post, padding=3)
        return torch.tanh(x)[:, 0]
