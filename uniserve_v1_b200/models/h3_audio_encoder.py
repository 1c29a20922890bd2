"""Audio VAE encoder: the DAC encoder that turns a reference track into its latent rows.

::

    block.0          conv 1 -> d channels, kernel 7, padding 3
    stage of stride r at width w:
        three residual units at dilations 1, 3, 9:  x += conv1x1(snake(conv7_dilated(snake(x))))
        snake;  conv w -> 2w, kernel 2r, stride r, padding ceil(r / 2)
    snake;  conv -> latent_dim, kernel 3, padding 1
    snake(x) = x + sin^2(alpha * x) / (alpha + 1e-9)        per-channel alpha

    projection (per stereo channel, frames as rows; the attention is causal over frames):
        h   = proj(norm3(x)) + attn_proj(pool(attention(qkv(norm1(x)))))
        out = mlp(norm2(h)) + h          mlp(y) = w2(gelu_tanh(w0(norm(y))) * w1(norm(y)))
    pool averages the heads and pools each head's width down to the latent channels.
    latent = (mean_proj(out) - latents_mean) / latents_std      the posterior's mean, no sample

A track of L samples is right-padded with zeros to whole hops (the product of the strides) and
gives L / hop frames per stereo channel; a mono track is two identical channels.  FP32
throughout (the values are amplitudes).  Rows come out time-major with the two channels of a
latent frame side by side, the order the denoiser's audio rows have here.

Reference behaviour: crates/nn/src/modules/codec.rs:1-19,
crates/models/src/minimax_h3/audio_vae.rs:14-22, 227-237, 444-500 (reference project paths).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as TF


@dataclass
class AudioEncoderConfig:
    channels: int = 64                       # d_model; every stage doubles it
    strides: tuple = (2, 4, 4, 5, 5)         # hop 800: 40 latent frames / s at 32 kHz
    latent_dim: int = 2048
    latent_channels: int = 32
    heads: int = 16
    sample_rate: int = 32000
    latents_mean: tuple = ()
    latents_std: tuple = ()

    @classmethod
    def tiny(cls, latent_channels: int = 8):
        return cls(channels=4, strides=(2, 4), latent_dim=32, latent_channels=latent_channels,
                   heads=2, sample_rate=320)

    @property
    def hop(self) -> int:
        return math.prod(self.strides)


def snake(x: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    a = alpha.view(1, -1, 1)
    return x + torch.sin(a * x).pow(2) / (a + 1e-9)


def padded_samples(samples: int, hop: int) -> int:
    if samples <= 0 or hop <= 0:
        raise ValueError(f"an audio track of {samples} samples in {hop}-sample latent frames "
                         "encodes to nothing")
    return (samples + hop - 1) // hop * hop


class AudioVaeEncoder:
    def __init__(self, cfg: AudioEncoderConfig, device="cpu"):
        c = cfg
        if c.latent_channels <= 0 or c.latent_dim <= c.latent_channels or \
                c.latent_dim % c.latent_channels or c.heads <= 0 or c.latent_dim % c.heads:
            raise ValueError("the audio encoder's latent channels and heads each divide its "
                             "features, which are wider than the channels")
        self.cfg, self.device, self.w = cfg, torch.device(device), {}

    def init_random(self, seed: int = 0, std: float = 0.3) -> "AudioVaeEncoder":
        c, g, w = self.cfg, torch.Generator().manual_seed(seed), self.w

        def t(name, *shape, fan=None):
            scale = std / math.sqrt(fan or shape[-1] if len(shape) > 1 else 1.0)
            w[name] = (torch.randn(*shape, generator=g) * scale).to(self.device)

        def conv(name, cin, cout, k):
            t(name + ".weight", cout, cin, k, fan=cin * k)
            w[name + ".bias"] = torch.zeros(cout, device=self.device)

        def alpha(name, ch):
            w[name] = (torch.rand(ch, generator=g) + 0.5).to(self.device)

        def lin(name, cin, cout):
            t(name + ".weight", cout, cin)
            w[name + ".bias"] = torch.zeros(cout, device=self.device)

        def norm(name, ch):
            w[name + ".weight"] = torch.ones(ch, device=self.device)
            w[name + ".bias"] = torch.zeros(ch, device=self.device)
        width = c.channels
        conv("encoder.block.0", 1, width, 7)
        for s, r in enumerate(c.strides):
            p = f"encoder.block.{s + 1}.block"
            for u in range(3):
                alpha(f"{p}.{u}.block.0.alpha", width)
                conv(f"{p}.{u}.block.1", width, width, 7)
                alpha(f"{p}.{u}.block.2.alpha", width)
                conv(f"{p}.{u}.block.3", width, width, 1)
            alpha(f"{p}.3.alpha", width)
            conv(f"{p}.4", width, 2 * width, 2 * r)
            width *= 2
        S = len(c.strides)
        alpha(f"encoder.block.{S + 1}.alpha", width)
        conv(f"encoder.block.{S + 2}", width, c.latent_dim, 3)
        D, C = c.latent_dim, c.latent_channels
        for n, ch in (("norm1", D), ("norm3", D), ("norm2", C), ("mlp.norm", C)):
            norm("pre_block." + n, ch)
        lin("pre_block.proj", D, C)
        lin("pre_block.attn.qkv", D, 3 * D)
        lin("pre_block.attn.proj", C, C)
        lin("pre_block.mlp.w0", C, 4 * C)
        lin("pre_block.mlp.w1", C, 4 * C)
        lin("pre_block.mlp.w2", 4 * C, C)
        conv("mean_proj", C, C, 1)
        return self

    # ----------------------------------------------------------------- forward --
    def features(self, samples: torch.Tensor) -> torch.Tensor:
        """samples [n, 1, L] (L whole hops) -> [n, latent_dim, L / hop]."""
        c, w = self.cfg, self.w
        cv = lambda name, x, **kw: TF.conv1d(x, w[name + ".weight"], w[name + ".bias"], **kw)
        x = cv("encoder.block.0", samples.to(self.device, torch.float32), padding=3)
        for s, r in enumerate(c.strides):
            p = f"encoder.block.{s + 1}.block"
            for u, d in enumerate((1, 3, 9)):
                y = cv(f"{p}.{u}.block.1", snake(x, w[f"{p}.{u}.block.0.alpha"]), padding=3 * d,
                       dilation=d)
                x = x + cv(f"{p}.{u}.block.3", snake(y, w[f"{p}.{u}.block.2.alpha"]))
            x = cv(f"{p}.4", snake(x, w[f"{p}.3.alpha"]), stride=r, padding=(r + 1) // 2)
        S = len(c.strides)
        return cv(f"encoder.block.{S + 2}", snake(x, w[f"encoder.block.{S + 1}.alpha"]), padding=1)

    def project(self, rows: torch.Tensor) -> torch.Tensor:
        """One channel's frames [frames, latent_dim] -> [frames, latent_channels]."""
        c, w = self.cfg, self.w
        ln = lambda n, x: TF.layer_norm(x, (x.shape[-1],), w[n + ".weight"], w[n + ".bias"], 1e-5)
        li = lambda n, x: TF.linear(x, w[n + ".weight"], w[n + ".bias"])
        T, H = rows.shape[0], c.heads
        hd = c.latent_dim // H
        q, k, v = li("pre_block.attn.qkv", ln("pre_block.norm1", rows)).view(T, 3, H, hd).unbind(1)
        a = TF.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None],
                                            v.transpose(0, 1)[None], is_causal=True)[0]
        pooled = TF.adaptive_avg_pool2d(a.permute(1, 0, 2), (1, c.latent_channels))[:, 0]
        h = li("pre_block.proj", ln("pre_block.norm3", rows)) + li("pre_block.attn.proj", pooled)
        y = ln("pre_block.mlp.norm", ln("pre_block.norm2", h))
        y = TF.gelu(li("pre_block.mlp.w0", y), approximate="tanh") * li("pre_block.mlp.w1", y)
        return li("pre_block.mlp.w2", y) + h

    def encode(self, samples: torch.Tensor) -> torch.Tensor:
        """samples [2, 1, L] FP32 (the stereo pair, L whole hops) -> normalised latent rows
        [2 * frames, latent_channels]: frame-major, a frame's two channels side by side."""
        c = self.cfg
        if samples.dim() != 3 or samples.shape[0] != 2 or samples.shape[1] != 1 or \
                samples.shape[2] == 0 or samples.shape[2] % c.hop or samples.dtype != torch.float32:
            raise ValueError(f"the audio encoder reads the stereo pair as FP32 [2, 1, samples] of "
                             f"whole {c.hop}-sample latent frames, not {tuple(samples.shape)}")
        f = self.features(samples)
        out = torch.stack([self.project(f[ch].t().contiguous()) for ch in range(2)], 0)
        mean = TF.conv1d(out.permute(0, 2, 1), self.w["mean_proj.weight"],
                         self.w["mean_proj.bias"]).permute(0, 2, 1)          # [2, frames, C]
        if c.latents_mean:
            mean = (mean - torch.tensor(c.latents_mean, device=self.device)) / \
                torch.tensor(c.latents_std, device=self.device)
        return mean.permute(1, 0, 2).reshape(-1, c.latent_channels).contiguous()


def load_wav(url: str, sample_rate: int) -> torch.Tensor:
    """A PCM WAV file (``file://`` or base64 ``data:`` URL) -> FP32 [2, 1, samples] at
    ``sample_rate`` (linear resampling; a mono track becomes two identical channels)."""
    import base64
    import io
    import wave
    if url.startswith("data:"):
        head, _, payload = url.partition(",")
        if not head.endswith(";base64"):
            raise ValueError("data URLs must be base64-encoded")
        raw = base64.b64decode(payload, validate=True)
    elif url.startswith("file://"):
        from ..server.images import read_file_url      # media-directory rule of the deployment
        raw = read_file_url(url)
    else:
        raise ValueError("audio URLs must be data: or file:// URLs; remote URLs are not fetched")
    try:
        with wave.open(io.BytesIO(raw)) as wv:
            n, ch, width, rate = wv.getnframes(), wv.getnchannels(), wv.getsampwidth(), \
                wv.getframerate()
            pcm = wv.readframes(n)
    except (wave.Error, EOFError) as e:
        raise ValueError(f"cannot decode the audio track: {e}")
    if width != 2 or ch not in (1, 2) or n == 0:
        raise ValueError("audio tracks are 16-bit PCM WAV, mono or stereo, of at least a sample")
    x = torch.frombuffer(bytearray(pcm), dtype=torch.int16).float().div(32768.0).view(n, ch).t()
    if ch == 1:
        x = x.expand(2, -1)
    x = x.contiguous()[:, None, :]
    if rate != sample_rate:
        x = TF.interpolate(x, size=max(1, round(n * sample_rate / rate)), mode="linear",
                           align_corners=False)
    return x.contiguous()
