"""Video VAE encoder: the causal convolutional network that turns a condition's pixels (a
keyframe, a reference clip) into its latent.

Structure (FP32 throughout; convolutions are library calls, this is not a hot path)::

    conv_in      3x3x3, two zero frames in front (causal in time), one pixel around in space
    stage i      ``layers_per_block`` residual blocks (per-frame GroupNorm -> SiLU -> causal
                 conv, twice; 1x1x1 shortcut when the width changes), then, when the stage
                 strides, a 3x3x3 convolution with stride (t, s, s): two zero frames in front
                 and none behind, so T frames become ceil(T / t); one row below and one column
                 to the right when s == 2
    norm_out     per-frame GroupNorm -> SiLU;  conv_out to 2 * latent channels (mean | logvar)
    quant_conv   1x1x1 on the moments

``encode_condition`` samples the posterior under a seed (the same condition always encodes to
the same latent): ``mean + exp(0.5 * clamp(logvar, -30, 20)) * noise`` rounded through FP16, then
``(sample - latents_mean) / latents_std`` per channel.  With ``tile`` set, a raster wider than
the tile is encoded in overlapping tiles whose projected moments cross-fade where they meet.

Reference behaviour: crates/models/src/minimax_h3/video_vae.rs:46-55, 852-886, 1082-1120
(reference project paths).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as TF

PIXEL_MEAN = (0.485, 0.456, 0.406)
PIXEL_STD = (0.229, 0.224, 0.225)


@dataclass
class VideoEncoderConfig:
    in_channels: int = 3
    latent_channels: int = 24
    block_out_channels: tuple = (128, 256, 512, 512, 512)
    spatial_downsample_factors: tuple = (2, 2, 2, 2, 1)
    temporal_downsample_factors: tuple = (1, 2, 2, 1, 1)
    layers_per_block: int = 2
    norm_num_groups: int = 32
    norm_eps: float = 1e-6
    latents_mean: tuple = ()
    latents_std: tuple = ()
    tile: int = 0          # pixels a side of an encode tile (0: whole rasters)
    tile_overlap: int = 0  # pixels two neighbouring tiles share

    @classmethod
    def tiny(cls, latent_channels: int = 4, spatial: int = 4):
        n = {4: 2, 8: 3, 16: 4, 32: 5, 64: 6}[spatial]
        return cls(latent_channels=latent_channels, block_out_channels=(8,) * n + (16,),
                   spatial_downsample_factors=(2,) * n + (1,),
                   temporal_downsample_factors=(1,) * (n - 2) + (2, 2, 1),
                   layers_per_block=1, norm_num_groups=4)

    @property
    def spatial(self) -> int:
        out = 1
        for s in self.spatial_downsample_factors:
            out *= s
        return out

    @property
    def temporal(self) -> int:
        out = 1
        for s in self.temporal_downsample_factors:
            out *= s
        return out


def causal_pad(x: torch.Tensor, left=1, right=1, top=1, bottom=1, front=2) -> torch.Tensor:
    return TF.pad(x, (left, right, top, bottom, front, 0))


def frame_norm(x: torch.Tensor, groups: int, w, b, eps: float) -> torch.Tensor:
    """GroupNorm of every frame by itself: x [n, c, d, h, w]."""
    n, c, d, h, wd = x.shape
    y = TF.group_norm(x.permute(0, 2, 1, 3, 4).reshape(n * d, c, h, wd), groups, w, b, eps)
    return y.view(n, d, c, h, wd).permute(0, 2, 1, 3, 4)


class VideoVaeEncoder:
    def __init__(self, cfg: VideoEncoderConfig, device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        if len({len(cfg.block_out_channels), len(cfg.spatial_downsample_factors),
                len(cfg.temporal_downsample_factors)}) != 1:
            raise ValueError("the encoder's stages, spatial strides and temporal strides differ "
                             "in number")
        if any(s not in (1, 2) for s in cfg.spatial_downsample_factors):
            raise ValueError("a spatial stride of the video encoder is neither one nor two")
        self.w: dict = {}

    def init_random(self, seed: int = 0, std: float = 0.05) -> "VideoVaeEncoder":
        c, g = self.cfg, torch.Generator().manual_seed(seed)

        def conv(name, cin, cout, k):
            self.w[name + ".weight"] = (torch.randn(cout, cin, k, k, k, generator=g) * std /
                                        max(1.0, (cin * k ** 3 / 27) ** 0.5) * 3).to(self.device)
            self.w[name + ".bias"] = torch.zeros(cout, device=self.device)

        def norm(name, ch):
            self.w[name + ".weight"] = torch.ones(ch, device=self.device)
            self.w[name + ".bias"] = torch.zeros(ch, device=self.device)
        width = c.block_out_channels[0]
        conv("encoder.conv_in", c.in_channels, width, 3)
        for i, out in enumerate(c.block_out_channels):
            for j in range(c.layers_per_block):
                p = f"encoder.down_blocks.{i}.resnets.{j}"
                cin = width if j == 0 else out
                norm(p + ".norm1", cin)
                conv(p + ".conv1", cin, out, 3)
                norm(p + ".norm2", out)
                conv(p + ".conv2", out, out, 3)
                if cin != out:
                    conv(p + ".conv_shortcut", cin, out, 1)
            if c.spatial_downsample_factors[i] * c.temporal_downsample_factors[i] > 1:
                conv(f"encoder.down_blocks.{i}.downsamplers.0.conv", out, out, 3)
            width = out
        norm("encoder.norm_out", width)
        conv("encoder.conv_out", width, 2 * c.latent_channels, 3)
        conv("quant_conv", 2 * c.latent_channels, 2 * c.latent_channels, 1)
        return self

    def load_state(self, loader, prefix: str = "vae.") -> "VideoVaeEncoder":
        """Tensors by the names ``init_random`` makes, under ``prefix``."""
        self.init_random(0)
        for name in list(self.w):
            self.w[name] = loader.get(prefix + name).to(device=self.device, dtype=torch.float32)
        return self

    def _conv(self, name, x, stride=(1, 1, 1)):
        return TF.conv3d(x, self.w[name + ".weight"], self.w[name + ".bias"], stride=stride)

    def _resnet(self, p: str, x: torch.Tensor) -> torch.Tensor:
        c, w = self.cfg, self.w
        h = TF.silu(frame_norm(x, c.norm_num_groups, w[p + ".norm1.weight"], w[p + ".norm1.bias"],
                               c.norm_eps))
        h = self._conv(p + ".conv1", causal_pad(h))
        h = TF.silu(frame_norm(h, c.norm_num_groups, w[p + ".norm2.weight"], w[p + ".norm2.bias"],
                               c.norm_eps))
        h = self._conv(p + ".conv2", causal_pad(h))
        if p + ".conv_shortcut.weight" in w:
            x = self._conv(p + ".conv_shortcut", x)
        return x + h

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """pixels [n, 3, T, H, W] FP32 -> moments [n, 2 * C, ceil(T / temporal), H / s, W / s]
        (before ``quant_conv``)."""
        c = self.cfg
        h = self._conv("encoder.conv_in", causal_pad(pixels.to(self.device, torch.float32)))
        for i in range(len(c.block_out_channels)):
            for j in range(c.layers_per_block):
                h = self._resnet(f"encoder.down_blocks.{i}.resnets.{j}", h)
            s, t = c.spatial_downsample_factors[i], c.temporal_downsample_factors[i]
            if s * t > 1:
                # halving space pads one row below and one column to the right only
                padded = TF.pad(h, (0, 1, 0, 1, 2, 0)) if s == 2 else causal_pad(h)
                h = self._conv(f"encoder.down_blocks.{i}.downsamplers.0.conv", padded, (t, s, s))
        w = self.w
        h = TF.silu(frame_norm(h, c.norm_num_groups, w["encoder.norm_out.weight"],
                               w["encoder.norm_out.bias"], c.norm_eps))
        return self._conv("encoder.conv_out", causal_pad(h))

    def moments(self, pixels: torch.Tensor) -> torch.Tensor:
        """pixels [3, T, H, W] -> projected moments [2 * C, T', H / s, W / s].  A raster wider
        than the configured tile is encoded tile by tile (each tile's moments projected by
        ``quant_conv``) and the tiles cross-fade over their overlap."""
        c = self.cfg
        H, W = pixels.shape[2:]
        one = lambda px: self._conv("quant_conv", self.forward(px[None]))[0]
        if not c.tile or (H <= c.tile and W <= c.tile):
            return one(pixels)
        if c.tile % c.spatial or c.tile_overlap % c.spatial or not 0 <= c.tile_overlap < c.tile:
            raise ValueError("encode tiles and their overlap are whole latent cells, the overlap "
                             "smaller than the tile")
        step, s, tiles = c.tile - c.tile_overlap, c.spatial, []
        ys = list(range(0, max(H - c.tile_overlap, 1), step))
        xs = list(range(0, max(W - c.tile_overlap, 1), step))
        for y0 in ys:
            for x0 in xs:
                tiles.append((y0 // s, x0 // s, one(pixels[:, :, y0:y0 + c.tile, x0:x0 + c.tile])))
        return blend_tiles(tiles, H // s, W // s, c.tile_overlap // s)

    def encode_condition(self, pixels: torch.Tensor, seed: int = 0) -> torch.Tensor:
        """pixels [3, T, H, W] normalised by the ImageNet constants (one frame for a still) ->
        the normalised latent [C, ceil(T / temporal), H / s, W / s] in FP32."""
        from ..ops.diffusion import philox_normal
        c = self.cfg
        if pixels.dim() != 4 or pixels.shape[0] != c.in_channels:
            raise ValueError(f"the video encoder reads [{c.in_channels}, frames, height, width]")
        if pixels.shape[2] % c.spatial or pixels.shape[3] % c.spatial:
            raise ValueError(f"a condition's raster is whole {c.spatial}-pixel cells")
        m = self.moments(pixels)
        mean, logvar = m[:c.latent_channels], m[c.latent_channels:].clamp(-30.0, 20.0)
        noise = philox_normal(tuple(mean.shape), seed, 7, 1.0, self.device)
        z = (mean + torch.exp(0.5 * logvar) * noise).half().float()
        if c.latents_mean:
            mu = torch.tensor(c.latents_mean, device=self.device).view(-1, 1, 1, 1)
            sd = torch.tensor(c.latents_std, device=self.device).view(-1, 1, 1, 1)
            z = (z - mu) / sd
        return z


def blend_tiles(tiles: list, height: int, width: int, overlap: int) -> torch.Tensor:
    """Stitches ``tiles`` = [(row, column, tensor [..., h, w])] into [..., height, width]: where
    two tiles meet, the earlier fades out and the later fades in linearly over ``overlap`` cells
    (weights i / (overlap + 1)); a tile's outer edges keep full weight."""
    first = tiles[0][2]
    out = torch.zeros(*first.shape[:-2], height, width, dtype=first.dtype, device=first.device)
    total = torch.zeros(height, width, dtype=first.dtype, device=first.device)
    for y0, x0, t in tiles:
        h, w = t.shape[-2:]

        def ramp(n, origin, limit):
            r = torch.ones(n, dtype=first.dtype, device=first.device)
            k = min(overlap, n)
            if k and origin > 0:                      # fades in over what the previous tile covers
                r[:k] = torch.arange(1, k + 1, device=first.device) / (k + 1)
            if k and origin + n < limit:              # fades out under the next tile
                r[n - k:] = torch.minimum(r[n - k:], torch.arange(k, 0, -1, device=first.device)
                                          / (k + 1))
            return r
        wgt = ramp(h, y0, height)[:, None] * ramp(w, x0, width)[None, :]
        out[..., y0:y0 + h, x0:x0 + w] += t * wgt
        total[y0:y0 + h, x0:x0 + w] += wgt
    return out / total.clamp_min(1e-12)


def normalize_pixels(rgb_u8: torch.Tensor) -> torch.Tensor:
    """uint8 [T, H, W, 3] -> FP32 [3, T, H, W] normalised by the ImageNet mean and deviation."""
    x = rgb_u8.float().div(255.0)
    mean = torch.tensor(PIXEL_MEAN, device=x.device)
    std = torch.tensor(PIXEL_STD, device=x.device)
    return ((x - mean) / std).permute(3, 0, 1, 2).contiguous()
