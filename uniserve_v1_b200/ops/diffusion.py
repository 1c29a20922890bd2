"""Diffusion-side operators: addressable noise, Euler step, patch layout."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import native as N

N.register_signatures({
    "us_philox_normal": (N.I, [N.P, N.L, ctypes.c_ulonglong, ctypes.c_uint, N.F, N.P]),
    "us_scaled_add": (N.I, [N.P, N.P, N.F, N.L, N.P]),
    "us_patchify": (N.I, [N.P, N.P, N.I, N.I, N.I, N.I, N.I, N.P]),
    "us_value_first_swiglu": (N.I, [N.P, N.P, N.L, N.I, N.P]),
})

M32 = np.uint64(0xFFFFFFFF)


def _philox_np(seed: int, positions: np.ndarray, stage: int, draw: int):
    """Vectorised Philox4x32-10, bit-identical to csrc/include/us_philox.h."""
    from ..utils.philox import splitmix64
    k = splitmix64(seed & 0xFFFFFFFFFFFFFFFF)
    k0 = np.uint64(k & 0xFFFFFFFF)
    k1 = np.uint64((k >> 32) & 0xFFFFFFFF)
    pos = positions.astype(np.uint64)
    c0, c1 = pos & M32, (pos >> np.uint64(32)) & M32
    c2 = np.full_like(c0, stage)
    c3 = np.full_like(c0, draw)
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c0
        p1 = np.uint64(0xCD9E8D57) * c2
        hi0, lo0 = (p0 >> np.uint64(32)) & M32, p0 & M32
        hi1, lo1 = (p1 >> np.uint64(32)) & M32, p1 & M32
        c0, c1, c2, c3 = hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0
        k0 = (k0 + np.uint64(0x9E3779B9)) & M32
        k1 = (k1 + np.uint64(0xBB67AE85)) & M32
    return c0, c1


def philox_normal(shape, seed: int, stream_id: int = 0, scale: float = 1.0, device="cpu"):
    """FP32 standard normals; element i depends on (seed, stream_id, i) only."""
    n = 1
    for s in shape:
        n *= s
    dev = torch.device(device)
    if dev.type == "cuda":
        out = torch.empty(n, dtype=torch.float32, device=dev)
        N.call("us_philox_normal", N.ptr(out), n, seed & 0xFFFFFFFFFFFFFFFF, stream_id, scale,
               N.stream())
        return out.view(*shape)
    pairs = (n + 1) // 2
    w0, w1 = _philox_np(seed, np.arange(pairs, dtype=np.uint64), stream_id, 1)
    u0 = ((w0 >> np.uint64(8)).astype(np.float32) + np.float32(0.5)) * np.float32(1 / 16777216)
    u1 = ((w1 >> np.uint64(8)).astype(np.float32) + np.float32(0.5)) * np.float32(1 / 16777216)
    r = np.sqrt(np.float32(-2.0) * np.log(u0))
    ang = np.float32(6.283185307179586) * u1
    z = np.stack([r * np.cos(ang), r * np.sin(ang)], axis=1).reshape(-1)[:n]
    return torch.from_numpy((z * np.float32(scale)).astype(np.float32)).view(*shape)


def scaled_add_(x, v, s: float):
    """x += v * s in FP32 (Euler step)."""
    if not x.is_cuda:
        x.add_(v, alpha=s)
        return x
    assert x.dtype == torch.float32 and v.dtype == torch.float32 and x.is_contiguous()
    N.call("us_scaled_add", N.ptr(x), N.ptr(v.contiguous()), float(s), x.numel(), N.stream())
    return x


def patchify(latent):
    """[C, F, H, W] fp32 -> [F*(H/2)*(W/2), C*4]."""
    C, Fr, H, W = latent.shape
    if not latent.is_cuda:
        x = latent.view(C, Fr, H // 2, 2, W // 2, 2).permute(1, 2, 4, 0, 3, 5)
        return x.reshape(Fr * (H // 2) * (W // 2), C * 4).contiguous()
    rows = torch.empty(Fr * (H // 2) * (W // 2), C * 4, dtype=torch.float32, device=latent.device)
    N.call("us_patchify", N.ptr(latent.contiguous()), N.ptr(rows), C, Fr, H, W, 0, N.stream())
    return rows


def unpatchify(rows, C, Fr, H, W):
    if not rows.is_cuda:
        x = rows.view(Fr, H // 2, W // 2, C, 2, 2).permute(3, 0, 1, 4, 2, 5)
        return x.reshape(C, Fr, H, W).contiguous()
    latent = torch.empty(C, Fr, H, W, dtype=torch.float32, device=rows.device)
    N.call("us_patchify", N.ptr(latent), N.ptr(rows.contiguous()), C, Fr, H, W, 1, N.stream())
    return latent
