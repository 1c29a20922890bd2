"""NVFP4: 4-bit E2M1 values in blocks of 16 with an E4M3 scale per block and an FP32
scale per tensor (the ModelOpt export format).

    value = e2m1(nibble) * e4m3(block scale) * global scale

Two values share a byte, the even element in the low nibble.  ``quantize`` follows the
ModelOpt recipe: the global scale maps the tensor's amax to 6 * 448, each block scale is
``block amax / 6`` expressed in units of the global scale and rounded to E4M3, and the
elements are rounded to the nearest representable magnitude (ties to the even code).

This package serves such checkpoints by expanding them when they are loaded
(``checkpoint/quantized.py``); a block-scaled FP4 tensor-core GEMM is not part of it.

Reference behaviour: crates/nn/src/quantization/nvfp4.rs, docs/configuration.md:300-312
(reference project paths).
"""
from __future__ import annotations

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
BLOCK = 16
E2M1_MAX, E4M3_MAX = 6.0, 448.0


def _table(device, dtype=torch.float32) -> torch.Tensor:
    mags = torch.tensor(E2M1_VALUES, dtype=dtype, device=device)
    return torch.cat([mags, -mags])                       # code = sign << 3 | magnitude


def unpack(packed: torch.Tensor) -> torch.Tensor:
    """[..., K / 2] uint8 -> [..., K] codes 0..15 (uint8)."""
    lo, hi = packed & 0xF, packed >> 4
    return torch.stack([lo, hi], dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def pack(codes: torch.Tensor) -> torch.Tensor:
    c = codes.reshape(*codes.shape[:-1], codes.shape[-1] // 2, 2)
    return (c[..., 0] | (c[..., 1] << 4)).to(torch.uint8)


def dequantize(packed: torch.Tensor, block_scale: torch.Tensor, global_scale,
               dtype=torch.bfloat16) -> torch.Tensor:
    """packed [..., M, K / 2] uint8, block_scale [..., M, K / 16] (float8_e4m3fn or its
    bytes), global_scale scalar -> [..., M, K]."""
    if block_scale.dtype == torch.uint8:
        block_scale = block_scale.view(torch.float8_e4m3fn)
    vals = _table(packed.device)[unpack(packed).long()]
    K = vals.shape[-1]
    assert K % BLOCK == 0 and block_scale.shape[-1] == K // BLOCK
    s = block_scale.float() * float(global_scale)
    out = vals.reshape(*vals.shape[:-1], K // BLOCK, BLOCK) * s[..., None]
    return out.reshape(*vals.shape).to(dtype)


def quantize(w: torch.Tensor):
    """w [..., M, K] (K a multiple of 16) -> (packed uint8 [..., M, K / 2],
    block_scale float8_e4m3fn [..., M, K / 16], global_scale FP32 scalar tensor)."""
    K = w.shape[-1]
    assert K % BLOCK == 0
    f = w.float()
    amax = f.abs().max()
    gscale = torch.where(amax > 0, amax / (E2M1_MAX * E4M3_MAX), torch.ones_like(amax))
    blocks = f.reshape(*f.shape[:-1], K // BLOCK, BLOCK)
    bmax = blocks.abs().amax(-1)
    bscale = (bmax / E2M1_MAX / gscale).clamp(max=E4M3_MAX).to(torch.float8_e4m3fn)
    denom = bscale.float() * gscale
    scaled = torch.where(denom[..., None] > 0, blocks / denom[..., None].clamp(min=1e-30),
                         torch.zeros_like(blocks))
    mags = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=w.device)
    mag = scaled.abs().clamp(max=E2M1_MAX)
    # nearest representable magnitude; ties go to the even code (0, 1.0, 2.0, 4.0 ...)
    d = (mag[..., None] - mags).abs()
    idx = d.argmin(-1)
    nxt = (idx + 1).clamp(max=7)
    tie = (d.gather(-1, nxt[..., None])[..., 0] == d.gather(-1, idx[..., None])[..., 0]) & \
        (nxt != idx)
    idx = torch.where(tie & (idx % 2 == 1), nxt, idx)
    codes = (idx | ((scaled < 0).long() << 3)).to(torch.uint8)
    return pack(codes.reshape(*f.shape)), bscale, gscale.reshape(())
