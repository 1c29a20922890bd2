"""FP8 (E4M3) quantisation and block-scaled GEMMs.

Weights of block-quantised checkpoints carry one FP32 scale per 128 x 128 block
(``weight_scale_inv``); activations are quantised on the fly with one scale per
row and 128-wide K block, stored transposed ``[K / 128, rows_ld]`` so that a GEMM
tile reads the scales of its rows contiguously.  The reference serves per-tensor
FP8 (static ``input_scale`` or dynamic amax / 448, crates/ops/src/fp8.rs:1-40,
crates/nn/src/quantization/dynamic.rs, reference project paths) and refuses the
block-scaled form; both are provided here.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import native as N
from .functional import _ACT, _block_n, _cuda

N.register_signatures({
    "us_gemm_fp8_block": (N.I, [N.P, N.P, N.P, N.P, N.L, N.P, N.I, N.I, N.I, N.I, N.I, N.L, N.L,
                                N.L, N.I, N.I, N.I, N.I, N.P, N.P, N.P, N.P, N.P, N.P, N.I, N.I,
                                N.P]),
    "us_fp8_quantize_rows_block128": (N.I, [N.P, N.L, N.P, N.L, N.P, N.L, N.I, N.I, N.P, N.P]),
    "us_fp8_quantize_tensor": (N.I, [N.P, N.P, N.L, N.F, N.P, N.P, N.P]),
})

E4M3_MAX = 448.0
BF16 = torch.bfloat16
PAD_ROWS = 256          # scale rows a tile may read past the last valid row


# ---------------------------------------------------------------- weights ----
def quantize_weight_block128(w: torch.Tensor):
    """[..., M, K] (M, K multiples of 128) -> (e4m3 bytes [..., M, K] uint8,
    scales [..., M / 128, K / 128] fp32) with w ~= q * scale."""
    *lead, M, K = w.shape
    assert M % 128 == 0 and K % 128 == 0
    b = w.float().reshape(*lead, M // 128, 128, K // 128, 128)
    amax = b.abs().amax(dim=(-3, -1))
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (b * (1.0 / scale)[..., :, None, :, None]).to(torch.float8_e4m3fn)
    return q.reshape(*lead, M, K).view(torch.uint8).contiguous(), scale.contiguous()


def dequantize_weight_block128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    *lead, M, K = q.shape
    f = q.view(torch.float8_e4m3fn).float().reshape(*lead, M // 128, 128, K // 128, 128)
    return (f * scale[..., :, None, :, None]).reshape(*lead, M, K)


# ------------------------------------------------------------- activations ---
def quantize_rows_block128(x: torch.Tensor, live=None, q=None, scales=None):
    """x [T, K] bf16 -> (q [T, K] uint8 e4m3, scales [K / 128, ld] fp32, ld >= T + 256)."""
    T, K = x.shape
    assert K % 128 == 0
    if q is None:
        q = torch.zeros(T + PAD_ROWS, K, dtype=torch.uint8, device=x.device)[:T]
    if scales is None:
        scales = torch.ones(K // 128, T + PAD_ROWS, dtype=torch.float32, device=x.device)
    if not _cuda(x):
        b = x.float().reshape(T, K // 128, 128)
        amax = b.abs().amax(-1)
        s = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
        q.copy_((b * (1.0 / s)[..., None]).to(torch.float8_e4m3fn).reshape(T, K).view(torch.uint8))
        scales[:, :T] = s.t()
        return q, scales
    assert x.dtype == BF16 and x.stride(1) == 1
    N.call("us_fp8_quantize_rows_block128", N.ptr(x), x.stride(0), N.ptr(q), q.stride(0),
           N.ptr(scales), scales.stride(0), T, K, N.ptr(live) if live is not None else None,
           N.stream())
    return q, scales


def dequantize_rows_block128(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    T, K = q.shape
    f = q.view(torch.float8_e4m3fn).float().reshape(T, K // 128, 128)
    return (f * scales[:, :T].t()[..., None]).reshape(T, K)


def quantize_tensor(x: torch.Tensor, scale: float | None = None):
    """Per-tensor: q = x / scale.  Without a scale it is measured on the device
    (amax / 448).  Returns (q uint8 like x, scale tensor [1] fp32)."""
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    if not _cuda(x):
        s = float(scale) if scale else max(float(x.float().abs().max()) / E4M3_MAX, 1e-30)
        q.copy_((x.float() * (1.0 / s)).to(torch.float8_e4m3fn).view(torch.uint8))
        return q, torch.tensor([s])
    x = x.contiguous()
    out_scale = torch.empty(1, dtype=torch.float32, device=x.device)
    scratch = None if scale else torch.zeros(1, dtype=torch.float32, device=x.device)
    N.call("us_fp8_quantize_tensor", N.ptr(x), N.ptr(q), x.numel(), float(scale or 0.0),
           N.ptr(scratch) if scratch is not None else None, N.ptr(out_scale), N.stream(),
           launches=1 if scale else 2)
    return q, out_scale


# ------------------------------------------------------------------ GEMMs ----
def linear_fp8_block(x, wq, w_scale, gated=False, act="silu", stepwise=False, out_dtype=None,
                     xq=None, x_scale=None):
    """y = x @ dequant(wq).T for block-scaled weights ``wq`` [M(, x2 gated), K] uint8 with
    ``w_scale`` [rows / 128, K / 128].  ``x`` is bf16 (quantised here per row and
    K block) unless ``xq``/``x_scale`` are given."""
    if not _cuda(wq):
        if xq is None:
            xq, x_scale = quantize_rows_block128(x)
        xf = dequantize_rows_block128(xq, x_scale)
        wf = dequantize_weight_block128(wq, w_scale)
        y = xf @ wf.t()
        if gated:
            M = wq.shape[0] // 2
            g = y[:, M:]
            if act == "silu":
                a = torch.nn.functional.silu(g)
            else:
                a = torch.nn.functional.gelu(g, approximate="tanh")
            y = y[:, :M] * a
        return y.to(out_dtype or BF16)
    if xq is None:
        xq, x_scale = quantize_rows_block128(x)
    T, K = xq.shape
    rows_w = wq.shape[0]
    M = rows_w // 2 if gated else rows_w
    odt = out_dtype or BF16
    out = torch.empty(T, M, dtype=odt, device=wq.device)
    bn = min(_block_n(T, gated), 64 if gated else 128)
    code = _ACT["silu_stepwise" if (act == "silu" and stepwise) else act] if gated else 0
    N.call("us_gemm_fp8_block", N.ptr(wq), N.ptr(w_scale), N.ptr(xq), N.ptr(x_scale),
           x_scale.stride(0), N.ptr(out), 1, rows_w, M, K, T, wq.stride(0), xq.stride(0), M,
           1 if gated else 0, M if gated else 0, code, 0 if odt == BF16 else 1, None, None, None,
           None, None, None, 0, bn, N.stream())
    return out


@dataclass
class Fp8Experts:
    """Block-quantised stacked expert weights of one layer."""
    w13: torch.Tensor      # [E, 2I, H] uint8
    w13_scale: torch.Tensor
    w2: torch.Tensor       # [E, H, I] uint8
    w2_scale: torch.Tensor

    @staticmethod
    def from_bf16(w13: torch.Tensor, w2: torch.Tensor) -> "Fp8Experts":
        q13, s13 = quantize_weight_block128(w13)
        q2, s2 = quantize_weight_block128(w2)
        return Fp8Experts(q13, s13, q2, s2)


def moe_experts_fp8(x, ids, weights, ex: Fp8Experts, e_lo=0, act="silu", ws=None, out=None):
    """Routed experts with block-scaled FP8 weights: sort, gather, quantise the
    permuted rows, grouped FC1 (gated activation fused), quantise, grouped FC2,
    weighted un-permute."""
    from .functional import MoeWorkspace
    if not _cuda(x):
        from . import reference as R
        w13 = dequantize_weight_block128(ex.w13, ex.w13_scale)
        w2 = dequantize_weight_block128(ex.w2, ex.w2_scale)
        return R.moe_experts(x, ids, weights, w13, w2, e_lo, act, False)
    T, H = x.shape
    top_k = ids.shape[1]
    E, I2, _ = ex.w13.shape
    I_ = I2 // 2
    if ws is None:
        ws = MoeWorkspace.create(T, top_k, E, H, I_, x.device)
    if ws.block_n > 64:
        raise ValueError("the gated FP8 GEMM serves row tiles of at most 64")
    R_ = T * top_k
    q8 = getattr(ws, "_fp8", None)
    if q8 is None:
        dev = x.device
        q8 = dict(
            xq=torch.zeros(R_ + PAD_ROWS, H, dtype=torch.uint8, device=dev)[:R_],
            xs=torch.ones(H // 128, R_ + PAD_ROWS, dtype=torch.float32, device=dev),
            hq=torch.zeros(R_ + PAD_ROWS, I_, dtype=torch.uint8, device=dev)[:R_],
            hs=torch.ones(I_ // 128, R_ + PAD_ROWS, dtype=torch.float32, device=dev))
        ws._fp8 = q8
    st = N.stream()
    N.call("us_moe_sort", N.ptr(ids), R_, e_lo, E, ws.block_n, ws.max_tiles,
           N.ptr(ws.sorted_route), N.ptr(ws.perm_of_route), N.ptr(ws.expert_offsets),
           N.ptr(ws.tile_group), N.ptr(ws.tile_row0), N.ptr(ws.tile_rows), N.ptr(ws.num_tiles), st)
    total = ws.expert_offsets[E:]
    N.call("us_moe_gather", N.ptr(x), N.ptr(ws.sorted_route), N.ptr(total), R_, top_k, H,
           N.ptr(ws.xp), st)
    quantize_rows_block128(ws.xp, total, q8["xq"], q8["xs"])
    tiles = (N.ptr(ws.tile_group), N.ptr(ws.tile_row0), N.ptr(ws.tile_rows), N.ptr(ws.num_tiles),
             ws.max_tiles, ws.block_n)
    N.call("us_gemm_fp8_block", N.ptr(ex.w13), N.ptr(ex.w13_scale), N.ptr(q8["xq"]),
           N.ptr(q8["xs"]), q8["xs"].stride(0), N.ptr(ws.h), E, I2, I_, H, R_, H, H, I_, 1, I_,
           _ACT[act], 0, None, None, *tiles, st)
    quantize_rows_block128(ws.h, total, q8["hq"], q8["hs"])
    N.call("us_gemm_fp8_block", N.ptr(ex.w2), N.ptr(ex.w2_scale), N.ptr(q8["hq"]),
           N.ptr(q8["hs"]), q8["hs"].stride(0), N.ptr(ws.y), E, H, H, I_, R_, I_, I_, H, 0, 0, 0,
           0, None, None, *tiles, st)
    if out is None:
        out = torch.empty(T, H, dtype=BF16, device=x.device)
    N.call("us_moe_unpermute", N.ptr(ws.y), N.ptr(ws.perm_of_route), N.ptr(weights), T, top_k, H,
           N.ptr(out), st)
    return out


# ------------------------------------------------- per-tensor weights, per-row rows ----
N.register_signatures({
    "us_gemm_fp8_rowscale": (N.I, [N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.L, N.L, N.L, N.I, N.I, N.I,
                                   N.I, N.P, N.I, N.P]),
    "us_fp8_quantize_rows": (N.I, [N.P, N.L, N.P, N.L, N.P, N.I, N.I, N.F, N.P]),
})


def quantize_weight_tensor(w: torch.Tensor):
    """One scale for the whole tensor (the ModelOpt / dynamic per-tensor form):
    returns (e4m3 bytes like w, scale as a Python float)."""
    amax = float(w.float().abs().max())
    scale = amax / E4M3_MAX if amax > 0 else 1.0
    q = (w.float() * (1.0 / scale)).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
    return q, scale


def quantize_rows(x: torch.Tensor, weight_scale: float = 1.0):
    """x [T, K] bf16 -> (q [T, K] uint8 e4m3, out_scale [T] = row scale * weight_scale)."""
    T, K = x.shape
    if not _cuda(x):
        amax = x.float().abs().amax(-1)
        s = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
        q = (x.float() * (1.0 / s)[:, None]).to(torch.float8_e4m3fn).view(torch.uint8)
        return q, s * weight_scale
    assert x.dtype == BF16 and x.stride(1) == 1
    q = torch.empty(T, K, dtype=torch.uint8, device=x.device)
    s = torch.empty(T, dtype=torch.float32, device=x.device)
    N.call("us_fp8_quantize_rows", N.ptr(x), x.stride(0), N.ptr(q), K, N.ptr(s), T, K,
           float(weight_scale), N.stream())
    return q, s


def linear_fp8(x, wq, w_scale: float, gated=False, act="silu", stepwise=False, out_dtype=None):
    """y = x @ (wq * w_scale).T with per-tensor FP8 weights and per-row dynamic FP8
    activations, FP32 accumulation over the whole K, scales applied in the epilogue
    (before the gated activation).  ``wq`` [M (x 2 when gated), K] uint8."""
    xq, xs = quantize_rows(x, w_scale)
    rows_w, K = wq.shape
    M = rows_w // 2 if gated else rows_w
    T = x.shape[0]
    odt = out_dtype or BF16
    if not _cuda(x):
        y = (xq.view(torch.float8_e4m3fn).float() @ wq.view(torch.float8_e4m3fn).float().t()) * \
            xs[:, None]
        if gated:
            g = y[:, M:]
            a = torch.nn.functional.silu(g) if act == "silu" else \
                torch.nn.functional.gelu(g, approximate="tanh")
            y = y[:, :M] * a
        return y.to(odt)
    out = torch.empty(T, M, dtype=odt, device=x.device)
    code = _ACT["silu_stepwise" if (act == "silu" and stepwise) else act] if gated else 0
    N.call("us_gemm_fp8_rowscale", N.ptr(wq), N.ptr(xq), N.ptr(out), rows_w, M, K, T, wq.stride(0),
           K, M, 1 if gated else 0, M if gated else 0, code, 0 if odt == BF16 else 1, N.ptr(xs),
           128 if gated else 256, N.stream())
    return out
