"""Varlen flash attention (tcgen05) binding."""
from __future__ import annotations

import torch

from . import native as N
from . import reference as R

BF16 = torch.bfloat16

import os

_SIG = (N.I, [N.P, N.P, N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.I, N.I, N.I, N.L, N.L, N.L, N.L,
              N.F, N.I, N.P])
N.register_signatures({"us_flash_attn_varlen": _SIG, "us_flash_attn_varlen2": _SIG})

# Two kernels share one contract: the two-tile ping-pong kernel (default when a
# sequence has more than one 128-row query tile) and the single-tile kernel.
_SINGLE_TILE_ONLY = os.environ.get("US_FLASH_V1", "0") == "1"


def flash_attn_varlen(q, k, v, cu_q, cu_k, max_q, max_k, scale, causal, out=None):
    """q [Tq, Hq, D], k/v [Tk, Hkv, D] bf16 with contiguous (head, dim) and any
    row stride; cu_q/cu_k int32 [n+1] on the device.  Returns [Tq, Hq, D]."""
    lib = N.kernels()
    if not hasattr(lib, "us_flash_attn_varlen"):
        raise N.NativeMissing("the kernel library has no flash attention entry point: rebuild "
                              "it (`python -m uniserve_v1_b200.build`)")
    Tq, Hq, D = q.shape
    Tk, Hkv, _ = k.shape
    if D not in (64, 128) and D < 128 and D % 8 == 0:
        # other head widths (the 96-wide refiner heads): zero channels up to 128 add nothing
        # to q . k and give zero output channels, which are cut off again
        pad = 128 - D
        qp, kp, vp = (torch.nn.functional.pad(t, (0, pad)) for t in (q, k, v))
        full = flash_attn_varlen(qp, kp, vp, cu_q, cu_k, max_q, max_k, scale, causal)
        res = full[..., :D]
        if out is not None:
            out.copy_(res)
            return out
        return res.contiguous()
    assert q.dtype == BF16 and q.stride(2) == 1 and q.stride(1) == D
    assert k.stride(2) == 1 and k.stride(1) == D and v.stride(2) == 1 and v.stride(1) == D
    if out is None:
        out = torch.empty(Tq, Hq, D, dtype=BF16, device=q.device)
    n = cu_q.numel() - 1
    if D not in (64, 128):
        raise ValueError(f"flash attention serves head widths 64, 128 and multiples of 8 below "
                         f"128 (padded); got {D}")
    # head 64 is served by the two-tile kernel only
    name = "us_flash_attn_varlen" if (D == 128 and (_SINGLE_TILE_ONLY or max_q <= 128)) else \
        "us_flash_attn_varlen2"
    N.call(name, N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(out), N.ptr(cu_q),
           N.ptr(cu_k), n, Tq, Tk, Hq, Hkv, D, max_q, q.stride(0), k.stride(0), v.stride(0),
           out.stride(0), scale, int(causal), N.stream())
    return out
