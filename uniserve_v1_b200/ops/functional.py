"""Fused operators of the token and video paths.

Each function runs the hand-written sm_100a kernel when its inputs live on a
CUDA device and the FP32 PyTorch restatement from :mod:`.reference` otherwise
(CPU tests, the tiny CPU model).  On a GPU there is no fallback: a missing
kernel library raises.

The operator list follows the reference's ``ops`` crate (crates/ops/src/*.rs,
reference project paths): norm, rope, kv, attention, gemm, moe/{routing,sort,
grouped,combine}, sampler.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from . import native as N
from . import reference as R

BF16 = torch.bfloat16


def _cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


# ------------------------------------------------------------------ norms --
def rmsnorm(x, w, eps=1e-6, out=None):
    if not _cuda(x):
        return R.rmsnorm(x, w, eps)
    x2 = x.reshape(-1, x.shape[-1])
    assert x2.stride(-1) == 1 and x.dtype == BF16
    y = out if out is not None else torch.empty_like(x2)
    N.call("us_rmsnorm", N.ptr(x2), N.ptr(w), N.ptr(y), x2.shape[0], x2.shape[1],
           x2.stride(0), y.stride(0), eps, N.stream())
    return y.view(x.shape)


def add_rmsnorm(x, residual, w, eps=1e-6, out=None):
    """Residual stream in FP32: ``residual += x``; returns (normed bf16, residual).
    ``residual=None`` starts the stream (residual = x)."""
    if not _cuda(x):
        return R.add_rmsnorm(x, residual, w, eps)
    assert x.is_contiguous() and x.dtype == BF16
    first = residual is None
    if first:
        residual = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    y = out if out is not None else torch.empty_like(x)
    N.call("us_add_rmsnorm", N.ptr(x), N.ptr(residual), N.ptr(w), N.ptr(y), x.shape[0],
           x.shape[1], eps, int(first), N.stream())
    return y, residual


def add_rmsnorm_(x, residual, w, y, eps, first: bool):
    """In-place form for static graph buffers."""
    N.call("us_add_rmsnorm", N.ptr(x), N.ptr(residual), N.ptr(w), N.ptr(y), x.shape[0],
           x.shape[1], eps, int(first), N.stream())


def modulated_rmsnorm(x, w, table, idx, vectors_per_row, shift_slot, scale_slot, eps=1e-6):
    if not _cuda(x):
        return R.modulated_rmsnorm(x, w, table, idx, vectors_per_row, shift_slot, scale_slot, eps)
    y = torch.empty_like(x)
    N.call("us_modulated_rmsnorm", N.ptr(x), N.ptr(w), N.ptr(table), N.ptr(idx), vectors_per_row,
           shift_slot, scale_slot, N.ptr(y), x.shape[0], x.shape[1], eps, N.stream())
    return y


def gated_residual_(h, u, table, idx, vectors_per_row, gate_slot):
    """h += gate[idx] * u, in place; returns h."""
    if not _cuda(h):
        h.copy_(R.gated_residual(h, u, table, idx, vectors_per_row, gate_slot))
        return h
    N.call("us_gated_residual", N.ptr(h), N.ptr(u), N.ptr(table), N.ptr(idx), vectors_per_row,
           gate_slot, h.shape[0], h.shape[1], N.stream())
    return h


def layer_norm(x, w, b, eps=1e-5):
    if not _cuda(x):
        return R.layer_norm(x, w, b, eps)
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    y = torch.empty_like(x2)
    N.call("us_layer_norm", N.ptr(x2), N.ptr(w), N.ptr(b), N.ptr(y), x2.shape[0], x2.shape[1],
           eps, N.stream())
    return y.view(x.shape)


# ------------------------------------------------------------- rope + kv --
def qk_norm_rope_kv_(qkv, qw, kw, positions, inv_freq, slots, kcache, vcache, Hq, Hkv, D,
                     rot=None, interleaved=False, eps=1e-6):
    """Normalises and rotates the q and k heads of the fused projection output
    ``qkv [T, (Hq+2Hkv)*D]`` in place and writes k, v into the paged cache."""
    rot = D if rot is None else rot
    T = qkv.shape[0]
    if not _cuda(qkv):
        v3 = qkv.view(T, Hq + 2 * Hkv, D)
        q, k = R.qk_norm_rope(v3[:, :Hq], v3[:, Hq:Hq + Hkv], qw, kw, positions, inv_freq, rot,
                              interleaved, eps)
        v3[:, :Hq] = q
        v3[:, Hq:Hq + Hkv] = k
        if kcache is not None and slots is not None:
            R.kv_write(kcache, vcache, v3[:, Hq:Hq + Hkv], v3[:, Hq + Hkv:], slots)
        return qkv
    assert qkv.is_contiguous() and qkv.dtype == BF16
    N.call("us_qk_norm_rope_kv", N.ptr(qkv), N.ptr(qw), N.ptr(kw), N.ptr(positions),
           N.ptr(inv_freq), N.ptr(slots), N.ptr(kcache), N.ptr(vcache), T, Hq, Hkv, D, rot,
           int(interleaved), eps, N.stream())
    return qkv


def qk_norm_rope3_(q, k, qw, kw, coords, inv_freq, Hq, Hk, D, freqs_per_axis, eps=1e-6,
                   table=None):
    """Video transformer: per-head RMSNorm + three-axis rotary, in place.
    q [T, Hq*D] and k [T, Hk*D] may be column slices of a wider buffer."""
    T = q.shape[0]
    if not _cuda(q):
        qq, kk = R.qk_norm_rope3(q.reshape(T, Hq, D), k.reshape(T, Hk, D), qw, kw, coords,
                                 inv_freq, freqs_per_axis, eps)
        q.copy_(qq.reshape(T, Hq * D))
        k.copy_(kk.reshape(T, Hk * D))
        return q, k
    assert q.stride(1) == 1 and k.stride(1) == 1
    if table is not None:
        N.call("us_qk_norm_rope3_table", N.ptr(q), N.ptr(k), N.ptr(qw), N.ptr(kw), N.ptr(table),
               T, Hq, Hk, D, freqs_per_axis, q.stride(0), k.stride(0), eps, N.stream())
        return q, k
    N.call("us_qk_norm_rope3", N.ptr(q), N.ptr(k), N.ptr(qw), N.ptr(kw), N.ptr(coords),
           N.ptr(inv_freq), T, Hq, Hk, D, freqs_per_axis, q.stride(0), k.stride(0), eps,
           N.stream())
    return q, k


def rope3_table(coords, inv_freq):
    """(cos, sin) of every (row, axis, frequency): [T, 3 * F, 2] FP32, built once per
    request and read by ``qk_norm_rope3_`` instead of evaluating sincos per head."""
    ang = coords.t().float()[:, :, None] * inv_freq.float()[None, None, :]      # [T, 3, F]
    return torch.stack([ang.cos(), ang.sin()], -1).reshape(coords.shape[1], -1, 2).contiguous()


# -------------------------------------------------------------- attention --
import os as _os
DECODE_SIMT = _os.environ.get("US_DECODE_SIMT", "0") == "1"   # A/B switch: CUDA-core kernel


def decode_splits(B: int, Hkv: int, max_len: int, sm_count: int = 148) -> int:
    """Number of KV splits.  A CTA of the decode kernel has a fixed cost of several
    microseconds, so splits only pay while (sequence, kv head) pairs alone leave SMs idle:
    measured at 64 sequences x 1100 keys, 4 kv heads (256 pairs) run fastest unsplit
    (48 us against 58 us with two splits), 1 kv head (64 pairs) with three to four."""
    ctas = max(1, B * Hkv)
    want = max(1, 256 // ctas)
    by_len = max(1, max_len // 256)
    return int(max(1, min(want, by_len, 32)))


def decode_scratch(B: int, Hq: int, Hkv: int, D: int, splits: int, device):
    """(scratch bytes, arrival counters) for ``paged_decode_attention`` with its splits
    merged inside the kernel.  The counters start at zero and every call leaves them zero,
    so one pair serves every layer of a forward pass (calls ordered on the device)."""
    nbytes = N.kernels().us_paged_decode_scratch_bytes(B, Hq, D, max(1, splits))
    return (torch.empty(nbytes, dtype=torch.uint8, device=device),
            torch.zeros(B * Hkv, dtype=torch.int32, device=device))


# US_DECODE_PERSIST=0: bf16 pages go to the per-(sequence, kv head) kernel again (A/B switch)
DECODE_PERSIST = _os.environ.get("US_DECODE_PERSIST", "1") == "1"
PERSIST_SPLITS = 0      # ``splits`` value that selects the persistent kernel
PERSIST_MIN_PAIRS = int(_os.environ.get("US_DECODE_PERSIST_PAIRS", "148"))   # runner's threshold


def decode_persist_ok(B: int, Hq: int, Hkv: int, D: int, page_size: int, window: int,
                      fp8: bool = False) -> bool:
    """Whether the persistent decode-attention kernel serves this case (bf16 pages, head width
    128, pages dividing 128, no sliding window, at most 1024 sequences)."""
    return (DECODE_PERSIST and not DECODE_SIMT and not fp8 and D == 128 and 128 % page_size == 0
            and page_size >= 8 and Hq % Hkv == 0 and Hq // Hkv in (1, 2, 4, 8, 16)
            and not window and B <= 1024)


def decode_persist_scratch(B: int, Hkv: int, device):
    """(partial-output scratch, arrival counters) of the persistent decode-attention kernel:
    two slots per CTA, one counter per (sequence, kv head).  The counters start at zero and
    every call leaves them zero; calls that share the pair must be ordered on the device."""
    nbytes = N.kernels().us_paged_decode_persist_scratch_bytes()
    return (torch.empty(nbytes, dtype=torch.uint8, device=device),
            torch.zeros(B * Hkv, dtype=torch.int32, device=device))


def kv_write_scaled(k, v, slots, kcache, vcache, k_scale, v_scale):
    """Rows k, v [T, Hkv, D] (bf16, row-strided views allowed) into E4M3 pages (uint8
    [pages, page, Hkv, D]) with one FP32 scale per page and plane, derived by the write."""
    if not _cuda(k):
        return R.kv_write_scaled(kcache, vcache, k_scale, v_scale, k, v, slots)
    T, Hkv, D = k.shape
    assert k.dtype == BF16 and k.stride(2) == 1 and k.stride(1) == D and v.stride(1) == D
    assert kcache.dtype == torch.uint8 and k_scale.dtype == torch.float32
    N.call("us_kv_write_scaled", N.ptr(k), N.ptr(v), k.stride(0), v.stride(0), N.ptr(slots),
           N.ptr(kcache), N.ptr(vcache), N.ptr(k_scale), N.ptr(v_scale), T, kcache.shape[1], Hkv, D,
           N.stream())


def kv_gather(kcache, vcache, page_table, cu, total_rows, k_scale=None, v_scale=None, out=None,
              out_cu=None):
    """Cached rows of a batch as packed bf16: sequence s contributes its first
    cu[s + 1] - cu[s] cached positions (through ``page_table`` [B, max_pages]) to rows
    [cu[s], cu[s + 1]) of the result ([total_rows, Hkv, D] for K and for V), or to rows
    starting at ``out_cu[s]`` of a larger ``out``.  Pages are bf16, or E4M3 with scales.
    Nothing is read back to the host."""
    pages, page, Hkv, D = kcache.shape
    B = page_table.shape[0]
    if out is None:
        out = (torch.empty(total_rows, Hkv, D, dtype=BF16, device=kcache.device),
               torch.empty(total_rows, Hkv, D, dtype=BF16, device=kcache.device))
    ko, vo = out
    fp8 = k_scale is not None
    N.call("us_kv_gather", N.ptr(kcache), N.ptr(vcache), N.ptr(k_scale) if fp8 else None,
           N.ptr(v_scale) if fp8 else None, N.ptr(page_table), page_table.shape[1], N.ptr(cu),
           N.ptr(out_cu) if out_cu is not None else None, B, total_rows, page, Hkv, D, N.ptr(ko), N.ptr(vo), ko.stride(0), int(fp8), N.stream(),
           launches=1)
    return ko, vo


def paged_decode_attention(q, kcache, vcache, page_table, seq_lens, scale, splits=1, window=0,
                           out=None, scratch=None, Hq=None, D=None, counters=None, k_scale=None,
                           v_scale=None):
    """q: [B, Hq, D] (or a [B, >=Hq*D] row-strided view with Hq, D given);
    caches [pages, page_size, Hkv, D]; returns [B, Hq, D] bf16.  With ``counters`` (from
    ``decode_scratch``) the split merge happens inside the attention kernel.  With
    ``k_scale`` / ``v_scale`` [pages] the caches hold E4M3 bytes."""
    if not _cuda(q):
        return R.paged_decode_attention(q, kcache, vcache, page_table, seq_lens, scale, window,
                                        k_scale, v_scale)
    if q.dim() == 3:
        B, Hq, D = q.shape
        ldq = q.stride(0)
    else:
        B = q.shape[0]
        ldq = q.stride(0)
    pages, page_size, Hkv, _ = kcache.shape
    if out is None:
        out = torch.empty(B, Hq, D, dtype=BF16, device=q.device)
    ldo = out.stride(0)
    if splits > 1 and scratch is None:
        nbytes = N.kernels().us_paged_decode_scratch_bytes(B, Hq, D, splits)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    if k_scale is not None:
        splits = max(1, splits)
        if not (D == 128 and 128 % page_size == 0 and Hq // Hkv <= 16):
            raise ValueError("FP8 pages are served for head width 128, pages dividing 128 and "
                             "at most 16 query heads per key head")
        N.call("us_paged_decode_attention_fp8", N.ptr(q), N.ptr(kcache), N.ptr(vcache),
               N.ptr(k_scale), N.ptr(v_scale), N.ptr(page_table), N.ptr(seq_lens), N.ptr(out),
               N.ptr(scratch), N.ptr(counters) if counters is not None else None, B, Hq, Hkv, D,
               pages, page_table.shape[1], page_size, splits, window, scale, ldq, ldo, N.stream(),
               launches=1 if (counters is not None or splits == 1) else 2)
        return out
    if splits == PERSIST_SPLITS:
        # one CTA per SM over the launch's tile list (scratch / counters of decode_persist_scratch)
        if not decode_persist_ok(B, Hq, Hkv, D, page_size, window):
            raise ValueError("the persistent decode-attention kernel does not serve this case")
        if scratch is None or counters is None:
            scratch, counters = decode_persist_scratch(B, Hkv, q.device)
        N.call("us_paged_decode_attention_persist", N.ptr(q), N.ptr(kcache), N.ptr(vcache),
               N.ptr(page_table), N.ptr(seq_lens), N.ptr(out), N.ptr(scratch), N.ptr(counters),
               B, Hq, Hkv, D, pages, page_table.shape[1], page_size, scale, ldq, ldo, N.stream())
        return out
    if D == 128 and 128 % page_size == 0 and Hq // Hkv <= 16 and not DECODE_SIMT:
        # keys-on-M tcgen05 kernel
        if counters is not None:
            N.call("us_paged_decode_attention_tc_merged", N.ptr(q), N.ptr(kcache), N.ptr(vcache),
                   N.ptr(page_table), N.ptr(seq_lens), N.ptr(out), N.ptr(scratch),
                   N.ptr(counters), B, Hq, Hkv, D, pages, page_table.shape[1], page_size, splits,
                   window, scale, ldq, ldo, N.stream())
            return out
        N.call("us_paged_decode_attention_tc", N.ptr(q), N.ptr(kcache), N.ptr(vcache),
               N.ptr(page_table), N.ptr(seq_lens), N.ptr(out), N.ptr(scratch), B, Hq, Hkv, D,
               pages, page_table.shape[1], page_size, splits, window, scale, ldq, ldo,
               N.stream(), launches=2 if splits > 1 else 1)
        return out
    N.call("us_paged_decode_attention", N.ptr(q), N.ptr(kcache), N.ptr(vcache),
           N.ptr(page_table), N.ptr(seq_lens), N.ptr(out), N.ptr(scratch), B, Hq, Hkv, D,
           page_table.shape[1], page_size, splits, window, scale, ldq, ldo, N.stream(),
           launches=2 if splits > 1 else 1)
    return out


# ------------------------------------------------------------------ GEMMs --
# US_LINEAR_DECODE=0: projections of at most 64 rows go to the tcgen05 kernel as well
LINEAR_DECODE = _os.environ.get("US_LINEAR_DECODE", "1") == "1"
# weights up to this many elements take it (larger ones are bandwidth-bound: tcgen05 + TMA)
LINEAR_DECODE_MAX = int(_os.environ.get("US_LINEAR_DECODE_MAX", str(4 << 20)))


def _block_n(rows: int, dual: bool) -> int:
    for bn in (16, 32, 64, 128):
        if rows <= bn:
            return bn
    return 128 if dual else 256


def linear(x, w, bias=None, out_dtype=None, out=None, block_n=None):
    """y[rows, M] = x[rows, K] @ w[M, K]^T (+ bias).  bf16 operands, FP32
    accumulation in tensor memory, output bf16 or fp32."""
    out_dtype = out_dtype or x.dtype
    if not _cuda(x):
        return R.linear(x, w, bias, out_dtype)
    assert x.dtype == BF16 and w.dtype == BF16
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    if not w.is_contiguous():
        w = w.contiguous()
    if x2.shape[1] % 8:                       # TMA rows are 16-byte multiples: pad K with zeros
        padk = 8 - x2.shape[1] % 8
        x2 = torch.nn.functional.pad(x2, (0, padk))
        w = torch.nn.functional.pad(w, (0, padk))
    rows, K = x2.shape
    M = w.shape[0]
    if out is None:
        out = torch.empty(rows, M, dtype=out_dtype, device=x.device)
    if rows == 0:
        return out
    if LINEAR_DECODE and rows <= 64 and K % 256 == 0 and block_n is None and \
            M * K <= LINEAR_DECODE_MAX and \
            out.dtype in (BF16, torch.float32) and x2.data_ptr() % 16 == 0 and \
            w.data_ptr() % 16 == 0 and w.stride(0) % 8 == 0:
        # decode-size projection: weight-streaming kernel (latency-bound shape)
        N.call("us_linear_decode", N.ptr(w), N.ptr(x2), N.ptr(out), N.ptr(bias), rows, M, K,
               w.stride(0), x2.stride(0), out.stride(0), int(out.dtype == torch.float32),
               0 if (bias is None or bias.dtype == BF16) else 1, N.stream())
        return out.view(*x.shape[:-1], M)
    bn = block_n or _block_n(rows, False)
    N.call("us_gemm_wx", N.ptr(w), N.ptr(x2), N.ptr(out), 1, M, M, K, rows, w.stride(0),
           x2.stride(0), out.stride(0), 0, 0, 0, 0 if out.dtype == BF16 else 1, N.ptr(bias),
           0 if (bias is None or bias.dtype == BF16) else 1, None, None, None, None, None, None,
           0, bn, N.stream())
    return out.view(*x.shape[:-1], M)


_ACT = {"silu": 0, "silu_stepwise": 1, "gelu_tanh": 2}


def linear_gated(x, w, act="silu", stepwise=False, out=None, block_n=None):
    """w [2*I, K] stacks the `first` rows then the `second` (gate) rows;
    returns first * act(second) as [rows, I] bf16, fused in the GEMM epilogue."""
    if not _cuda(x):
        return R.linear_gated(x, w, act, stepwise)
    x2 = x.reshape(-1, x.shape[-1])
    rows, K = x2.shape
    I2 = w.shape[0]
    I_ = I2 // 2
    if out is None:
        out = torch.empty(rows, I_, dtype=BF16, device=x.device)
    if rows == 0:
        return out
    bn = block_n or _block_n(rows, True)
    code = _ACT["silu_stepwise" if (act == "silu" and stepwise) else act]
    N.call("us_gemm_wx", N.ptr(w), N.ptr(x2), N.ptr(out), 1, I2, I_, K, rows, w.stride(0),
           x2.stride(0), out.stride(0), 1, I_, code, 0, None, 0, None, None, None, None, None,
           None, 0, bn, N.stream())
    return out


# -------------------------------------------------------------------- MoE --
def topk_softmax(logits, top_k, renorm=True, live=None, expert_map=None, load=None,
                 ids=None, weights=None):
    if not _cuda(logits):
        return R.topk_softmax(logits, top_k, renorm)
    T, E = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    if ids is None:
        ids = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
        weights = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    N.call("us_topk_softmax", N.ptr(logits), N.ptr(ids), N.ptr(weights), T, E, top_k,
           int(renorm), N.ptr(live), N.ptr(expert_map), N.ptr(load), N.stream())
    return ids, weights


# rows per local expert from which the grouped expert GEMMs take 256-row tiles on the CTA-pair
# kernel (US_MOE_PAIR_ROWS; a huge value keeps the single-CTA kernel)
MOE_PAIR_MIN_ROWS = int(_os.environ.get("US_MOE_PAIR_ROWS", "64"))


@dataclass
class MoeWorkspace:
    """Static buffers of one MoE layer invocation (shared by all layers)."""
    sorted_route: torch.Tensor
    perm_of_route: torch.Tensor
    expert_offsets: torch.Tensor
    tile_group: torch.Tensor
    tile_row0: torch.Tensor
    tile_rows: torch.Tensor
    num_tiles: torch.Tensor
    xp: torch.Tensor      # [R, H] permuted activations
    h: torch.Tensor       # [R, I]
    y: torch.Tensor       # [R, H]
    block_n: int
    max_tiles: int
    sync: Optional[torch.Tensor] = None   # grid-wide counters of the fused route kernel
    live_tiles: int = 0                   # expected number of non-empty row tiles

    @staticmethod
    def create(T, top_k, E_local, H, I, device, block_n=None, E_total=None):
        """``E_total``: experts of the whole model when this rank holds only ``E_local`` of
        them (the routes then spread over all ranks; sizes the expected live tiles)."""
        R_ = T * top_k
        if block_n is None:
            avg = max(1, R_ // max(1, E_local))
            block_n = 16 if avg <= 16 else 32 if avg <= 32 else 64 if avg <= 64 else 128
            # prefill-size batches (a few hundred rows per expert): 256-row tiles on CTA pairs
            if R_ // max(1, E_total or E_local) >= MOE_PAIR_MIN_ROWS:
                block_n = 256
        max_tiles = min(R_, E_local) + R_ // block_n + 1
        i32 = dict(dtype=torch.int32, device=device)
        return MoeWorkspace(
            sorted_route=torch.zeros(R_, **i32), perm_of_route=torch.zeros(R_, **i32),
            expert_offsets=torch.zeros(E_local + 1, **i32),
            tile_group=torch.zeros(max_tiles, **i32), tile_row0=torch.zeros(max_tiles, **i32),
            tile_rows=torch.zeros(max_tiles, **i32), num_tiles=torch.zeros(1, **i32),
            xp=torch.zeros(R_ + 256, H, dtype=BF16, device=device)[:R_],
            h=torch.zeros(R_ + 256, I, dtype=BF16, device=device)[:R_],
            y=torch.empty(R_, H, dtype=BF16, device=device),
            block_n=block_n, max_tiles=max_tiles, sync=torch.zeros(4, **i32),
            live_tiles=MoeWorkspace._expected_tiles(R_, E_local, E_total or E_local, block_n))

    @staticmethod
    def _expected_tiles(R_, E_local, E_total, block_n) -> int:
        if E_local <= 0:
            return 0
        per = R_ / max(1, E_total)                        # mean routes per expert
        hit = E_local * (1.0 - math.exp(-per))            # experts with at least one route
        return max(1, int(math.ceil(hit + E_local * per / block_n)))


def route_and_sort(logits, top_k, renorm, ws, e_lo, E_local):
    """``topk_softmax`` and the route sort of ``moe_experts`` in one launch (at most 512
    tokens); the workspace is then passed to ``moe_experts(..., presorted=True)``."""
    T, E_all = logits.shape
    ids = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    weights = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    N.call("us_route_sort", N.ptr(logits), N.ptr(ids), N.ptr(weights), T, E_all, top_k,
           int(renorm), None, e_lo, E_local, ws.block_n, ws.max_tiles, N.ptr(ws.sorted_route),
           N.ptr(ws.perm_of_route), N.ptr(ws.expert_offsets), N.ptr(ws.tile_group),
           N.ptr(ws.tile_row0), N.ptr(ws.tile_rows), N.ptr(ws.num_tiles), N.stream())
    return ids, weights


def route_sort_gather(logits, x, top_k, renorm, ws, e_lo, E_local, live=None):
    """``topk_softmax``, the route sort and the row gather of ``moe_experts`` in one launch
    (at most 512 tokens); pass the workspace on with ``moe_experts(..., pregathered=True)``."""
    T, E_all = logits.shape
    ids = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    weights = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    N.call("us_route_sort_gather", N.ptr(logits), N.ptr(ids), N.ptr(weights), T, E_all, top_k,
           int(renorm), N.ptr(live), e_lo, E_local, ws.block_n, ws.max_tiles,
           N.ptr(ws.sorted_route), N.ptr(ws.perm_of_route), N.ptr(ws.expert_offsets),
           N.ptr(ws.tile_group), N.ptr(ws.tile_row0), N.ptr(ws.tile_rows), N.ptr(ws.num_tiles),
           N.ptr(x), x.shape[1], N.ptr(ws.xp), N.ptr(ws.sync), N.stream())
    return ids, weights


def unpermute_add_rmsnorm(y_perm, perm, weights, residual, w, eps=1e-6):
    """The weighted un-permute of the expert rows, the residual add and the RMSNorm of the
    next block in one launch: returns (normed bf16 [T, H], FP32 residual)."""
    T, top_k = perm.shape
    H = w.shape[0]
    first = residual is None
    if first:
        residual = torch.empty(T, H, dtype=torch.float32, device=y_perm.device)
    y = torch.empty(T, H, dtype=BF16, device=y_perm.device)
    N.call("us_unpermute_add_rmsnorm", N.ptr(y_perm), N.ptr(perm), N.ptr(weights), T, top_k, H,
           N.ptr(residual), N.ptr(w), N.ptr(y), eps, int(first), N.stream())
    return y, residual


def moe_experts(x, ids, weights, w13, w2, e_lo=0, act="silu", stepwise=False, ws=None, out=None,
                presorted=False, pregathered=False, defer_unpermute=False):
    """Routed experts: sort routes by local expert, gather rows, grouped FC1 with
    the gated activation fused, grouped FC2, weighted un-permute (FP32, one
    rounding).  w13 [E,2I,H] (first/up rows, then gate rows), w2 [E,H,I].
    ``pregathered``: ``route_sort_gather`` already filled the workspace.
    ``defer_unpermute``: returns (expert rows [R, H], perm [T, top_k]) for a consumer that
    forms the weighted sum itself (``unpermute_add_rmsnorm``, the fused all-reduce)."""
    if not _cuda(x):
        return R.moe_experts(x, ids, weights, w13, w2, e_lo, act, stepwise)
    T, H = x.shape
    top_k = ids.shape[1]
    E, I2, _ = w13.shape
    I_ = I2 // 2
    if ws is None:
        ws = MoeWorkspace.create(T, top_k, E, H, I_, x.device)
    R_ = T * top_k
    st = N.stream()
    if not presorted and not pregathered:
        N.call("us_moe_sort", N.ptr(ids), R_, e_lo, E, ws.block_n, ws.max_tiles,
               N.ptr(ws.sorted_route), N.ptr(ws.perm_of_route), N.ptr(ws.expert_offsets),
               N.ptr(ws.tile_group), N.ptr(ws.tile_row0), N.ptr(ws.tile_rows),
               N.ptr(ws.num_tiles), st)
    if not pregathered:
        total = ws.expert_offsets[E:]
        N.call("us_moe_gather", N.ptr(x), N.ptr(ws.sorted_route), N.ptr(total), R_, top_k, H,
               N.ptr(ws.xp), st)
    code = _ACT["silu_stepwise" if (act == "silu" and stepwise) else act]
    # FC1: [R, H] x [E, 2I, H] -> [R, I] with first * act(gate)
    live = ws.live_tiles
    if live:
        N.kernels().us_gemm_wx_hint(live * ((I_ + 127) // 128))
    N.call("us_gemm_wx", N.ptr(w13), N.ptr(ws.xp), N.ptr(ws.h), E, I2, I_, H, R_, H, H, I_, 1, I_,
           code, 0, None, 0, None, None, N.ptr(ws.tile_group), N.ptr(ws.tile_row0),
           N.ptr(ws.tile_rows), N.ptr(ws.num_tiles), ws.max_tiles, ws.block_n, st)
    # FC2: [R, I] x [E, H, I] -> [R, H]
    if live:
        N.kernels().us_gemm_wx_hint(live * ((H + 127) // 128))
    N.call("us_gemm_wx", N.ptr(w2), N.ptr(ws.h), N.ptr(ws.y), E, H, H, I_, R_, I_, I_, H, 0, 0, 0,
           0, None, 0, None, None, N.ptr(ws.tile_group), N.ptr(ws.tile_row0), N.ptr(ws.tile_rows),
           N.ptr(ws.num_tiles), ws.max_tiles, ws.block_n, st)
    if defer_unpermute:
        return ws.y, ws.perm_of_route.view(T, top_k)
    if out is None:
        out = torch.empty(T, H, dtype=BF16, device=x.device)
    N.call("us_moe_unpermute", N.ptr(ws.y), N.ptr(ws.perm_of_route), N.ptr(weights), T, top_k, H,
           N.ptr(out), st)
    return out


# --------------------------------------------------------------- sampling --
def argmax(logits, out=None):
    if not _cuda(logits):
        return R.argmax(logits)
    B, V = logits.shape
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    N.call("us_argmax", N.ptr(logits), B, V, logits.stride(0), N.ptr(out), N.stream())
    return out


def logits_shape_(logits, ban_mask=None, bias_csr=None, out_counts=None, prompt_mask=None,
                  rep=None, freq=None, pres=None, temp=None):
    """In place on FP32 logits.  bias_csr = (offsets[B+1] i32, ids i32, vals f32)."""
    B, V = logits.shape
    bo, bi, bv = bias_csr if bias_csr is not None else (None, None, None)
    N.call("us_logits_shape", N.ptr(logits), B, V, logits.stride(0), N.ptr(ban_mask), N.ptr(bo),
           N.ptr(bi), N.ptr(bv), N.ptr(out_counts), N.ptr(prompt_mask), N.ptr(rep), N.ptr(freq),
           N.ptr(pres), N.ptr(temp), N.stream(), launches=2 if bo is not None else 1)
    return logits


def sample_from_logits(logits, top_k, top_p, min_p, seeds, positions, out=None):
    """top_k i32 [B], top_p/min_p f32 [B], seeds u64-as-i64 [B], positions i64 [B]."""
    if not _cuda(logits):
        return R.sample_from_logits(logits, top_k, top_p, min_p, seeds, positions)
    B, V = logits.shape
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    N.call("us_sample_from_logits", N.ptr(logits), B, V, logits.stride(0), N.ptr(top_k),
           N.ptr(top_p), N.ptr(min_p), N.ptr(seeds), N.ptr(positions), N.ptr(out), N.stream())
    return out


def logprob_stats(logits, chosen):
    if not _cuda(logits):
        return R.logprob_stats(logits, chosen)
    B, V = logits.shape
    dev = logits.device
    lse = torch.empty(B, dtype=torch.float32, device=dev)
    lp = torch.empty(B, dtype=torch.float32, device=dev)
    rank = torch.empty(B, dtype=torch.int32, device=dev)
    N.call("us_logprob_stats", N.ptr(logits), B, V, logits.stride(0), N.ptr(chosen), N.ptr(lse),
           N.ptr(lp), N.ptr(rank), N.stream())
    return lse, lp, rank


# ------------------------------------------------------------------- misc --
def embedding(ids, table, vocab_lo=0, vocab_hi=None, out=None):
    vocab_hi = vocab_lo + table.shape[0] if vocab_hi is None else vocab_hi
    if not _cuda(table):
        return R.embedding(ids, table, vocab_lo, vocab_hi)
    T = ids.shape[0]
    if out is None:
        out = torch.empty(T, table.shape[1], dtype=table.dtype, device=table.device)
    N.call("us_embedding", N.ptr(ids), N.ptr(table), T, table.shape[1], vocab_lo, vocab_hi,
           N.ptr(out), N.stream())
    return out


def gather_rows(src, idx, out=None):
    if not _cuda(src):
        ok = idx >= 0
        g = src[idx.clamp_min(0).long()]
        return g * ok[:, None].to(g.dtype)
    M = idx.shape[0]
    H = src.shape[1]
    if out is None:
        out = torch.empty(M, H, dtype=src.dtype, device=src.device)
    N.call("us_gather_rows", N.ptr(src), N.ptr(idx), M, H, src.stride(0), N.ptr(out), N.stream())
    return out


def decode_advance_(sampled, input_ids, positions, seq_lens, slots, page_table, page_size,
                    live=None, history=None, step=None):
    B = sampled.shape[0]
    if not _cuda(sampled):
        n = B if live is None else int(live)
        input_ids[:n] = sampled[:n]
        positions[:n] += 1
        seq_lens[:n] = positions[:n] + 1
        pos = positions[:n].long()
        pg = page_table[torch.arange(n), pos // page_size]
        slots[:n] = pg * page_size + (pos % page_size).to(slots.dtype)
        slots[n:] = -1
        if history is not None and step is not None and int(step) < history.shape[0]:
            history[int(step)] = -1
            history[int(step), :n] = sampled[:n]
            step += 1
        return
    N.call("us_decode_advance", N.ptr(sampled), N.ptr(input_ids), N.ptr(positions),
           N.ptr(seq_lens), N.ptr(slots), N.ptr(page_table), page_table.shape[1], page_size, B,
           N.ptr(live), N.ptr(history), history.shape[1] if history is not None else 0,
           history.shape[0] if history is not None else 0,
           N.ptr(step), N.stream(), launches=2 if step is not None else 1)
