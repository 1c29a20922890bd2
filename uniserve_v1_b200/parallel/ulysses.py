"""Ulysses sequence parallelism with the all-to-alls fused into the GEMMs.

Out: the QKV projection GEMM stores each output tile straight into the buffer of
the rank that owns those heads (peer stores from the epilogue), so the
"rows -> heads" all-to-all and its pack/unpack copies do not exist as separate
steps.  Back: the flash-attention epilogue stores every output row into the
buffer of the rank that owns the row, at the columns of the producing rank's
heads, so the "heads -> rows" all-to-all rides on the attention kernel and
``to_out`` is a local GEMM.  (A ``to_out`` that pulls its K slices from the
peers with TMA exists as ``us_gemm_wx_pull``; peer memory is not cached in the
local L2, so every weight tile re-fetched its activation tile over NVLink and the
push form replaced it.)  Two flag barriers per block order the phases; buffers
live in the symmetric heap.

Baseline for comparison is ``H3Transformer._attention`` with NCCL ``all_to_all``
(reference: crates/nn/src/modules/ulysses.rs:264-307, :348-388, reference
project paths).
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import functional as F
from ..ops import native as N
from ..ops.flash import flash_attn_varlen
from .symm import FusedComm

N.register_signatures({
    "us_gemm_wx_scatter": (N.I, [N.P, N.P, N.I, N.I, N.I, N.L, N.L, N.L, N.P, N.I, N.I, N.I, N.P]),
    "us_flash_attn_push": (N.I, [N.P, N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.L, N.L, N.L, N.F,
                                 N.P, N.I, N.I, N.I, N.L, N.P]),
    "us_gemm_wx_pull": (N.I, [N.P, N.P, N.I, N.I, N.P, N.I, N.I, N.I, N.L, N.L, N.L, N.I, N.I,
                              N.P]),
})

SITE_QKV, SITE_ATT, SITE_B1, SITE_B2 = 0, 1, 2, 3


class FusedUlysses:
    def __init__(self, ctx, device, rows_all: int, heads_local: int, head_dim: int):
        ax = ctx.axis("ulysses")
        self.P, self.rank = ax.size, ax.rank
        self.W = 3 * heads_local * head_dim
        site_bytes = rows_all * self.W * 2
        self.fc = FusedComm(ax.group, ax.rank, ax.size, device, hidden=0, sites=6,
                            site_bytes=site_bytes)
        self.rows_all = rows_all
        self._ptr_arrays = {}

    def close(self):
        self.fc.close()

    def _ptrs(self, site: int, byte_offset: int = 0):
        key = (site, byte_offset)
        arr = self._ptr_arrays.get(key)
        if arr is None:
            arr = (ctypes.c_void_p * self.P)(*[self.fc.peer_site_ptr(r, site) + byte_offset
                                               for r in range(self.P)])
            self._ptr_arrays[key] = arr
        return arr

    def attention(self, model, blk, n: torch.Tensor, layout) -> torch.Tensor:
        cfg = model.cfg
        P, hl, D, W = self.P, model.heads_local, cfg.head_dim, self.W
        rows, ro, H = layout.rows, layout.rows_own, cfg.hidden_size
        assert rows <= self.rows_all
        st = N.stream()
        bn = F._block_n(ro, False)
        # rows -> heads: projection tiles land in the owners' buffers
        with model._range("qkv_scatter"):
            N.call("us_gemm_wx_scatter", N.ptr(blk.qkv), N.ptr(n), P * W, H, ro, H, n.stride(0),
                   W, self._ptrs(SITE_QKV), W, self.rank * ro, bn, st)
        with model._range("barrier_1"):
            self.fc.barrier(SITE_B1)
        full = self.fc.site_tensor(SITE_QKV, rows, W)
        q, k, v = full[:, :hl * D], full[:, hl * D:2 * hl * D], full[:, 2 * hl * D:]
        with model._range("rope"):
            F.qk_norm_rope3_(q, k, blk.q_norm, blk.k_norm, layout.coords, model.inv_freq, hl, hl,
                             D, cfg.rope_freqs_per_axis, cfg.eps,
                             table=layout.rope_table(model.inv_freq))
        cu_q, cu_k = layout.cu(n.device)
        # heads -> rows: the attention epilogue stores every output row into the buffer of
        # the rank that owns it (columns of this rank's heads), so each row crosses NVLink
        # once and to_out reads local memory only
        inner = P * hl * D
        with model._range("flash"):
            N.call("us_flash_attn_push", N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(cu_q), N.ptr(cu_k),
                   rows, layout.used, hl, hl, full.stride(0), full.stride(0), full.stride(0),
                   model.scale, self._ptrs(SITE_ATT), P, ro, self.rank * hl * D, inner, st)
        with model._range("barrier_2"):
            self.fc.barrier(SITE_B2)
        att = self.fc.site_tensor(SITE_ATT, ro, inner)
        with model._range("to_out"):
            out = F.linear(att, blk.to_out)
        return out
