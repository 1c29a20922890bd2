"""Tensor parallelism with the collectives fused into the GEMMs.

The residual stream is kept sequence-parallel: every rank owns ``rows / P`` rows
of the FP32 residual and of the normalised activations.  Around it

* a **column-parallel** linear (QKV, MLP up/gate) reads the normalised rows of
  *all* ranks: the all-gather is the GEMM's own operand traffic (TMA loads from the
  peers' buffers, one tensor map per rank, no cluster multicast);
* a **row-parallel** linear (attention output, MLP down) produces a partial sum
  of every row: its epilogue stores each tile into the slot of the rank that owns
  the rows (reduce-scatter as peer stores), and the owner sums the ``P`` slots in
  FP32 inside the residual-add + RMSNorm kernel that follows anyway.

Two flag barriers per linear pair order the phases; buffers live in the
symmetric heap.  The unfused baseline is an NCCL all-reduce after every
row-parallel linear (reference: crates/nn/src/modules/linear.rs:650-695,
reference project path).
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import functional as F
from ..ops import native as N
from .symm import FusedComm

N.register_signatures({
    "us_gemm_wx_gather": (N.I, [N.P, N.P, N.I, N.I, N.P, N.I, N.I, N.I, N.I, N.L, N.L, N.L, N.I,
                                N.I, N.I, N.I, N.I, N.P]),
    "us_gemm_wx_reduce_scatter": (N.I, [N.P, N.P, N.I, N.I, N.I, N.L, N.L, N.L, N.P, N.I, N.I, N.I,
                                        N.I, N.I, N.P]),
    "us_reduce_slots_add_rmsnorm": (N.I, [N.P, N.I, N.P, N.P, N.P, N.I, N.I, N.L, N.F, N.I, N.P]),
})

SITE_NORM_A, SITE_NORM_B, SITE_SLOTS, SITE_B0, SITE_B1 = 0, 1, 2, 3, 4


def _row_block(rows_own: int) -> int:
    for bn in (256, 128, 64, 32, 16):
        if rows_own % bn == 0:
            return bn
    raise ValueError("rows per rank must be a multiple of 16")


class FusedTP:
    def __init__(self, group, rank: int, world: int, device, rows_all: int, hidden: int):
        assert rows_all % world == 0
        self.P, self.rank, self.H = world, rank, hidden
        self.rows, self.ro = rows_all, rows_all // world
        self.bn = _row_block(self.ro)
        self.fc = FusedComm(group, rank, world, device, hidden=0, sites=5,
                            site_bytes=world * self.ro * hidden * 2)
        self._ptrs = {}

    def close(self):
        self.fc.close()

    def ptrs(self, site: int):
        arr = self._ptrs.get(site)
        if arr is None:
            arr = (ctypes.c_void_p * self.P)(*[self.fc.peer_site_ptr(r, site)
                                               for r in range(self.P)])
            self._ptrs[site] = arr
        return arr

    def norm_rows(self, site: int) -> torch.Tensor:
        """This rank's normalised rows [rows_own, hidden] inside the heap."""
        return self.fc.site_tensor(site, self.ro, self.H)

    # ------------------------------------------------------------------ GEMMs --
    def gather_linear(self, w: torch.Tensor, site: int, gated: bool = False,
                      act: str = "silu") -> torch.Tensor:
        """y[rows, M] = concat_p(norm rows of rank p) @ w.T with this rank's weight
        shard ``w`` [M, hidden] (or [2M, hidden] value-then-gate when ``gated``)."""
        M = w.shape[0] // 2 if gated else w.shape[0]
        out = torch.empty(self.rows, M, dtype=torch.bfloat16, device=w.device)
        N.call("us_gemm_wx_gather", N.ptr(w), self.ptrs(site), self.P, self.ro, N.ptr(out),
               w.shape[0], M, self.H, self.rows, w.stride(0), self.H, M, 1 if gated else 0,
               M if gated else 0, F._ACT[act] if gated else 0, 0, self.bn, N.stream())
        return out

    def reduce_scatter_linear(self, w: torch.Tensor, x: torch.Tensor) -> None:
        """Partial product x @ w.T ([rows, hidden]) pushed row-interval-wise into the
        owners' slot buffers."""
        assert x.shape[0] == self.rows and w.shape[0] == self.H
        if not x.is_contiguous():
            x = x.contiguous()
        N.call("us_gemm_wx_reduce_scatter", N.ptr(w), N.ptr(x), self.H, x.shape[1], self.rows,
               w.stride(0), x.stride(0), self.H, self.ptrs(SITE_SLOTS), self.P, self.ro,
               self.rank, 0, self.bn, N.stream())

    def reduce_add_rmsnorm(self, residual: torch.Tensor, w: torch.Tensor, out_site: int,
                           eps: float, first: bool = False) -> torch.Tensor:
        """residual(own rows) += sum of the slots; the normalised rows go to ``out_site``."""
        y = self.norm_rows(out_site)
        slots = self.fc.site_tensor(SITE_SLOTS, self.P * self.ro, self.H)
        N.call("us_reduce_slots_add_rmsnorm", N.ptr(slots), self.P, N.ptr(residual), N.ptr(w),
               N.ptr(y), self.ro, self.H, self.H, eps, 1 if first else 0, N.stream())
        return y

    # ----------------------------------------------------------------- blocks --
    def mlp(self, residual: torch.Tensor, in_site: int, w13: torch.Tensor, w2: torch.Tensor,
            next_norm_w: torch.Tensor, out_site: int, eps: float) -> torch.Tensor:
        """Gated MLP over the normalised rows in ``in_site``; leaves the updated
        residual (own rows) and the next normalised rows in ``out_site``."""
        self.fc.barrier(SITE_B0)                      # everyone's rows are in place
        hidden = self.gather_linear(w13, in_site, gated=True)
        self.reduce_scatter_linear(w2, hidden)
        self.fc.barrier(SITE_B1)                      # every partial has landed
        return self.reduce_add_rmsnorm(residual, next_norm_w, out_site, eps)
