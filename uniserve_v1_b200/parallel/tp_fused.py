"""Tensor parallelism with the collectives fused into the GEMMs.

The residual stream is kept sequence-parallel: every rank owns ``rows / P`` rows
of the FP32 residual and of the normalised activations.  Around it

* a **row-parallel** linear (attention output, MLP down) produces a partial sum
  of every row: its epilogue stores each tile into the slot of the rank that owns
  the rows (reduce-scatter as peer stores), and the owner sums the ``P`` slots in
  FP32 inside the residual-add + RMSNorm kernel that follows anyway;
* that same kernel stores the normalised rows into *every* rank's copy of the
  gathered activations (all-gather as peer stores from the producer), so the
  **column-parallel** linear that follows (QKV, MLP up/gate) is a local GEMM over
  all rows.  Each row crosses NVLink once per peer.  (A GEMM that instead pulls the
  peers' rows through its operand loads exists as ``us_gemm_wx_gather``; peer
  memory is not cached in the local L2, so every weight tile re-fetched its
  activation tile over NVLink, and the producer-side form replaced it.)

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
    "us_reduce_slots_add_rmsnorm": (N.I, [N.P, N.I, N.P, N.P, N.P, N.I, N.I, N.I, N.L, N.F, N.I,
                                          N.P]),
    "us_push_rows_to_slots": (N.I, [N.P, N.L, N.P, N.I, N.I, N.I, N.I, N.I, N.P]),
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
        self.rows_max = rows_all
        self.fc = FusedComm(group, rank, world, device, hidden=0, sites=7,
                            site_bytes=rows_all * hidden * 2)
        self._ptrs = {}
        self.set_rows(rows_all)
        self._flip = 0

    def set_rows(self, rows: int) -> None:
        """The row count of the calls that follow (a multiple of 16 x world, at most the count
        the heap was sized for).  Rank r owns rows [r * rows / P, (r + 1) * rows / P)."""
        assert rows % (16 * self.P) == 0 and rows <= self.rows_max, (rows, self.rows_max)
        self.rows, self.ro = rows, rows // self.P
        self.bn = _row_block(self.ro)
        self.calls += 1

    calls = 0

    @staticmethod
    def padded(rows: int, world: int) -> int:
        unit = 16 * world
        return (rows + unit - 1) // unit * unit

    def barrier(self) -> None:
        """The next of the two barrier sites in turn (a site's flags may be reused only after
        another site's barrier was crossed)."""
        self.fc.barrier(SITE_B0 if self._flip == 0 else SITE_B1)
        self._flip ^= 1

    def push_rows(self, x: torch.Tensor) -> None:
        """Partial rows [rows, hidden] (bf16, any row stride) into the owners' slot of this
        rank: the reduce-scatter of a partial sum that did not come out of a GEMM."""
        assert x.shape[0] == self.rows and x.shape[1] == self.H and x.stride(1) == 1
        N.call("us_push_rows_to_slots", N.ptr(x), x.stride(0), self.ptrs(SITE_SLOTS), self.P,
               self.rows, self.H, self.ro, self.rank, N.stream())

    def close(self):
        self.fc.close()

    def ptrs(self, site: int):
        arr = self._ptrs.get(site)
        if arr is None:
            arr = (ctypes.c_void_p * self.P)(*[self.fc.peer_site_ptr(r, site)
                                               for r in range(self.P)])
            self._ptrs[site] = arr
        return arr

    def gathered(self, site: int) -> torch.Tensor:
        """This rank's copy of the gathered normalised rows [rows, hidden] in the heap."""
        return self.fc.site_tensor(site, self.rows, self.H)

    def own_rows(self, site: int) -> torch.Tensor:
        return self.gathered(site)[self.rank * self.ro:(self.rank + 1) * self.ro]

    def _own_row_ptrs(self, site: int):
        """Address of this rank's row interval inside every rank's gathered buffer."""
        key = ("rows", site, self.ro)
        arr = self._ptrs.get(key)
        if arr is None:
            off = self.rank * self.ro * self.H * 2
            arr = (ctypes.c_void_p * self.P)(*[self.fc.peer_site_ptr(r, site) + off
                                               for r in range(self.P)])
            self._ptrs[key] = arr
        return arr

    # ------------------------------------------------------------------ GEMMs --
    def gather_linear(self, w: torch.Tensor, site: int, gated: bool = False,
                      act: str = "silu") -> torch.Tensor:
        """y[rows, M] = (all ranks' normalised rows) @ w.T with this rank's weight shard
        ``w`` [M, hidden] (or [2M, hidden] value-then-gate when ``gated``); the rows were
        gathered by their producers, so this is a local GEMM."""
        x = self.gathered(site)
        return F.linear_gated(x, w, act=act) if gated else F.linear(x, w)

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
        """residual(own rows) += sum of the slots; the normalised rows are stored into
        every rank's gathered buffer ``out_site``.  Returns this rank's view of its rows."""
        slots = self.fc.site_tensor(SITE_SLOTS, self.P * self.ro, self.H)
        N.call("us_reduce_slots_add_rmsnorm", N.ptr(slots), self.P, N.ptr(residual), N.ptr(w),
               self._own_row_ptrs(out_site), self.P, self.ro, self.H, self.H, eps,
               1 if first else 0, N.stream())
        return self.own_rows(out_site)

    # ----------------------------------------------------------------- blocks --
    def mlp(self, residual: torch.Tensor, in_site: int, w13: torch.Tensor, w2: torch.Tensor,
            next_norm_w: torch.Tensor, out_site: int, eps: float) -> torch.Tensor:
        """Gated MLP over the gathered normalised rows in ``in_site``; leaves the updated
        residual (own rows) and the next normalised rows, gathered, in ``out_site``."""
        self.fc.barrier(SITE_B0)                      # everyone's rows have arrived here
        hidden = self.gather_linear(w13, in_site, gated=True)
        self.reduce_scatter_linear(w2, hidden)
        self.fc.barrier(SITE_B1)                      # every partial has landed
        return self.reduce_add_rmsnorm(residual, next_norm_w, out_site, eps)


def attach_fused_tp(model, rows_max: int = 8192):
    """Gives a tensor-parallel model the heap of its fused prefill path (collective: every rank
    of the tensor group calls it).  ``rows_max``: the largest prefill chunk."""
    ctx = model.ctx
    if ctx.tp_size <= 1 or model.device.type != "cuda" or model.pp != 1:
        return None
    ax = ctx.axis("tensor")
    model.tp_fused = FusedTP(ax.group, ax.rank, ax.size, model.device,
                             FusedTP.padded(rows_max, ax.size), model.cfg.hidden_size)
    return model.tp_fused
