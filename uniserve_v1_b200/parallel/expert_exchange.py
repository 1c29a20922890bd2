"""Expert-parallel token exchange (dispatch / combine) over peer memory.

Data-parallel attention + expert parallelism: every rank keeps its own tokens,
experts are whole on one rank.  Per MoE layer the source side routes and pushes
token rows into the expert ranks' windows (``route_dispatch``), the expert side
sorts what arrived and runs the grouped FC1 / FC2 where FC2's epilogue applies
the gate weight and stores each row into the token owner's combine buffer, and
the owner's next norm sums the k rows (``combine_add_rmsnorm``).  With disjoint
``source_ranks`` / ``expert_ranks`` the same exchange is the attention-FFN
disaggregated layout.  Steps are lock-step: every rank takes part in every layer
of every step (idle ranks join with zero live tokens).

Reference behaviour: docs/expert_parallelism.md:5-31, :58-85;
crates/engine/src/runner/causal_lm/experts.rs:377-460 (reference project paths).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import functional as F
from ..ops import native as N

N.register_signatures({
    "us_ep_create": (N.I, [N.I, N.I, N.I, N.I, N.I, N.P, N.P]),
    "us_ep_attach": (N.I, [N.P, N.P]),
    "us_ep_destroy": (N.I, [N.P]),
    "us_ep_window": (N.P, [N.P, N.I]),
    "us_ep_peer_recv": (N.P, [N.P, N.I]),
    "us_ep_route_dispatch": (N.I, [N.P, N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.P]),
    "us_ep_wait": (N.I, [N.P, N.I, N.I, N.I, N.P]),
    "us_ep_signal_combined": (N.I, [N.P, N.I, N.I, N.P]),
    "us_ep_combine_add_rmsnorm": (N.I, [N.P, N.P, N.P, N.P, N.P, N.P, N.I, N.F, N.I, N.I, N.P]),
    "us_gemm_fp8_block_route_push": (N.I, [N.P, N.P, N.P, N.P, N.L, N.I, N.I, N.I, N.I, N.L, N.L,
                                           N.L, N.P, N.I, N.P, N.P, N.I, N.P, N.P, N.P, N.P, N.I,
                                           N.I, N.P]),
    "us_gemm_wx_route_push": (N.I, [N.P, N.P, N.I, N.I, N.I, N.I, N.L, N.L, N.L, N.P, N.I, N.P,
                                    N.P, N.I, N.P, N.P, N.P, N.P, N.I, N.I, N.P]),
})


class _DevBuf:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1",
                                         "data": (ptr, False), "version": 2}


class ExpertExchange:
    def __init__(self, group, rank: int, world: int, device, t_max: int, top_k: int, hidden: int,
                 num_experts: int, inter: int, source_ranks=None, expert_ranks=None):
        self.group, self.rank, self.world = group, rank, world
        self.device = torch.device(device)
        self.T, self.k, self.H, self.E, self.I = t_max, top_k, hidden, num_experts, inter
        self.source_ranks = tuple(source_ranks if source_ranks is not None else range(world))
        self.expert_ranks = tuple(expert_ranks if expert_ranks is not None else range(world))
        # both role sets are contiguous rank ranges
        assert list(self.source_ranks) == list(range(self.source_ranks[0], self.source_ranks[-1] + 1))
        assert list(self.expert_ranks) == list(range(self.expert_ranks[0], self.expert_ranks[-1] + 1))
        self.is_source = rank in self.source_ranks
        self.is_expert = rank in self.expert_ranks
        self.experts_per_rank = num_experts // len(self.expert_ranks)
        assert self.experts_per_rank * len(self.expert_ranks) == num_experts
        self.e_lo = (rank - self.expert_ranks[0]) * self.experts_per_rank if self.is_expert else 0
        lib = N.kernels()
        handle = (ctypes.c_ubyte * 64)()
        self.h = ctypes.c_void_p()      # this exchange's handle (a process may hold several)
        N.check(lib.us_ep_create(world, rank, t_max, top_k, hidden, handle, ctypes.byref(self.h)),
                "us_ep_create")
        if world > 1:
            gathered = [None] * world
            dist.all_gather_object(gathered, bytes(handle), group=group)
            blob = b"".join(gathered)
            buf = (ctypes.c_ubyte * len(blob)).from_buffer_copy(blob)
            N.check(lib.us_ep_attach(self.h, buf), "us_ep_attach")
            dist.barrier(group=group)
        R = world * t_max * top_k

        def view(which, nbytes, dtype, shape):
            raw = torch.as_tensor(_DevBuf(lib.us_ep_window(self.h, which), nbytes), device=self.device)
            return raw.view(dtype).view(*shape)

        self.win_x = view(0, world * t_max * hidden * 2, torch.bfloat16, (world * t_max, hidden))
        self.win_ids = view(1, R * 4, torch.int32, (world * t_max, top_k))
        self.win_w = view(2, R * 4, torch.float32, (R,))
        self.recv_ptrs = (ctypes.c_void_p * world)(*[lib.us_ep_peer_recv(self.h, r) for r in range(world)])
        self._ws = {}

    def workspace(self, t_step: int):
        """Sort / GEMM workspace for a step of ``t_step`` rows per source (the window
        stride of that step; the same on every rank, which run in lock step)."""
        ws = self._ws.get(t_step)
        if ws is None:
            ws = F.MoeWorkspace.create(self.world * t_step, self.k, self.experts_per_rank, self.H,
                                       self.I, self.device)
            if ws.block_n > 128:
                # FC2 pushes its rows to the token owners from the single-CTA grouped kernel's
                # epilogue: 128-row tiles (the 256-row tiles belong to the CTA-pair kernel)
                ws = F.MoeWorkspace.create(self.world * t_step, self.k, self.experts_per_rank,
                                           self.H, self.I, self.device, block_n=128)
            self._ws[t_step] = ws
        return ws

    def close(self):
        if self.h:
            N.kernels().us_ep_destroy(self.h)
            self.h = ctypes.c_void_p()

    # ------------------------------------------------------------- source side --
    def dispatch(self, x, ids, weights, live=None) -> None:
        """Pushes the rows of this rank's tokens to the ranks that own their experts."""
        T = x.shape[0]
        assert T <= self.T, f"step of {T} rows exceeds the exchange capacity {self.T}"
        N.call("us_ep_route_dispatch", self.h, N.ptr(x), N.ptr(ids), N.ptr(weights), N.ptr(live), T,
               self.experts_per_rank, self.expert_ranks[0], N.stream())

    def combine_add_rmsnorm(self, ids, live, residual, w, eps: float):
        T = ids.shape[0]
        y = torch.empty(T, self.H, dtype=torch.bfloat16, device=self.device)
        N.call("us_ep_combine_add_rmsnorm", self.h, N.ptr(ids), N.ptr(live), N.ptr(residual), N.ptr(w),
               N.ptr(y), T, eps, self.expert_ranks[0], self.expert_ranks[-1] + 1, N.stream())
        return y, residual

    # ------------------------------------------------------------- expert side --
    def experts(self, w13, w2, t_step: int, act: str = "silu") -> None:
        """Waits for every source's rows, runs the local experts over what arrived and
        pushes the weighted outputs to the token owners.  ``t_step`` is the row count
        per source of this step (the windows are laid out with that stride)."""
        ws, st = self.workspace(t_step), N.stream()
        E, I2, H = w13.shape
        I_ = I2 // 2
        R = self.world * t_step * self.k
        N.call("us_ep_wait", self.h, 0, self.source_ranks[0], self.source_ranks[-1] + 1, st)
        N.call("us_moe_sort", N.ptr(self.win_ids), R, self.e_lo, E, ws.block_n, ws.max_tiles,
               N.ptr(ws.sorted_route), N.ptr(ws.perm_of_route), N.ptr(ws.expert_offsets),
               N.ptr(ws.tile_group), N.ptr(ws.tile_row0), N.ptr(ws.tile_rows),
               N.ptr(ws.num_tiles), st)
        total = ws.expert_offsets[E:]
        N.call("us_moe_gather", N.ptr(self.win_x), N.ptr(ws.sorted_route), N.ptr(total), R, self.k,
               H, N.ptr(ws.xp), st)
        N.call("us_gemm_wx", N.ptr(w13), N.ptr(ws.xp), N.ptr(ws.h), E, I2, I_, H, R, H, H, I_, 1,
               I_, F._ACT[act], 0, None, 0, None, None, N.ptr(ws.tile_group), N.ptr(ws.tile_row0),
               N.ptr(ws.tile_rows), N.ptr(ws.num_tiles), ws.max_tiles, ws.block_n, st)
        N.call("us_gemm_wx_route_push", N.ptr(w2), N.ptr(ws.h), E, H, I_, R, I_, I_, H,
               self.recv_ptrs, self.world, N.ptr(ws.sorted_route), N.ptr(self.win_w),
               t_step * self.k, N.ptr(ws.tile_group), N.ptr(ws.tile_row0), N.ptr(ws.tile_rows),
               N.ptr(ws.num_tiles), ws.max_tiles, ws.block_n, st)
        N.call("us_ep_signal_combined", self.h, self.source_ranks[0], self.source_ranks[-1] + 1, st)

    def experts_fp8(self, ex, t_step: int, act: str = "silu") -> None:
        """``experts`` with block-scaled FP8 weights (``ops.fp8.Fp8Experts``): the rows
        that arrived are quantised per row and 128-wide K block before each grouped
        GEMM; FC2's epilogue pushes the weighted rows to the token owners."""
        from ..ops import fp8 as Q
        ws, st = self.workspace(t_step), N.stream()
        if ws.block_n > 64:
            ws = self._ws[t_step] = F.MoeWorkspace.create(
                self.world * t_step, self.k, self.experts_per_rank, self.H, self.I, self.device,
                block_n=64)
        E, I2, H = ex.w13.shape
        I_ = I2 // 2
        R = self.world * t_step * self.k
        q8 = getattr(ws, "_fp8", None)
        if q8 is None:
            z = lambda r, c: torch.zeros(r + Q.PAD_ROWS, c, dtype=torch.uint8,
                                         device=self.device)[:r]
            o = lambda kb, r: torch.ones(kb, r + Q.PAD_ROWS, dtype=torch.float32,
                                         device=self.device)
            q8 = ws._fp8 = dict(xq=z(R, H), xs=o(H // 128, R), hq=z(R, I_), hs=o(I_ // 128, R))
        N.call("us_ep_wait", self.h, 0, self.source_ranks[0], self.source_ranks[-1] + 1, st)
        N.call("us_moe_sort", N.ptr(self.win_ids), R, self.e_lo, E, ws.block_n, ws.max_tiles,
               N.ptr(ws.sorted_route), N.ptr(ws.perm_of_route), N.ptr(ws.expert_offsets),
               N.ptr(ws.tile_group), N.ptr(ws.tile_row0), N.ptr(ws.tile_rows),
               N.ptr(ws.num_tiles), st)
        total = ws.expert_offsets[E:]
        N.call("us_moe_gather", N.ptr(self.win_x), N.ptr(ws.sorted_route), N.ptr(total), R, self.k,
               H, N.ptr(ws.xp), st)
        Q.quantize_rows_block128(ws.xp, total, q8["xq"], q8["xs"])
        tiles = (N.ptr(ws.tile_group), N.ptr(ws.tile_row0), N.ptr(ws.tile_rows),
                 N.ptr(ws.num_tiles), ws.max_tiles, ws.block_n)
        N.call("us_gemm_fp8_block", N.ptr(ex.w13), N.ptr(ex.w13_scale), N.ptr(q8["xq"]),
               N.ptr(q8["xs"]), q8["xs"].stride(0), N.ptr(ws.h), E, I2, I_, H, R, H, H, I_, 1, I_,
               F._ACT[act], 0, None, None, *tiles, st)
        Q.quantize_rows_block128(ws.h, total, q8["hq"], q8["hs"])
        N.call("us_gemm_fp8_block_route_push", N.ptr(ex.w2), N.ptr(ex.w2_scale), N.ptr(q8["hq"]),
               N.ptr(q8["hs"]), q8["hs"].stride(0), E, H, I_, R, I_, I_, H, self.recv_ptrs,
               self.world, N.ptr(ws.sorted_route), N.ptr(self.win_w), t_step * self.k, *tiles, st)
        N.call("us_ep_signal_combined", self.h, self.source_ranks[0], self.source_ranks[-1] + 1, st)


class HostExpertExchange:
    """The same exchange for CPU ranks (gloo): the calls and their lock-step contract are
    those of ``ExpertExchange``; rows travel through host collectives.  It exists for the
    host-side logic (capacity agreement, idle-rank joins, disjoint attention / expert roles)
    to be tested without GPUs, and for CPU deployments of the tiny model.

    Per layer every rank takes part in two collectives, in this order: an all-gather of
    (rows, ids, weights) of ``t_step`` rows per rank, and an all-reduce of the experts'
    weighted output rows.  A source-only rank joins the first in ``dispatch`` and the second
    in ``combine_add_rmsnorm``; an expert-only rank does both in ``experts``; a rank with
    both roles gathers in ``experts`` (after its own ``dispatch`` stashed the rows)."""
    host = True

    def __init__(self, group, rank: int, world: int, t_max: int, top_k: int, hidden: int,
                 num_experts: int, source_ranks=None, expert_ranks=None):
        self.group, self.rank, self.world = group, rank, world
        self.T, self.k, self.H, self.E = t_max, top_k, hidden, num_experts
        self.source_ranks = tuple(source_ranks if source_ranks is not None else range(world))
        self.expert_ranks = tuple(expert_ranks if expert_ranks is not None else range(world))
        self.is_source = rank in self.source_ranks
        self.is_expert = rank in self.expert_ranks
        self.experts_per_rank = num_experts // len(self.expert_ranks)
        assert self.experts_per_rank * len(self.expert_ranks) == num_experts
        self.e_lo = (self.expert_ranks.index(rank)) * self.experts_per_rank if self.is_expert else 0
        self.device = torch.device("cpu")
        self._mine = None
        self._partial = None
        self.layers = 0

    def close(self):
        pass

    def _gather(self, t_step: int):
        x, ids, w = self._mine if self._mine is not None else (
            torch.zeros(t_step, self.H), torch.full((t_step, self.k), -1, dtype=torch.int32),
            torch.zeros(t_step, self.k))
        self._mine = None
        xs = [torch.empty_like(x) for _ in range(self.world)]
        is_ = [torch.empty_like(ids) for _ in range(self.world)]
        ws = [torch.empty_like(w) for _ in range(self.world)]
        dist.all_gather(xs, x.contiguous(), group=self.group)
        dist.all_gather(is_, ids.contiguous(), group=self.group)
        dist.all_gather(ws, w.contiguous(), group=self.group)
        return torch.cat(xs), torch.cat(is_), torch.cat(ws)

    def dispatch(self, x, ids, weights, live=None) -> None:
        T = x.shape[0]
        assert T <= self.T, f"step of {T} rows exceeds the exchange capacity {self.T}"
        ids, weights = ids.clone().to(torch.int32), weights.clone().float()
        if live is not None:
            n = int(live)
            ids[n:] = -1
            weights[n:] = 0
        self._mine = (x.float(), ids, weights)
        self._t = T
        if not self.is_expert:
            self._gather(T)             # source-only: joins the gather, keeps nothing

    def experts(self, w13, w2, t_step: int, act: str = "silu") -> None:
        from ..ops import reference as R
        # An expert-only rank joins the all-reduce of a layer's output when the source ranks
        # do: at THEIR next use of this exchange (their combine runs at the start of the next
        # layer, after the other micro-batch's collectives), so it is held back until this
        # exchange's next call, or ``flush`` at the end of the forward.
        self.flush()
        x, ids, w = self._gather(t_step)
        out = R.moe_experts(x, ids, w, w13.float(), w2.float(), e_lo=self.e_lo, act=act).float()
        self.layers += 1
        if self.is_source:
            self._partial = out
        else:
            self._held = out

    def flush(self) -> None:
        """Expert-only ranks: joins the all-reduce of the output held back by ``experts``."""
        held = getattr(self, "_held", None)
        if held is not None:
            self._held = None
            dist.all_reduce(held, group=self.group)     # nothing to keep

    def combine_add_rmsnorm(self, ids, live, residual, w, eps: float):
        from ..ops import reference as R
        T = ids.shape[0]
        out = self._partial if self._partial is not None else \
            torch.zeros(self.world * T, self.H)
        self._partial = None
        dist.all_reduce(out, group=self.group)
        mine = out[self.rank * T:(self.rank + 1) * T]
        return R.add_rmsnorm(mine.to(w.dtype), residual, w, eps)
