"""Symmetric peer-memory heap and the collectives fused into their consumers.

One process per GPU.  Each rank allocates a heap, the ranks trade CUDA IPC
handles through ``torch.distributed`` (plumbing only) and map each other's heap;
from then on the data path is the hand-written kernels of
``csrc/fused/peer_comm.cu``: peer loads/stores over NVLink plus system-scope
flags, no NCCL call.  The reference's equivalent mechanism is its own
``alltoall`` expert-exchange transport (VMM windows + P2P ld/st + release/acquire
flags; crates/ops/kernels/expert_exchange/alltoall/src/exchange.cu:16-31,
reference project path); its tensor-parallel sums go through NCCL.

A *site* is a collective call position of one forward pass; ``begin_forward``
resets the site cursor, every fused collective takes the next site.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import native as N

N.register_signatures({
    "us_symm_create": (N.I, [N.I, N.I, N.I, N.L, N.P]),
    "us_symm_attach": (N.I, [N.P]),
    "us_symm_destroy": (N.I, []),
    "us_symm_site_ptr": (N.P, [N.I]),
    "us_symm_site_bytes": (N.L, []),
    "us_allreduce_add_rmsnorm": (N.I, [N.I, N.P, N.P, N.P, N.I, N.I, N.F, N.I, N.P]),
    "us_symm_allreduce": (N.I, [N.I, N.P, N.L, N.I, N.P]),
    "us_symm_allgather": (N.I, [N.I, N.P, N.L, N.P]),
    "us_symm_peer_site_ptr": (N.P, [N.I, N.I]),
    "us_symm_barrier": (N.I, [N.I, N.P]),
})


class _DevBuf:
    """Exposes a raw device pointer through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1",
                                         "data": (ptr, False), "version": 2}


class FusedComm:
    MAX_ROWS = 256

    def __init__(self, group, rank: int, world: int, device, hidden: int, sites: int = 256,
                 max_rows: int = 256, site_bytes: int = 0):
        self.group, self.rank, self.world = group, rank, world
        self.device = torch.device(device)
        self.sites = sites
        self.max_rows = min(max_rows, self.MAX_ROWS)
        self.site_bytes = ((site_bytes or self.max_rows * hidden * 4) + 255) & ~255
        self.cursor = 0
        lib = N.kernels()
        handle = (ctypes.c_ubyte * 64)()
        N.check(lib.us_symm_create(world, rank, sites, self.site_bytes, handle), "us_symm_create")
        mine = bytes(handle)
        if world > 1:
            gathered = [None] * world
            dist.all_gather_object(gathered, mine, group=group)
            blob = b"".join(gathered)
            buf = (ctypes.c_ubyte * len(blob)).from_buffer_copy(blob)
            N.check(lib.us_symm_attach(buf), "us_symm_attach")
            dist.barrier(group=group)
        self._views = {}

    def close(self):
        N.kernels().us_symm_destroy()

    # ------------------------------------------------------------------ sites --
    def begin_forward(self) -> None:
        self.cursor = 0

    def next_site(self) -> int:
        s = self.cursor
        self.cursor += 1
        if self.cursor > self.sites:
            raise RuntimeError("forward pass uses more collective sites than the heap holds")
        return s

    def site_tensor(self, site: int, rows: int, cols: int, dtype=torch.bfloat16) -> torch.Tensor:
        """This rank's buffer of ``site`` viewed as [rows, cols]; producers write here."""
        key = (site, rows, cols, dtype)
        t = self._views.get(key)
        if t is None:
            nbytes = rows * cols * torch.empty(0, dtype=dtype).element_size()
            assert nbytes <= self.site_bytes, (nbytes, self.site_bytes)
            ptr = N.kernels().us_symm_site_ptr(site)
            raw = torch.as_tensor(_DevBuf(ptr, nbytes), device=self.device)
            t = raw.view(dtype).view(rows, cols)
            self._views[key] = t
        return t

    def peer_site_ptr(self, rank: int, site: int) -> int:
        """Address (in this process) of ``rank``'s buffer of ``site``."""
        return N.kernels().us_symm_peer_site_ptr(rank, site)

    def barrier(self, site: int) -> None:
        """Stream-ordered group barrier (flags over peer memory, bounded wait)."""
        N.call("us_symm_barrier", site, N.stream())

    def fits(self, rows: int, cols: int, elem: int = 2) -> bool:
        return rows <= self.max_rows and rows * cols * elem <= self.site_bytes

    # ------------------------------------------------------------- collectives --
    def allreduce_add_rmsnorm(self, site: int, rows: int, residual, w, eps: float):
        """Sums the partial rows every rank wrote into ``site``, adds them to the
        FP32 residual stream (``residual=None`` starts it) and normalises."""
        H = w.shape[0]
        first = residual is None
        if first:
            residual = torch.empty(rows, H, dtype=torch.float32, device=self.device)
        y = torch.empty(rows, H, dtype=torch.bfloat16, device=self.device)
        N.call("us_allreduce_add_rmsnorm", site, N.ptr(residual), N.ptr(w), N.ptr(y), rows, H, eps,
               int(first), N.stream())
        return y, residual

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Generic sum over the group (copies x into a site first)."""
        if not self.fits(x.shape[0] if x.dim() > 1 else 1, x.shape[-1], x.element_size()) \
                or (x.numel() * x.element_size()) % 16:
            dist.all_reduce(x, group=self.group)
            return x
        site = self.next_site()
        buf = self.site_tensor(site, x.numel(), 1, x.dtype)
        buf.view(-1).copy_(x.reshape(-1))
        out = torch.empty_like(x)
        N.call("us_symm_allreduce", site, N.ptr(out), x.numel() * x.element_size(),
               int(x.dtype == torch.float32), N.stream())
        return out


def attach_fused(ctx, device, hidden: int = 2048, sites: int = 256) -> FusedComm:
    """Creates the heap over the context's tensor group and hooks it in."""
    ax = ctx.axis("tensor")
    fc = FusedComm(ax.group, ax.rank, ax.size, device, hidden, sites)
    ctx.fused = fc
    return fc
