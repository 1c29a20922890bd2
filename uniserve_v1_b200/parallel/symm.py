"""Symmetric peer-memory heap and the collectives fused into their consumers.

One process per GPU.  Each rank allocates a heap, the ranks trade CUDA IPC
handles through ``torch.distributed`` (plumbing only) and map each other's heap;
from then on the data path is the hand-written kernels of
``csrc/fused/peer_comm.cu``: peer loads/stores over NVLink plus system-scope
flags, no NCCL call.  The reference's equivalent mechanism is its own
``alltoall`` expert-exchange transport (VMM windows + P2P ld/st + release/acquire
flags; crates/ops/kernels/expert_exchange/alltoall/src/exchange.cu:16-31,
reference project path); its tensor-parallel sums go through NCCL.

A *site* is a named buffer of the heap with its own flags; the decode-size collectives
take theirs from a small ring (``next_site``).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import native as N

N.register_signatures({
    "us_symm_create": (N.I, [N.I, N.I, N.I, N.L, N.P, N.P]),
    "us_symm_create_loopback": (N.I, [N.I, N.I, N.I, N.L, N.P]),
    "us_symm_attach": (N.I, [N.P, N.P]),
    "us_symm_destroy": (N.I, [N.P]),
    "us_symm_reset": (N.I, [N.P, N.P]),
    "us_symm_site_ptr": (N.P, [N.P, N.I]),
    "us_symm_site_bytes": (N.L, [N.P]),
    "us_symm_allreduce_add_rmsnorm": (N.I, [N.P, N.I, N.P, N.P, N.P, N.P, N.I, N.P, N.P, N.P, N.I,
                                            N.I, N.F, N.I, N.P]),
    "us_symm_argmax": (N.I, [N.P, N.I, N.P, N.L, N.I, N.I, N.I, N.P, N.P]),
    "us_symm_allreduce": (N.I, [N.P, N.I, N.P, N.L, N.I, N.P]),
    "us_symm_allgather": (N.I, [N.P, N.I, N.P, N.L, N.P]),
    "us_symm_peer_site_ptr": (N.P, [N.P, N.I, N.I]),
    "us_symm_barrier": (N.I, [N.P, N.I, N.P]),
    "us_set_peer_wait_clocks": (N.I, [N.L]),
    "us_status_copy_async": (N.I, [N.P, N.P]),
    "us_status_clear_async": (N.I, [N.P]),
})


class _DevBuf:
    """Exposes a raw device pointer through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1",
                                         "data": (ptr, False), "version": 2}


class FusedComm:
    """One symmetric heap over a process group.  A process may hold several (one per
    parallel axis).

    Sites ``0 .. sites - 3`` are handed out in a ring by ``next_site`` for the decode-size
    collectives; ``SITE_ARGMAX`` and ``SITE_AUX`` (the last two) are reserved.  Rules the
    kernels rely on, kept here:

    * every rank issues the same sequence of collectives with the same row counts (the
      flag protocol is per CTA index of a site);
    * the push-form all-reduce and the arg-max exchange double-buffer their slots by the
      parity of the device-side epoch, so they may reuse a site back to back;
    * the pull-form ``all_reduce`` has an arrival barrier only: its buffer may be
      rewritten only after another barrier was crossed, so a back-to-back reuse of its
      site gets a barrier on ``SITE_AUX`` first (``_guard_reuse``).
    """
    MAX_ROWS = 256

    def __init__(self, group, rank: int, world: int, device, hidden: int, sites: int = 10,
                 max_rows: int = 256, site_bytes: int = 0, loopback: bool = False):
        self.group, self.rank, self.world = group, rank, world
        self.device = torch.device(device)
        self.sites = sites
        self.max_rows = min(max_rows, self.MAX_ROWS)
        # a push-form site holds 2 (parity) x world slots of [max_rows, hidden] bf16
        self.site_bytes = ((site_bytes or 2 * world * self.max_rows * hidden * 2) + 255) & ~255
        self.ring = max(1, sites - 2)
        self.SITE_ARGMAX, self.SITE_AUX = sites - 2, sites - 1
        self.cursor = 0
        self._last_pull_site = None
        lib = N.kernels()
        self.h = ctypes.c_void_p()
        if loopback:
            N.check(lib.us_symm_create_loopback(world, rank, sites, self.site_bytes,
                                                ctypes.byref(self.h)), "us_symm_create_loopback")
        else:
            handle = (ctypes.c_ubyte * 64)()
            N.check(lib.us_symm_create(world, rank, sites, self.site_bytes, handle,
                                       ctypes.byref(self.h)), "us_symm_create")
            if world > 1:
                gathered = [None] * world
                dist.all_gather_object(gathered, bytes(handle), group=group)
                blob = b"".join(gathered)
                buf = (ctypes.c_ubyte * len(blob)).from_buffer_copy(blob)
                N.check(lib.us_symm_attach(self.h, buf), "us_symm_attach")
                dist.barrier(group=group)
        self._views = {}

    def close(self):
        if self.h:
            N.kernels().us_symm_destroy(self.h)
            self.h = ctypes.c_void_p()
            self._views = {}

    def reset(self) -> None:
        """Zeroes flags and epochs after a failed wait.  Collective on the host: every rank
        calls it with none of its kernels in flight."""
        torch.cuda.synchronize(self.device)
        if self.world > 1 and self.group is not None:
            dist.barrier(group=self.group)
        N.call("us_symm_reset", self.h, N.stream(), launches=0)
        torch.cuda.synchronize(self.device)
        if self.world > 1 and self.group is not None:
            dist.barrier(group=self.group)

    # ------------------------------------------------------------------ sites --
    def begin_forward(self) -> None:
        self.cursor = 0

    def next_site(self) -> int:
        s = self.cursor % self.ring
        self.cursor += 1
        return s

    def site_tensor(self, site: int, rows: int, cols: int, dtype=torch.bfloat16) -> torch.Tensor:
        """This rank's buffer of ``site`` viewed as [rows, cols]; producers write here."""
        key = (site, rows, cols, dtype)
        t = self._views.get(key)
        if t is None:
            nbytes = rows * cols * torch.empty(0, dtype=dtype).element_size()
            assert nbytes <= self.site_bytes, (nbytes, self.site_bytes)
            ptr = N.kernels().us_symm_site_ptr(self.h, site)
            raw = torch.as_tensor(_DevBuf(ptr, nbytes), device=self.device)
            t = raw.view(dtype).view(rows, cols)
            self._views[key] = t
        return t

    def peer_site_ptr(self, rank: int, site: int) -> int:
        """Address (in this process) of ``rank``'s buffer of ``site``."""
        return N.kernels().us_symm_peer_site_ptr(self.h, rank, site)

    def barrier(self, site: int) -> None:
        """Stream-ordered group barrier (flags over peer memory, bounded wait)."""
        N.call("us_symm_barrier", self.h, site, N.stream())

    def fits(self, rows: int, cols: int, elem: int = 2) -> bool:
        """Whether ``rows`` partial rows fit the push-form all-reduce."""
        return rows <= self.max_rows and 2 * self.world * rows * cols * elem <= self.site_bytes

    def _guard_reuse(self, site: int) -> None:
        if self._last_pull_site == site:
            self.barrier(self.SITE_AUX)
        self._last_pull_site = site

    # ------------------------------------------------------------- collectives --
    def allreduce_add_rmsnorm(self, partial, residual, w, eps: float, routed=None):
        """Sums every rank's partial rows [rows, H] (push form, one NVLink crossing), adds
        them to the FP32 residual stream (``residual=None`` starts it) and normalises.
        ``routed = (y_perm, perm, weights)`` forms the partial rows inside the kernel as the
        weighted sum of the token's local expert rows instead (``partial`` is then None)."""
        H = w.shape[0]
        rows = partial.shape[0] if routed is None else routed[1].shape[0]
        first = residual is None
        if first:
            residual = torch.empty(rows, H, dtype=torch.float32, device=self.device)
        y = torch.empty(rows, H, dtype=torch.bfloat16, device=self.device)
        site = self.next_site()
        if routed is None:
            assert partial.is_contiguous() and partial.dtype == torch.bfloat16
            N.call("us_symm_allreduce_add_rmsnorm", self.h, site, N.ptr(partial), None, None, None,
                   0, N.ptr(residual), N.ptr(w), N.ptr(y), rows, H, eps, int(first), N.stream())
        else:
            y_perm, perm, weights = routed
            N.call("us_symm_allreduce_add_rmsnorm", self.h, site, None, N.ptr(y_perm), N.ptr(perm),
                   N.ptr(weights), perm.shape[1], N.ptr(residual), N.ptr(w), N.ptr(y), rows, H,
                   eps, int(first), N.stream())
        return y, residual

    def argmax(self, logits: torch.Tensor, cols: int, col0: int) -> torch.Tensor:
        """Greedy tokens of a vocabulary-sharded head: ``logits`` [B, >= cols] FP32 are this
        rank's columns [col0, col0 + cols); the same int32 [B] comes back on every rank."""
        B = logits.shape[0]
        assert logits.dtype == torch.float32 and logits.stride(1) == 1 and B <= self.max_rows
        out = torch.empty(B, dtype=torch.int32, device=self.device)
        N.call("us_symm_argmax", self.h, self.SITE_ARGMAX, N.ptr(logits), logits.stride(0), B,
               cols, col0, N.ptr(out), N.stream())
        return out

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Generic sum over the group (copies x into a site first; pull form)."""
        nbytes = x.numel() * x.element_size()
        if nbytes > self.site_bytes or nbytes % 16:
            dist.all_reduce(x, group=self.group)
            return x
        site = self.next_site()
        self._guard_reuse(site)
        buf = self.site_tensor(site, x.numel(), 1, x.dtype)
        buf.view(-1).copy_(x.reshape(-1))
        out = torch.empty_like(x)
        N.call("us_symm_allreduce", self.h, site, N.ptr(out), nbytes,
               int(x.dtype == torch.float32), N.stream())
        return out


def set_peer_wait_clocks(clocks: int) -> None:
    """Budget (SM clocks) of every wait on another GPU's flag on the current device;
    0 restores the default of about 1.5 s."""
    N.check(N.kernels().us_set_peer_wait_clocks(int(clocks)), "us_set_peer_wait_clocks")


def attach_fused(ctx, device, hidden: int = 2048, sites: int = 10) -> FusedComm:
    """Creates the heap over the context's tensor group and hooks it in."""
    ax = ctx.axis("tensor")
    fc = FusedComm(ax.group, ax.rank, ax.size, device, hidden, sites)
    ctx.fused = fc
    return fc
