"""Distributed weight data parallelism: data-parallel ranks that keep the routed experts
sharded among themselves in memory and READ the shards they miss from their peers, instead
of exchanging tokens.

Every rank is a whole attention replica with its own requests.  The experts of each MoE
layer are resident as ``world`` shards, one per rank, inside a symmetric heap (a site per
layer, laid out ``[w13 shard | w2 shard]``).  When a layer runs, the rank assembles all of
its experts in one of two local buffers: its own shard by a local copy, the others by
copies out of the peers' heaps over NVLink (copy engines, one ``cudaMemcpyAsync`` per
shard and tensor).  The copies of layer i + 1 are issued on a side stream when layer i
starts its experts and overlap its GEMMs; two events per buffer order the streams (ready:
the compute stream may read it; consumed: the side stream may overwrite it).  Tokens never
leave their rank, so there is no dispatch, no combine and no step agreement between the
ranks; the price is (world - 1) / world of a layer's expert bytes over NVLink per layer and
rank, which pays for prefill-sized batches (a 1.2 GB layer is 1.4 ms of link time at
770 GB/s) and not for decode-sized ones.

Weights are read-only after loading: no flag protocol is needed, only the host-side
barrier after the shards were written.  ``HostWeightPeers`` is the same interface for CPU
ranks (gloo all-gather of the shards), used by the CPU tests.

Reference behaviour: docs/expert_parallelism.md:3, docs/admin.md:270 (reference project
paths).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import native as N
from .symm import FusedComm, _DevBuf

N.register_signatures({
    "us_copy_async": (N.I, [N.P, N.P, N.L, N.P]),
})


class WeightPeers:
    def __init__(self, group, rank: int, world: int, device, layers: list, experts_local: int,
                 hidden: int, inter: int, dtype=torch.bfloat16):
        """``layers``: indices of the MoE layers this rank runs (site order)."""
        self.group, self.rank, self.world = group, rank, world
        self.device = torch.device(device)
        self.layers = list(layers)
        self.site_of = {layer: i for i, layer in enumerate(self.layers)}
        self.El, self.H, self.I = experts_local, hidden, inter
        esz = torch.empty(0, dtype=dtype).element_size()
        self.dtype = dtype
        self.n13 = experts_local * 2 * inter * hidden          # elements of a w13 shard
        self.n2 = experts_local * hidden * inter
        self.b13, self.b2 = self.n13 * esz, self.n2 * esz
        self.heap = FusedComm(group, rank, world, device, hidden=0, sites=len(self.layers) + 2,
                              site_bytes=self.b13 + self.b2)
        E = world * experts_local
        self.full13 = [torch.empty(E, 2 * inter, hidden, dtype=dtype, device=device) for _ in (0, 1)]
        self.full2 = [torch.empty(E, hidden, inter, dtype=dtype, device=device) for _ in (0, 1)]
        self.side = torch.cuda.Stream(device=device)
        self.ready = [torch.cuda.Event() for _ in (0, 1)]
        self.consumed = [torch.cuda.Event() for _ in (0, 1)]
        self.issued: dict = {}                 # layer -> buffer its gather was issued into
        self.bytes_read = 0                    # from peers, since creation

    # ------------------------------------------------------------------ shards --
    def shard(self, layer: int):
        """This rank's resident shard of ``layer`` as (w13 [El, 2I, H], w2 [El, H, I]) views of
        the heap; the loader writes the weights here."""
        site = self.site_of[layer]
        ptr = N.kernels().us_symm_site_ptr(self.heap.h, site)
        raw = torch.as_tensor(_DevBuf(ptr, self.b13 + self.b2), device=self.device)
        w13 = raw[:self.b13].view(self.dtype).view(self.El, 2 * self.I, self.H)
        w2 = raw[self.b13:].view(self.dtype).view(self.El, self.H, self.I)
        return w13, w2

    def publish(self) -> None:
        """After every rank wrote its shards: they may be read from now on."""
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)

    # ------------------------------------------------------------------ gather --
    def prefetch(self, layer: int) -> None:
        """Issues the copies that assemble ``layer``'s experts (side stream)."""
        if layer in self.issued or layer not in self.site_of:
            return
        buf = self._next
        self._next ^= 1
        self.issued[layer] = buf
        site = self.site_of[layer]
        self.side.wait_event(self.consumed[buf])          # whoever used this buffer is done
        st = ctypes.c_void_p(self.side.cuda_stream)
        d13, d2 = self.full13[buf], self.full2[buf]
        for r in range(self.world):
            src = self.heap.peer_site_ptr(r, site)
            N.call("us_copy_async", ctypes.c_void_p(d13.data_ptr() + r * self.b13),
                   ctypes.c_void_p(src), self.b13, st, launches=0)
            N.call("us_copy_async", ctypes.c_void_p(d2.data_ptr() + r * self.b2),
                   ctypes.c_void_p(src + self.b13), self.b2, st, launches=0)
            if r != self.rank:
                self.bytes_read += self.b13 + self.b2
        self.ready[buf].record(self.side)

    def layer_weights(self, layer: int, next_layer: Optional[int] = None):
        """All experts of ``layer`` as (w13 [E, 2I, H], w2 [E, H, I]); the copies of
        ``next_layer`` start now and overlap this layer's GEMMs.  Call ``release(layer)``
        after the layer's last kernel was issued."""
        self.prefetch(layer)
        buf = self.issued[layer]
        torch.cuda.current_stream(self.device).wait_event(self.ready[buf])
        if next_layer is not None:
            self.prefetch(next_layer)
        return self.full13[buf], self.full2[buf]

    def release(self, layer: int) -> None:
        buf = self.issued.pop(layer)
        self.consumed[buf].record(torch.cuda.current_stream(self.device))

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        self.heap.close()

    _next = 0


class HostWeightPeers:
    """The same interface over a host (gloo) group: a layer's shards are all-gathered when it
    runs.  For CPU ranks and tests."""

    def __init__(self, group, rank: int, world: int, layers: list, experts_local: int,
                 hidden: int, inter: int, dtype=torch.float32):
        self.group, self.rank, self.world = group, rank, world
        self.layers = list(layers)
        self.El, self.H, self.I = experts_local, hidden, inter
        self.shards = {layer: (torch.zeros(experts_local, 2 * inter, hidden, dtype=dtype),
                               torch.zeros(experts_local, hidden, inter, dtype=dtype))
                       for layer in self.layers}
        self.bytes_read = 0

    def shard(self, layer: int):
        return self.shards[layer]

    def publish(self) -> None:
        if self.world > 1:
            dist.barrier(group=self.group)

    def prefetch(self, layer: int) -> None:
        pass

    def layer_weights(self, layer: int, next_layer: Optional[int] = None):
        out = []
        for t in self.shards[layer]:
            box = [torch.empty_like(t) for _ in range(self.world)]
            if self.world > 1:
                dist.all_gather(box, t.contiguous(), group=self.group)
            else:
                box[0] = t
            out.append(torch.cat(box, 0))
            self.bytes_read += (self.world - 1) * t.numel() * t.element_size()
        return out[0], out[1]

    def release(self, layer: int) -> None:
        pass

    def close(self) -> None:
        pass


def attach_weight_peers(model, group, rank: int, world: int):
    """Moves a model's resident expert shards (loaded with an expert axis of ``world``, no
    tensor split) into a ``WeightPeers`` heap and switches its MoE layers to read all experts
    through it.  Collective: every rank of ``group`` calls it."""
    cfg = model.cfg
    moe_layers = [i for i, lw in enumerate(model.layers)
                  if lw is not None and not lw.dense and lw.w13 is not None]
    if model.device.type == "cuda":
        peers = WeightPeers(group, rank, world, model.device, moe_layers, model.E_local,
                            cfg.hidden_size, cfg.moe_intermediate_size, model.dtype)
    else:
        peers = HostWeightPeers(group, rank, world, moe_layers, model.E_local, cfg.hidden_size,
                                cfg.moe_intermediate_size, model.dtype)
    for i in moe_layers:
        lw = model.layers[i]
        w13, w2 = peers.shard(i)
        w13.copy_(lw.w13)
        w2.copy_(lw.w2)
        lw.w13, lw.w2 = w13, w2
        lw.index = i
    peers.publish()
    model.weight_peers = peers
    model.moe_layer_order = moe_layers
    # routing sees every expert: all of them are run here
    model.E_resident, model.e_res_lo = model.E_local, model.e_lo
    model.E_local, model.e_lo = cfg.num_experts, 0
    model._moe_ws.clear()
    return peers
