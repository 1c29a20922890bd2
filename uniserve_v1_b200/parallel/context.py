"""Per-rank parallel context: which groups a forward pass runs along.

A forward carries up to four groups, selected by axis name, mirroring the
reference's multi-axis contexts (``ULYSSES, GATHER, TENSOR, LAYER``;
crates/ops/src/collective.rs:285-309, crates/nn/src/family.rs:610-616, reference
project paths).  One process drives one GPU; groups are ``torch.distributed``
process groups (NCCL on GPUs, gloo on CPU ranks).  Collectives default to the
library path; when a symmetric peer heap is attached the tensor-axis reductions
run through the hand-written peer-memory kernels instead.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist

AXES = ("tensor", "expert", "ulysses", "gather", "layer", "data")


@dataclass
class Axis:
    group: Optional[object] = None     # torch.distributed process group
    rank: int = 0
    size: int = 1
    ranks: tuple = (0,)                # global ranks of the members


@dataclass
class ParallelContext:
    world_rank: int = 0
    world_size: int = 1
    axes: dict = field(default_factory=dict)
    fused = None                       # parallel.symm.FusedComm when peer memory is mapped
    expert_parallel: bool = False

    @classmethod
    def single(cls) -> "ParallelContext":
        return cls()

    def axis(self, name: str) -> Axis:
        return self.axes.get(name) or Axis()

    @property
    def tp_size(self) -> int:
        return self.axis("tensor").size

    @property
    def tp_rank(self) -> int:
        return self.axis("tensor").rank

    @property
    def ep_size(self) -> int:
        return self.axis("expert").size

    @property
    def ep_rank(self) -> int:
        return self.axis("expert").rank

    # -- construction ---------------------------------------------------------
    @classmethod
    def from_world(cls, tensor: int = 1, expert: int = 1, ulysses: int = 1, gather: int = 1,
                   layer: int = 1, expert_over_tensor: bool = False) -> "ParallelContext":
        """Builds axis groups over the default process group.  Rank order is
        (layer, gather, ulysses, tensor) with tensor fastest.  With
        ``expert_over_tensor`` the expert axis is the tensor group itself
        (whole experts per tensor rank)."""
        if not dist.is_initialized():
            assert tensor * ulysses * gather * layer == 1
            return cls.single()
        world, rank = dist.get_world_size(), dist.get_rank()
        sizes = {"tensor": tensor, "ulysses": ulysses, "gather": gather, "layer": layer}
        prod = tensor * ulysses * gather * layer
        assert world % prod == 0, f"world {world} not divisible by {sizes}"
        sizes["data"] = world // prod
        order = ["tensor", "ulysses", "gather", "layer", "data"]
        strides, s = {}, 1
        for name in order:
            strides[name] = s
            s *= sizes[name]
        coords = {name: (rank // strides[name]) % sizes[name] for name in order}
        ctx = cls(world_rank=rank, world_size=world)
        for name in order:
            n = sizes[name]
            if n == 1:
                ctx.axes[name] = Axis(None, 0, 1, (rank,))
                continue
            # every rank must create every group in the same order
            mine = None
            others = [o for o in order if o != name]
            bases = set()
            for r in range(world):
                base = r - ((r // strides[name]) % n) * strides[name]
                bases.add(base)
            for base in sorted(bases):
                members = tuple(base + i * strides[name] for i in range(n))
                g = dist.new_group(list(members))
                if rank in members:
                    mine = Axis(g, members.index(rank), n, members)
            ctx.axes[name] = mine
        # "sequence": every rank that holds a row interval of the same clip, ordered
        # by interval (gather place major, Ulysses member minor).
        if ulysses > 1 and gather > 1:
            su, sg = strides["ulysses"], strides["gather"]
            bases = sorted({r - ((r // su) % ulysses) * su - ((r // sg) % gather) * sg
                            for r in range(world)})
            for base in bases:
                members = tuple(base + iu * su + ig * sg
                                for ig in range(gather) for iu in range(ulysses))
                g = dist.new_group(list(members))
                if rank in members:
                    ctx.axes["sequence"] = Axis(g, members.index(rank), len(members), members)
        else:
            ctx.axes["sequence"] = ctx.axes["gather"] if gather > 1 else ctx.axes["ulysses"]
        if expert_over_tensor:
            ctx.axes["expert"] = ctx.axes["tensor"]
            ctx.expert_parallel = True
        elif expert > 1:
            assert expert == world, "a separate expert axis spans the world"
            ctx.axes["expert"] = Axis(dist.group.WORLD, rank, world, tuple(range(world)))
            ctx.expert_parallel = True
        return ctx

    # -- collectives ------------------------------------------------------------
    def all_reduce(self, x: torch.Tensor, axis: str = "tensor") -> torch.Tensor:
        a = self.axis(axis)
        if a.size == 1:
            return x
        if self.fused is not None and axis == "tensor" and x.is_cuda:
            return self.fused.all_reduce(x)
        dist.all_reduce(x, group=a.group)
        return x

    def all_reduce_tp(self, x: torch.Tensor) -> torch.Tensor:
        return self.all_reduce(x, "tensor")

    def all_gather_rows(self, x: torch.Tensor, axis: str) -> torch.Tensor:
        a = self.axis(axis)
        if a.size == 1:
            return x
        out = torch.empty((a.size * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=a.group)
        return out

    def all_gather_tp_cols(self, x: torch.Tensor) -> torch.Tensor:
        """[rows, c] per rank -> [rows, P*c] in rank order."""
        a = self.axis("tensor")
        if a.size == 1:
            return x
        g = self.all_gather_rows(x, "tensor")            # [P*rows, c]
        return g.view(a.size, x.shape[0], x.shape[1]).permute(1, 0, 2).reshape(x.shape[0], -1)

    def all_to_all(self, x: torch.Tensor, axis: str) -> torch.Tensor:
        """x [P, ...] block i goes to member i; returns [P, ...] received blocks."""
        a = self.axis(axis)
        if a.size == 1:
            return x
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x.contiguous(), group=a.group)
        return out

    def broadcast(self, x: torch.Tensor, src_index: int, axis: str) -> torch.Tensor:
        a = self.axis(axis)
        if a.size == 1:
            return x
        dist.broadcast(x, src=a.ranks[src_index], group=a.group)
        return x

    def barrier(self):
        if dist.is_initialized():
            dist.barrier()
