"""Lock-step joins of expert ranks in the disaggregated (attention / experts) layout.

Expert ranks hold no attention and no requests; every forward of the attention
ranks is a *join* for them: they must run the expert side of every layer of that
forward with the same per-source row count.  The first attention rank announces
each forward over a host-side (gloo) control group just before issuing it; expert
ranks sit in ``ExpertJoinLoop.run`` and mirror it: an eager forward, a graph
capture, or ``n`` replays of a captured graph.  All attention ranks run the same
sequence themselves (they are driven in lock step by the same schedule).

Reference behaviour: crates/engine/src/runner/causal_lm/experts.rs:377-421
(enter / join), :438-460 (capacity agreement) — reference project paths.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class StepAnnouncer:
    """Attention side.  Only the group's first member sends; the others no-op."""

    def __init__(self, control_group, src_global_rank: int, is_sender: bool):
        self.group, self.src, self.is_sender = control_group, src_global_rank, is_sender

    def __call__(self, kind: str, rows: int, count: int = 1) -> None:
        if self.is_sender:
            dist.broadcast_object_list([(kind, int(rows), int(count))], src=self.src,
                                       group=self.group)

    def stop(self) -> None:
        self("stop", 0, 0)


class ExpertJoinLoop:
    """Expert side: mirrors announced forwards until ``stop``."""

    def __init__(self, model, control_group, src_global_rank: int):
        self.model, self.group, self.src = model, control_group, src_global_rank
        self.graphs: dict = {}
        self.pool = None
        self.joins = 0

    def run(self) -> int:
        while True:
            box = [None]
            dist.broadcast_object_list(box, src=self.src, group=self.group)
            kind, rows, count = box[0]
            if kind == "stop":
                return self.joins
            micro = kind.endswith("+micro")      # the step runs as two half-batches
            if micro:
                kind = kind[:-len("+micro")]
            if kind == "eager":
                for _ in range(count):
                    self.model.forward_experts_only(rows, micro=micro)
                    self.joins += 1
            elif kind == "capture":
                g = torch.cuda.CUDAGraph()
                if self.pool is None:
                    self.pool = torch.cuda.graph_pool_handle()
                torch.cuda.synchronize()
                with torch.cuda.graph(g, pool=self.pool):
                    self.model.forward_experts_only(rows, micro=micro)
                self.graphs[(rows, micro)] = g
            elif kind == "replay":
                g = self.graphs[(rows, micro)]
                for _ in range(count):
                    g.replay()
                    self.joins += 1
            else:
                raise RuntimeError(f"unknown join message {kind!r}")
