"""Serving on an expert union: data-parallel attention with expert parallelism, and
attention / expert disaggregation.

A union is a set of ranks whose every MoE layer is one lock-step token exchange
(``parallel/expert_exchange.py``).  *Attention members* each own a scheduler, a KV cache
and their own requests; *expert members* (the disaggregated layout) hold experts only.
Because every layer is an exchange, the members step together:

1. **Plan.**  Every attention member schedules its own batch (or finds it has none).
2. **Agree.**  One host all-gather of (kind, rows) over the control group; the step's
   *capacity* is the largest row count, rounded up to a capacity class (the decode buckets,
   then powers of two).  Nobody has work: no step.
3. **Run.**  Every attention member runs its batch padded to the capacity; a member with
   no batch *joins*: the whole forward with zero live rows, so its dispatch and combine
   kernels (and, when it also holds experts, its expert GEMMs over the others' rows) are
   issued.  Expert members run the expert side of every layer at that capacity.

Decode steps of a capacity class replay one CUDA graph per class; the capacity travels as
the graph's bucket, the live row count as a device word.

``UnionFront`` is what the HTTP process drives: the calls of an engine (``add_request``,
``abort``, ``step``, ``has_work``).  It places each request on the member with the fewest
requests in flight, ships placements and aborts with the tick's first collective and
collects every member's outputs with its second.

Reference behaviour: crates/engine/src/runner/causal_lm/experts.rs:75-102 (capacity
classes), :377-421 (enter / join), :438-460 (agreement by host all-gather);
docs/expert_parallelism.md:5-31, :58-85 (reference project paths).
"""
from __future__ import annotations

import time
from dataclasses import asdict, is_dataclass
from typing import Optional

import torch.distributed as dist

from .runner import DECODE_BUCKETS
from .types import SamplingParams, StepOutput

PREFILL_CLASSES = (512, 1024, 2048, 4096, 8192, 16384)


def capacity_class(rows: int, limit: int) -> int:
    """Smallest capacity class that holds ``rows`` (0 stays 0); never above ``limit``."""
    if rows <= 0:
        return 0
    for c in DECODE_BUCKETS + PREFILL_CLASSES:
        if rows <= c <= limit:
            return c
    if rows <= limit:
        return limit
    raise ValueError(f"a step of {rows} rows exceeds the union's capacity {limit}")


class UnionMember:
    """One rank of the union.  ``engine`` is the member's own ``LLMEngine`` (attention
    members) or None (expert members, which only need ``model``)."""

    def __init__(self, control_group, rank: int, world: int, source_ranks, expert_ranks,
                 engine=None, model=None, capacity_limit: int = 8192,
                 exchange_free: bool = False, microbatches: int = 1):
        self.group, self.rank, self.world = control_group, rank, world
        self.sources, self.experts = tuple(source_ranks), tuple(expert_ranks)
        self.engine = engine
        self.model = model if model is not None else engine.model
        self.is_source = rank in self.sources
        self.limit = capacity_limit
        # members that move no tokens between them (weights are read one-sidedly from the
        # peers): an idle member has nothing to join
        self.exchange_free = exchange_free
        # `moe_config.microbatches` >= 2: a step in which every member decodes (or idles) runs
        # as two interleaved half-batches, each through its own exchange, so that attention of
        # one half overlaps the experts of the other
        self.microbatches = microbatches if getattr(self.model, "micro_exchanges", None) else 1
        self.stats = {"ticks": 0, "steps": 0, "joins": 0, "idle_ticks": 0, "capacities": {}}
        if engine is not None:
            # a member's prefill chunk must fit the agreed capacity
            engine.config.max_num_batched_tokens = min(engine.config.max_num_batched_tokens,
                                                       capacity_limit)
            engine.config.chunked_prefill_size = min(engine.config.chunked_prefill_size,
                                                     capacity_limit)

    # ------------------------------------------------------------------ tick --
    def _agree(self, mine):
        box = [None] * self.world
        dist.all_gather_object(box, mine, group=self.group)
        return box

    def tick(self, outputs_of_last: Optional[list] = None):
        """One agreed step.  Returns (outputs of this member's batch, everything gathered:
        per rank (kind, rows, outputs handed in))."""
        self.stats["ticks"] += 1
        batch = None
        if self.is_source and self.engine is not None and self.engine.failed is None \
                and self.engine.has_work():
            batch = self.engine.scheduler.schedule()
        rows = 0
        if batch is not None:
            rows = batch.num_tokens if batch.kind == "prefill" else len(batch.chunks)
        gathered = self._agree((batch.kind if batch else None, rows, outputs_of_last or []))
        cap = capacity_class(max(g[1] for g in gathered), self.limit)
        if cap == 0:
            self.stats["idle_ticks"] += 1
            return [], gathered
        self.stats["capacities"][cap] = self.stats["capacities"].get(cap, 0) + 1
        # every member sees the same kinds, so every member takes the same decision
        micro = self.microbatches >= 2 and cap >= 2 and cap % 2 == 0 and \
            all(g[0] in (None, "decode") for g in gathered)
        self.model.microbatch_now = micro
        if micro:
            self.stats["micro_steps"] = self.stats.get("micro_steps", 0) + 1
        if not self.is_source:
            self.model.forward_experts_only(cap, micro=micro)
            self.stats["joins"] += 1
            return [], gathered
        if batch is None:
            if not self.exchange_free:
                self.engine.runner.join(cap)
                self.stats["joins"] += 1
            return [], gathered
        self.stats["steps"] += 1
        try:
            return self.engine.run_batch(batch, capacity=cap), gathered
        except Exception as e:          # the member's engine has stopped: fail its requests
            from .types import FinishReason
            outs = []
            sch = self.engine.scheduler
            for req in list(sch.running) + list(sch.waiting):
                outs.append(StepOutput(req.request_id, [], True, FinishReason.ERROR,
                                       error=f"fatal_worker_failure: {e}"))
            sch.running.clear()
            sch.waiting.clear()
            return outs, gathered


# ------------------------------------------------------------- front / loops --
def _apply(member: UnionMember, commands: list) -> bool:
    """Applies the leader's commands that concern this member; False on shutdown."""
    alive = True
    for c in commands:
        if c[0] == "add" and c[1] == member.rank and member.engine is not None:
            _, _, rid, ids, params, prio, salt, outputs = c
            sp = SamplingParams(**params) if isinstance(params, dict) else params
            try:
                member.engine.add_request(ids, sp, request_id=rid, priority=prio,
                                          cache_salt=salt, output_ids=outputs)
            except (ValueError, RuntimeError):
                pass          # the leader validated the request; a failed engine reports itself
        elif c[0] == "abort" and member.engine is not None:
            if c[1] in member.engine.scheduler.requests:
                member.engine.abort(c[1])
        elif c[0] == "shutdown":
            alive = False
    return alive


class UnionFront:
    """The leader's engine-shaped face of the union (rank ``leader`` of the control group,
    itself an attention member)."""

    def __init__(self, member: UnionMember, leader: int = 0):
        assert member.rank == leader and member.engine is not None
        self.member, self.leader = member, leader
        self.engine = member.engine
        self.pending: list = []
        self.where: dict = {}                         # request id -> member rank
        self.load = {r: 0 for r in member.sources}    # requests in flight per member
        self._carry: list = []
        self._ids = 0

    def __getattr__(self, name):                      # model, config, scheduler, stats, ...
        return getattr(self.engine, name)

    # ---------------------------------------------------------------- requests --
    def add_request(self, prompt_ids, params=None, request_id: Optional[str] = None,
                    priority: int = 0, cache_salt: Optional[str] = None,
                    output_ids: Optional[list] = None) -> str:
        V = self.engine.model.cfg.vocab_size
        if any((t < 0 or t >= V) for t in prompt_ids):
            raise ValueError("input_error: token id outside the vocabulary")
        if len(prompt_ids) == 0 or len(prompt_ids) + 1 > self.engine.config.max_model_len:
            raise ValueError("input_error: the prompt does not fit the context")
        self._ids += 1
        rid = request_id or f"ureq-{self._ids}"
        target = min(self.load, key=lambda r: (self.load[r], r))
        self.load[target] += 1
        self.where[rid] = target
        plain = asdict(params) if is_dataclass(params) else params
        self.pending.append(("add", target, rid, list(prompt_ids), plain, priority, cache_salt,
                             list(output_ids) if output_ids else None))
        return rid

    def abort(self, request_id: str) -> bool:
        known = request_id in self.where
        if known:
            self.pending.append(("abort", request_id))
            self.load[self.where.pop(request_id)] -= 1      # an aborted request reports nothing
        return known

    def has_work(self) -> bool:
        return bool(self.pending) or bool(self.where) or bool(self._carry)

    # -------------------------------------------------------------------- step --
    def _tick(self, commands: list) -> list:
        dist.broadcast_object_list([commands], src=self.leader, group=self.member.group)
        _apply(self.member, commands)
        mine, gathered = self.member.tick(None)
        outs = list(mine)
        for r, g in enumerate(gathered):
            if r != self.leader:
                outs.extend(g[2])
        for o in outs:
            if o.finished and o.request_id in self.where:
                self.load[self.where.pop(o.request_id)] -= 1
        return outs

    def step(self) -> list:
        cmds, self.pending = self.pending, []
        return self._tick(cmds)

    def shutdown(self) -> None:
        dist.broadcast_object_list([[("shutdown",)]], src=self.leader, group=self.member.group)

    def union_stats(self) -> dict:
        return dict(self.member.stats, load=dict(self.load))


def member_loop(member: UnionMember, leader: int = 0) -> int:
    """Every other rank of the union: applies the leader's commands and steps with it until
    shutdown.  An attention member hands its outputs in with the next tick's gather."""
    carry: list = []
    ticks = 0
    while True:
        box = [None]
        dist.broadcast_object_list(box, src=leader, group=member.group)
        if not _apply(member, box[0]):
            return ticks
        carry, _ = member.tick(carry)
        ticks += 1
