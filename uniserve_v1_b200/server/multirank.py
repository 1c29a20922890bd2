"""Serving on several ranks: one leader (HTTP + engine), followers in lock step.

Tensor-parallel and sequence-parallel deployments run one process per GPU.  The
engine's host state (scheduler, block manager, request table) is *replicated*:
every rank runs the same deterministic engine and applies the same ordered
stream of commands, so every rank builds the same batches, launches the same
kernels and draws the same tokens (logits are all-gathered, sampling is
addressed by (seed, position)).  Only the commands travel: the leader publishes,
per step, the requests it admitted or aborted since the last step followed by
``step``; followers block on the control group (gloo, host memory) and apply.

    leader:    eng = ReplicatedEngine(LLMEngine(...), bus)   # same API as LLMEngine
    follower:  follower_loop(LLMEngine(...), bus)

Video deployments do the same with one command per request (prompt + plan):
every rank of the sequence group runs ``VideoService.generate``.

``spawn_followers`` starts ranks 1..N-1 of a package's layout as child processes
of ``serve`` and returns the leader's context; ``torchrun``-style launches work too
(RANK / WORLD_SIZE / MASTER_* from the environment).

Reference behaviour: crates/engine/src/executor.rs:86-103 (submit / map / stamp over
worker groups), crates/engine/src/parallel.rs:1-39 (host collectives for agreement);
reference project paths.
"""
from __future__ import annotations

import logging
import os
import pickle
from dataclasses import asdict, is_dataclass
from typing import Optional

import torch
import torch.distributed as dist


class CommandBus:
    """Ordered broadcast of small Python objects from rank 0 over a gloo group."""

    def __init__(self, group=None, rank: Optional[int] = None):
        self.group = group
        self.rank = dist.get_rank() if rank is None else rank
        self.leader = self.rank == 0

    def publish(self, commands: list) -> None:
        assert self.leader
        blob = [pickle.dumps(commands)]
        dist.broadcast_object_list(blob, src=0, group=self.group)

    def receive(self) -> list:
        assert not self.leader
        blob = [None]
        dist.broadcast_object_list(blob, src=0, group=self.group)
        return pickle.loads(blob[0])

    def gather(self, payload: bytes) -> Optional[list]:
        """Every rank's ``payload`` in rank order on the leader (None elsewhere); called by
        all ranks at the same point of the command stream."""
        world = dist.get_world_size(self.group)
        box = [None] * world if self.leader else None
        dist.gather_object(payload, box, dst=0, group=self.group)
        return box


def _plain(params):
    return asdict(params) if is_dataclass(params) else params


def apply_commands(engine, commands: list, bus: Optional["CommandBus"] = None):
    """Applies one published batch of commands to a local engine.  Returns the
    outputs of the step it contained (or None) and whether to keep running.  ``export`` /
    ``import`` move a request's state between deployments: every rank lends (or takes) the
    KV heads it holds; the leader collects the frames over ``bus``."""
    from ..engine.types import SamplingParams
    outs, alive = None, True
    for c in commands:
        op = c[0]
        if op == "add":
            _, rid, ids, params, prio, salt, outputs = c
            sp = SamplingParams(**params) if isinstance(params, dict) else params
            try:
                engine.add_request(ids, sp, request_id=rid, priority=prio, cache_salt=salt,
                                   output_ids=outputs)
            except ValueError:
                pass        # the leader rejected it the same way and told its client
        elif op == "abort":
            engine.abort(c[1])
        elif op == "step":
            outs = engine.step()
        elif op == "burst":
            outs = engine.decode_burst(c[1])
        elif op == "export":
            from ..engine.handoff import export_request
            frame = export_request(engine, c[1]).to_bytes()
            engine.exported_frames = bus.gather(frame) if bus is not None else [frame]
        elif op == "import":
            from ..engine.handoff import handoffs_from_bytes, import_request
            try:
                hs = handoffs_from_bytes(c[2])
                for h in hs:
                    h.request_id = c[1]
                import_request(engine, hs)
                engine.import_error = None
            except Exception as e:      # every rank refuses the same body the same way
                engine.import_error = e
        elif op == "shutdown":
            alive = False
    return outs, alive


class ReplicatedEngine:
    """The leader's engine: same calls as ``LLMEngine``; admissions and aborts are
    queued and published together with the next step so that every rank applies
    them at the same point of the step sequence."""

    def __init__(self, engine, bus: CommandBus):
        self.engine, self.bus = engine, bus
        self.pending: list = []

    def __getattr__(self, name):          # stats, scheduler, failed, profiler, ...
        return getattr(self.engine, name)

    def add_request(self, prompt_ids, params=None, request_id: Optional[str] = None,
                    priority: int = 0, cache_salt: Optional[str] = None,
                    output_ids: Optional[list] = None) -> str:
        V = self.engine.model.cfg.vocab_size
        if any((t < 0 or t >= V) for t in prompt_ids):
            raise ValueError("input_error: token id outside the vocabulary")
        rid = request_id or f"req-{next(self.engine._ids)}"
        self.pending.append(("add", rid, list(prompt_ids), _plain(params), priority, cache_salt,
                             list(output_ids) if output_ids else None))
        return rid

    def abort(self, request_id: str) -> bool:
        known = any(c[0] == "add" and c[1] == request_id for c in self.pending) or \
            request_id in self.engine.scheduler.requests
        self.pending.append(("abort", request_id))
        return known

    def has_work(self) -> bool:
        return bool(self.pending) or self.engine.has_work()

    def _run(self, last) -> list:
        cmds, self.pending = self.pending + [last], []
        self.bus.publish(cmds)
        outs, _ = apply_commands(self.engine, cmds, self.bus)
        return outs or []

    def export_request(self, request_id: str) -> bytes:
        """Lends the request on every rank (between two steps) and returns the ranks' frames
        as one body (``engine.handoff.pack_frames``)."""
        from ..engine.handoff import pack_frames
        self._run(("export", request_id))
        return pack_frames(self.engine.exported_frames)

    def import_request(self, request_id: str, body: bytes) -> str:
        """Continues a lent request on every rank: each takes the KV heads it holds out of
        the exporter's frames, whatever the exporter's tensor-parallel degree was."""
        self._run(("import", request_id, bytes(body)))
        if self.engine.import_error is not None:
            raise self.engine.import_error
        return request_id

    def step(self) -> list:
        return self._run(("step",))

    def decode_burst(self, steps: int) -> list:
        return self._run(("burst", steps))

    def shutdown(self) -> None:
        self.bus.publish([("shutdown",)])


def follower_loop(engine, bus: CommandBus) -> int:
    """Applies the leader's commands until it says shutdown; returns the steps run."""
    steps = 0
    while True:
        cmds = bus.receive()
        _, alive = apply_commands(engine, cmds, bus)
        steps += sum(1 for c in cmds if c[0] in ("step", "burst"))
        if not alive:
            return steps


# ------------------------------------------------------------------- video ----
class ReplicatedVideoService:
    """Leader side of a sequence-parallel video deployment: every ``generate`` is
    announced to the followers, which run the same request."""

    def __init__(self, service, bus: CommandBus):
        self.service, self.bus = service, bus
        inner = service.generate

        def generate(job):
            self.bus.publish([("video", job.prompt, asdict(job.plan))])
            return inner(job)
        service.generate = generate

    def shutdown(self) -> None:
        self.bus.publish([("shutdown",)])


def video_follower_loop(service, bus: CommandBus) -> int:
    from .video_rules import VideoPlan
    from .video_service import VideoJob
    done = 0
    while True:
        for c in bus.receive():
            if c[0] == "shutdown":
                return done
            if c[0] == "video":
                try:
                    service.generate(VideoJob(c[1], VideoPlan(**c[2])))
                except (ValueError, OSError) as e:
                    # the request's own media or size: every rank refuses it at the same point,
                    # before any exchange, and the leader answers the client
                    logging.getLogger(__name__).warning("video request refused: %s", e)
                done += 1


# ------------------------------------------------------------------ launch ----
def package_parallelism(pkg) -> dict:
    """How the package's model (or denoiser) group is laid out: ``world`` ranks per copy
    and the axes to build - ``tensor`` / ``layer`` for text models, ``ulysses`` or
    ``gather`` for the video transformer.  A group with ``copies = N`` describes N
    replicas of that layout; one replica is served per ``serve`` command."""
    lay = pkg.layout()
    best = {"world": 1, "axes": {}}
    for g in lay["groups"]:
        copies = max(1, int(g.get("copies", 1) or 1))
        ranks = max(1, len(g["ranks"]) // copies)
        axes = {}
        blocks = g.get("blocks", {})
        tr = next((b for b in blocks.values()
                   if isinstance(b.get("sequence_parallel"), dict) and
                   b["sequence_parallel"].get("kind") not in (None, "", "none")), None)
        if tr:
            sp = tr["sequence_parallel"]
            if sp.get("kind") == "allgather":
                axes["gather"] = int(sp.get("allgather_degree") or ranks)
            elif sp.get("kind") == "hybrid":
                axes["ulysses"] = int(sp.get("ulysses_degree") or 2)
                axes["gather"] = int(sp.get("allgather_degree") or
                                     max(1, ranks // axes["ulysses"]))
            elif sp.get("kind") == "ulysses":
                axes["ulysses"] = int(sp.get("ulysses_degree") or ranks)
        model = blocks.get("model") or blocks.get("causal_lm")
        if model and not axes:
            tp = int(model.get("tensor_parallel_size", 1) or 1)
            pp = int(model.get("pipeline_parallel_size", 1) or 1)
            if tp > 1:
                axes["tensor"] = tp
            if pp > 1:
                axes["layer"] = pp
        world = 1
        for v in axes.values():
            world *= v
        if not axes and ranks > 1 and g.get("role") in ("model", None):
            axes, world = {"tensor": ranks}, ranks
        seq = "ulysses" in axes or "gather" in axes
        if world > best["world"] or (seq and not ("ulysses" in best["axes"] or
                                                  "gather" in best["axes"])):
            best = {"world": world, "axes": axes}
    return best


def package_union(pkg) -> Optional[dict]:
    """The expert union a package describes, or None.

    * ``moe_config.expert_parallel`` with ``data_parallel_size = N`` and no tensor
      parallelism: N attention members that each hold 1/N of the experts.
    * a worker group with ``role = "experts"``: the ranks of the model groups are the
      attention members, the ranks of the experts groups hold the experts (the
      disaggregated layout).  Attention members are data parallel: a
      ``tensor_parallel_size`` inside the attention group of such a layout is served as
      that many attention members.
    Returns {"sources": n, "experts": m, "shared": bool} (``shared``: every member has
    both roles)."""
    if not pkg.moe_config.expert_parallel:
        return None
    lay = pkg.layout()
    groups = lay["groups"]
    exp = sum(len(g["ranks"]) for g in groups if g.get("role") == "experts")
    if exp:
        src = sum(len(g["ranks"]) for g in groups if g.get("role") != "experts")
        return {"sources": max(1, src), "experts": exp, "shared": False}
    dp = int(lay.get("data_parallel_size") or 1)
    tp = max([int((g.get("blocks", {}).get("model") or {}).get("tensor_parallel_size", 1) or 1)
              for g in groups] + [int(pkg.top.get("tensor_parallel_size", 1) or 1)])
    if dp > 1 and tp == 1:
        return {"sources": dp, "experts": dp, "shared": True}
    return None


def package_world(pkg) -> int:
    u = package_union(pkg)
    if u:
        return u["sources"] + (0 if u["shared"] else u["experts"])
    return package_parallelism(pkg)["world"]


def init_rank(backend: Optional[str] = None):
    """Joins the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT and
    returns (rank, world, device, control group).  The control group is gloo."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", local) if cuda else torch.device("cpu")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if cuda:
            torch.cuda.set_device(local)
            dist.init_process_group(backend or "nccl", device_id=device)
        else:
            dist.init_process_group(backend or "gloo")
        control = dist.new_group(list(range(world)), backend="gloo")
    else:
        control = None
    return rank, world, device, control


def spawn_followers(world: int, argv: list, port: int) -> list:
    """Starts ranks 1..world-1 as child processes running ``argv`` (the same serve
    command) with the rank environment set; the caller becomes rank 0."""
    import subprocess
    import sys
    procs = []
    base = dict(os.environ, WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    for r in range(1, world):
        env = dict(base, RANK=str(r), LOCAL_RANK=str(r))
        procs.append(subprocess.Popen([sys.executable, "-m", "uniserve_v1_b200"] + argv, env=env))
    os.environ.update(base, RANK="0", LOCAL_RANK="0")
    return procs
