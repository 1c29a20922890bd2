"""Prefill / decode disaggregation: a request leaves the engine that computed its prompt
and continues on another one.

``export_request`` lends the request's state: its tokens, sampling parameters and the
contents of the KV pages that hold its computed positions, per layer, with the range
of KV heads the exporting rank owns.  ``import_request`` allocates pages on the
receiving engine, writes the pages in (selecting / concatenating head ranges when the
two sides shard the heads differently) and enqueues the request with its positions
marked computed, so its next step is a decode step.  Outputs are what one engine
would have produced: the decode side samples with the request's own lineage seed.

``Handoff.to_bytes`` / ``from_bytes`` frame the state for any byte transport;
``send`` / ``recv`` move it over a ``torch.distributed`` group (gloo on the host, NCCL
between GPUs).  ``PrefillDecodePair`` drives one prefill and one decode engine in the
roles of the configuration (``role = prefill | decode | mixed``).

Reference behaviour: docs/configuration.md:683-709, crates/storage-server/src/handoff.rs,
crates/storage/src/runtime.rs:394-402 (reference project paths).
"""
from __future__ import annotations

import io
from dataclasses import asdict, dataclass, field, is_dataclass
from typing import Optional

import torch

from .types import SamplingParams


@dataclass
class Handoff:
    request_id: str
    prompt_ids: list
    output_ids: list
    params: dict
    priority: int = 0
    cache_salt: Optional[str] = None
    num_computed: int = 0
    page_size: int = 16
    head_lo: int = 0                 # first KV head held by the exporting rank
    heads_total: int = 0             # KV heads of the model
    kv: list = field(default_factory=list)   # per layer (k, v) [pages, page, heads, D] or None

    def nbytes(self) -> int:
        return sum(k.numel() * k.element_size() * 2 for k, _ in (p for p in self.kv if p))

    def to_bytes(self) -> bytes:
        buf = io.BytesIO()
        d = asdict(self)
        d["kv"] = [None if p is None else (p[0].cpu(), p[1].cpu()) for p in self.kv]
        torch.save(d, buf)
        return buf.getvalue()

    @classmethod
    def from_bytes(cls, blob: bytes) -> "Handoff":
        return cls(**torch.load(io.BytesIO(blob), weights_only=False))


def export_request(engine, request_id: str, release: bool = True) -> Handoff:
    """Lends ``request_id`` (running, at least its prompt computed).  With ``release``
    the request ends here (its pages go back to the pool, committed prefix pages stay
    in the prefix cache)."""
    sch, runner = engine.scheduler, engine.runner
    req = sch.requests[request_id]
    assert not req.finished and req.num_computed >= len(req.prompt_ids), \
        "a request is lent once its prompt is computed"
    ps = runner.page_size
    n = (req.num_computed + ps - 1) // ps
    pages = torch.tensor(req.pages[:n], dtype=torch.long, device=runner.device)
    kv = []
    for pair in runner.kv_caches:
        if pair is None or pair[0] is None:
            kv.append(None)
        else:
            kv.append((pair[0].index_select(0, pages).clone(), pair[1].index_select(0, pages).clone()))
    model = engine.model
    params = req.params
    h = Handoff(request_id=req.request_id, prompt_ids=list(req.prompt_ids),
                output_ids=list(req.output_ids),
                params=asdict(params) if is_dataclass(params) else dict(params),
                priority=req.priority, cache_salt=req.cache_salt, num_computed=req.num_computed,
                page_size=ps, head_lo=model.ctx.tp_rank * model.Hkv // max(1, model.kv_rep),
                heads_total=model.cfg.num_key_value_heads, kv=kv)
    if release:
        from .types import FinishReason
        sch._finish(req, FinishReason.ABORT)
        del sch.requests[request_id]
    return h


def reshard_heads(shards: list, want_lo: int, want_n: int) -> torch.Tensor:
    """``shards``: (head_lo, tensor [pages, page, heads, D]) from the exporting ranks;
    returns heads [want_lo, want_lo + want_n) in order."""
    parts = []
    for lo, t in sorted(shards, key=lambda s: s[0]):
        a, b = max(lo, want_lo), min(lo + t.shape[2], want_lo + want_n)
        if a < b:
            parts.append(t[:, :, a - lo:b - lo])
    got = sum(p.shape[2] for p in parts)
    assert got == want_n, f"head range [{want_lo}, {want_lo + want_n}) not covered ({got})"
    return parts[0] if len(parts) == 1 else torch.cat(parts, 2)


def import_request(engine, handoffs) -> str:
    """Continues a lent request on ``engine``.  ``handoffs``: one ``Handoff`` or the list
    of every exporting rank's (head ranges are re-cut for this rank)."""
    hs = handoffs if isinstance(handoffs, (list, tuple)) else [handoffs]
    h = hs[0]
    sch, runner, model = engine.scheduler, engine.runner, engine.model
    assert h.page_size == runner.page_size, "both sides use the same page size"
    n = (h.num_computed + h.page_size - 1) // h.page_size
    pages = engine.blocks.allocate(n)
    if pages is None:
        raise RuntimeError("no free KV pages for the imported request")
    want_lo = model.ctx.tp_rank * model.Hkv // max(1, model.kv_rep)
    idx = torch.tensor(pages, dtype=torch.long, device=runner.device)
    for layer, pair in enumerate(runner.kv_caches):
        if pair is None or pair[0] is None:
            continue
        for which in (0, 1):
            shards = [(x.head_lo, x.kv[layer][which]) for x in hs if x.kv[layer] is not None]
            t = reshard_heads(shards, want_lo, pair[which].shape[2])
            pair[which].index_copy_(0, idx, t.to(device=runner.device, dtype=pair[which].dtype))
    rid = engine.add_request(h.prompt_ids, SamplingParams(**h.params), request_id=h.request_id,
                             priority=h.priority, cache_salt=h.cache_salt,
                             output_ids=h.output_ids)
    req = sch.requests[rid]
    req.pages, req.num_computed = list(pages), h.num_computed
    req.migrations += 1
    return rid


# ------------------------------------------------------------------ transport --
def send(h: Handoff, dst: int, group=None) -> None:
    import torch.distributed as dist
    blob = torch.frombuffer(bytearray(h.to_bytes()), dtype=torch.uint8)
    dist.send(torch.tensor([blob.numel()], dtype=torch.int64), dst, group=group)
    dist.send(blob, dst, group=group)


def recv(src: int, group=None) -> Handoff:
    import torch.distributed as dist
    n = torch.zeros(1, dtype=torch.int64)
    dist.recv(n, src, group=group)
    blob = torch.empty(int(n), dtype=torch.uint8)
    dist.recv(blob, src, group=group)
    return Handoff.from_bytes(blob.numpy().tobytes())


class PrefillDecodePair:
    """One prefill engine and one decode engine behind the calls of a single engine:
    prompts are computed on the first, every request moves as soon as it has its first
    token, the second one decodes.  ``moved_bytes`` counts the KV that travelled."""

    def __init__(self, prefill_engine, decode_engine, through_bytes: bool = False):
        self.prefill, self.decode = prefill_engine, decode_engine
        self.through_bytes = through_bytes
        self.moved_bytes = 0
        self.moved = 0

    def add_request(self, prompt_ids, params=None, **kw) -> str:
        return self.prefill.add_request(prompt_ids, params, **kw)

    def has_work(self) -> bool:
        return self.prefill.has_work() or self.decode.has_work()

    def step(self) -> list:
        outs = []
        if self.prefill.has_work():
            outs.extend(self.prefill.step())
            for req in list(self.prefill.scheduler.running):
                if req.output_ids and not req.finished:
                    h = export_request(self.prefill, req.request_id)
                    self.moved_bytes += h.nbytes()
                    self.moved += 1
                    if self.through_bytes:
                        h = Handoff.from_bytes(h.to_bytes())
                    import_request(self.decode, h)
        if self.decode.has_work():
            outs.extend(self.decode.step())
        return outs
