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
between GPUs).  A tensor-parallel deployment lends one frame per rank, packed into one
body (``pack_frames`` / ``handoffs_from_bytes``: the frames must describe one request and
cover the model's KV heads); the taker's ranks each re-cut the heads they hold, so the two
deployments need not share a tensor-parallel degree (``server/multirank.py``:
``ReplicatedEngine.export_request`` / ``import_request``).  ``PrefillDecodePair`` drives one prefill and one decode engine in the
roles of the configuration (``role = prefill | decode | mixed``).

Reference behaviour: docs/configuration.md:683-709, crates/storage-server/src/handoff.rs,
crates/storage/src/runtime.rs:394-402 (reference project paths).
"""
from __future__ import annotations

import json
import struct
from dataclasses import asdict, dataclass, field, is_dataclass
from typing import Optional

import torch

from .types import SamplingParams

MAGIC = b"USHO\x01"
MAX_HEADER = 64 << 20
MAX_LAYERS = 4096
_DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16,
           "float8_e4m3fn": torch.float8_e4m3fn, "uint8": torch.uint8}
_DTYPE_NAMES = {v: k for k, v in _DTYPES.items()}


class HandoffError(ValueError):
    """A framed request state that is malformed or does not fit the importing engine."""


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
        """Explicit framing, nothing executable: ``MAGIC | u32 header length | JSON header |
        raw tensor bytes``.  The header carries every scalar field and, per layer, the dtype,
        shape and byte range of the K and V page tensors."""
        tensors, blobs, off = [], [], 0
        for pair in self.kv:
            if pair is None:
                tensors.append(None)
                continue
            entry = []
            for t in pair:
                t = t.detach().cpu().contiguous()
                raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
                entry.append({"dtype": _DTYPE_NAMES[t.dtype], "shape": list(t.shape),
                              "offset": off, "nbytes": len(raw)})
                blobs.append(raw)
                off += len(raw)
            tensors.append(entry)
        d = asdict(self)
        d["kv"] = tensors
        head = json.dumps(d, separators=(",", ":")).encode()
        return b"".join([MAGIC, struct.pack("<I", len(head)), head, *blobs])

    @classmethod
    def from_bytes(cls, blob: bytes) -> "Handoff":
        """Parses the framing of ``to_bytes``; raises ``HandoffError`` on anything else (a
        pickle stream, a truncated body, ranges outside the body, unknown dtypes)."""
        blob = bytes(blob)
        if len(blob) < len(MAGIC) + 4 or blob[:len(MAGIC)] != MAGIC:
            raise HandoffError("not a hand-off frame")
        (n,) = struct.unpack_from("<I", blob, len(MAGIC))
        start = len(MAGIC) + 4
        if n > MAX_HEADER or start + n > len(blob):
            raise HandoffError("header length outside the body")
        try:
            d = json.loads(blob[start:start + n].decode())
        except (UnicodeDecodeError, ValueError) as e:
            raise HandoffError(f"header is not JSON: {e}") from None
        if not isinstance(d, dict) or set(d) != set(cls.__dataclass_fields__):
            raise HandoffError("header fields do not match the hand-off record")
        body = memoryview(blob)[start + n:]
        kv = []
        if not isinstance(d["kv"], list) or len(d["kv"]) > MAX_LAYERS:
            raise HandoffError("kv: not a list of layers")
        for entry in d["kv"]:
            if entry is None:
                kv.append(None)
                continue
            if not isinstance(entry, list) or len(entry) != 2:
                raise HandoffError("kv: a layer holds one K and one V tensor")
            pair = []
            for spec in entry:
                try:
                    dt = _DTYPES[spec["dtype"]]
                    shape = [int(x) for x in spec["shape"]]
                    off, nb = int(spec["offset"]), int(spec["nbytes"])
                except (KeyError, TypeError, ValueError):
                    raise HandoffError("kv: malformed tensor record") from None
                numel = 1
                for x in shape:
                    if x < 0:
                        raise HandoffError("kv: negative extent")
                    numel *= x
                if len(shape) != 4 or off < 0 or nb != numel * dt.itemsize or off + nb > len(body):
                    raise HandoffError("kv: tensor bytes outside the body")
                t = torch.frombuffer(bytearray(body[off:off + nb]), dtype=dt) if nb else \
                    torch.empty(0, dtype=dt)
                pair.append(t.reshape(shape))
            kv.append(tuple(pair))
        d["kv"] = kv
        h = cls(**d)
        h.check_fields()
        return h

    def check_fields(self) -> None:
        """Type and range checks that need no model (``validate_for`` adds the importer's)."""
        def ints(xs, what):
            if not isinstance(xs, list) or not all(isinstance(x, int) and not isinstance(x, bool)
                                                   and x >= 0 for x in xs):
                raise HandoffError(f"{what}: a list of non-negative token ids")
        if not isinstance(self.request_id, str) or len(self.request_id) > 256:
            raise HandoffError("request_id: a short string")
        ints(self.prompt_ids, "prompt_ids")
        ints(self.output_ids, "output_ids")
        if not isinstance(self.params, dict) or \
                not set(self.params) <= set(SamplingParams.__dataclass_fields__):
            raise HandoffError("params: unknown sampling field")
        for name in ("priority", "num_computed", "page_size", "head_lo", "heads_total"):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool):
                raise HandoffError(f"{name}: an integer")
        if self.cache_salt is not None and not isinstance(self.cache_salt, str):
            raise HandoffError("cache_salt: a string")
        if not self.prompt_ids or self.page_size <= 0 or self.num_computed < 0 or \
                self.num_computed > len(self.prompt_ids) + len(self.output_ids):
            raise HandoffError("num_computed exceeds the tokens of the request")

    def validate_for(self, engine) -> None:
        """Checks every field against the importing engine's model and cache before a page
        is written: vocabulary range, KV-head range, page size, page count and tensor shapes."""
        self.check_fields()
        runner, model = engine.runner, engine.model
        vocab = model.cfg.vocab_size
        if any(t >= vocab for t in self.prompt_ids) or any(t >= vocab for t in self.output_ids):
            raise HandoffError("token id outside the vocabulary")
        if self.page_size != runner.page_size:
            raise HandoffError(f"page size {self.page_size} differs from the importer's "
                               f"{runner.page_size}")
        if self.heads_total != model.cfg.num_key_value_heads:
            raise HandoffError("heads_total differs from the model's KV heads")
        max_len = getattr(getattr(engine, "config", None), "max_model_len", None)
        if max_len is not None and len(self.prompt_ids) + len(self.output_ids) >= max_len:
            raise HandoffError("the request is longer than the importer's context")
        if len(self.kv) != len(runner.kv_caches):
            raise HandoffError("kv: layer count differs from the importer's")
        n = (self.num_computed + self.page_size - 1) // self.page_size
        for pair, mine in zip(self.kv, runner.kv_caches):
            if pair is None:
                continue
            if mine is None or mine[0] is None:
                raise HandoffError("kv: pages for a layer this rank does not hold")
            for t, m in zip(pair, mine):
                heads = t.shape[2]
                if t.shape[0] != n or t.shape[1] != self.page_size or t.shape[3] != m.shape[3] \
                        or heads < 1 or self.head_lo < 0 \
                        or self.head_lo + heads > self.heads_total:
                    raise HandoffError("kv: page tensor shape does not fit the request")
                if not t.dtype.is_floating_point:
                    raise HandoffError("kv: pages are floating point")


def _export_plane(plane: torch.Tensor, pages: torch.Tensor) -> torch.Tensor:
    """Pages of a cache plane as floating-point values (E4M3 planes are expanded with their
    page scales, so a hand-off is independent of either side's cache type)."""
    sel = plane.index_select(0, pages)
    scale = getattr(plane, "page_scale", None)
    if scale is None:
        return sel.clone()
    return (sel.view(torch.float8_e4m3fn).float() *
            scale.index_select(0, pages)[:, None, None, None]).to(torch.bfloat16)


def _import_plane(plane: torch.Tensor, idx: torch.Tensor, t: torch.Tensor) -> None:
    scale = getattr(plane, "page_scale", None)
    if scale is None:
        plane.index_copy_(0, idx, t.to(plane.dtype))
        return
    f = t.float()
    s = f.abs().amax(dim=(1, 2, 3)).clamp_min(1e-12) / 448.0
    q = (f / s[:, None, None, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    plane.index_copy_(0, idx, q.view(torch.uint8))
    scale.index_copy_(0, idx, s)


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
            kv.append((_export_plane(pair[0], pages), _export_plane(pair[1], pages)))
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


# ------------------------------------------------------------- several ranks --
# A tensor-parallel exporter lends one frame per rank (each holds a range of the KV heads).
# They travel as one body: ``SET_MAGIC | u32 count | count x u64 length | frames``; a body
# that starts with MAGIC is a set of one.  The importer re-cuts the head ranges for its own
# ranks, so the two sides need not share a tensor-parallel degree.
SET_MAGIC = b"USHS"
MAX_FRAMES = 64


def pack_frames(frames: list) -> bytes:
    frames = [bytes(f) for f in frames]
    if len(frames) == 1:
        return frames[0]
    return b"".join([SET_MAGIC, struct.pack("<I", len(frames)),
                     *[struct.pack("<Q", len(f)) for f in frames], *frames])


def unpack_frames(blob: bytes) -> list:
    blob = bytes(blob)
    if blob[:len(MAGIC)] == MAGIC:
        return [blob]
    if len(blob) < len(SET_MAGIC) + 4 or blob[:len(SET_MAGIC)] != SET_MAGIC:
        raise HandoffError("not a hand-off frame")
    (n,) = struct.unpack_from("<I", blob, len(SET_MAGIC))
    if not 1 <= n <= MAX_FRAMES or len(blob) < len(SET_MAGIC) + 4 + 8 * n:
        raise HandoffError("frame count outside the body")
    sizes = struct.unpack_from(f"<{n}Q", blob, len(SET_MAGIC) + 4)
    off = len(SET_MAGIC) + 4 + 8 * n
    if off + sum(sizes) != len(blob):
        raise HandoffError("frame lengths do not add up to the body")
    out = []
    for sz in sizes:
        out.append(blob[off:off + sz])
        off += sz
    return out


def handoffs_from_bytes(blob: bytes) -> list:
    """The hand-offs of every exporting rank, checked to describe one request and to cover
    the model's KV heads exactly once."""
    hs = [Handoff.from_bytes(f) for f in unpack_frames(blob)]
    first = hs[0]
    cover = []
    for h in hs:
        if (h.request_id, h.prompt_ids, h.output_ids, h.num_computed, h.page_size,
                h.heads_total) != (first.request_id, first.prompt_ids, first.output_ids,
                                   first.num_computed, first.page_size, first.heads_total):
            raise HandoffError("the frames describe different requests")
        pair = next((p for p in h.kv if p is not None), None)
        if pair is not None:
            cover.append((h.head_lo, h.head_lo + pair[0].shape[2]))
    cover.sort()
    at = 0
    for lo, hi in cover:
        if lo > at:
            raise HandoffError(f"KV heads [{at}, {lo}) are in no frame")
        at = max(at, hi)
    if cover and at != first.heads_total:
        raise HandoffError(f"KV heads [{at}, {first.heads_total}) are in no frame")
    return hs


def _params_of(d: dict) -> SamplingParams:
    """Sampling parameters back from their JSON form (token-id keys and tuples restored)."""
    d = dict(d)
    if d.get("logit_bias"):
        d["logit_bias"] = {int(k): float(v) for k, v in d["logit_bias"].items()}
    if d.get("stop_token_ids") is not None:
        d["stop_token_ids"] = tuple(int(x) for x in d["stop_token_ids"])
    return SamplingParams(**d)


def reshard_heads(shards: list, want_lo: int, want_n: int) -> torch.Tensor:
    """``shards``: (head_lo, tensor [pages, page, heads, D]) from the exporting ranks;
    returns heads [want_lo, want_lo + want_n) in order."""
    parts, at = [], want_lo
    for lo, t in sorted(shards, key=lambda s: s[0]):
        # heads already taken from an earlier shard are skipped (ranks that replicate a KV
        # head all export it)
        a, b = max(lo, at), min(lo + t.shape[2], want_lo + want_n)
        if a < b:
            parts.append(t[:, :, a - lo:b - lo])
            at = b
    got = sum(p.shape[2] for p in parts)
    assert got == want_n, f"head range [{want_lo}, {want_lo + want_n}) not covered ({got})"
    return parts[0] if len(parts) == 1 else torch.cat(parts, 2)


def import_request(engine, handoffs) -> str:
    """Continues a lent request on ``engine``.  ``handoffs``: one ``Handoff`` or the list
    of every exporting rank's (head ranges are re-cut for this rank)."""
    hs = handoffs if isinstance(handoffs, (list, tuple)) else [handoffs]
    h = hs[0]
    sch, runner, model = engine.scheduler, engine.runner, engine.model
    for x in hs:
        x.validate_for(engine)
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
            _import_plane(pair[which], idx, t.to(device=runner.device))
    rid = engine.add_request(h.prompt_ids, _params_of(h.params), request_id=h.request_id,
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
