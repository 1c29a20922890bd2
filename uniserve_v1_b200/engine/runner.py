"""Causal-LM runner: turns a scheduled batch into device work and reads results back.

Decode runs from CUDA graphs, one per (bucket size, sampling variant), captured
largest bucket first into one shared memory pool; a batch runs in the smallest
bucket that holds it.  Everything a graph needs from the host travels as one
pinned input block copied with a single H2D copy into fixed device addresses;
nothing is called back from a stream.  The graph also advances the device-side
step state (next input token, position, length, cache slot), so several steps can
be replayed back to back without the host.

Reference behaviour: crates/engine/src/runner/causal_lm.rs:2643 (start),
runner/graphs/mod.rs:957-1011 (prepare_inputs / replay), runner/buckets.rs:9-15
(smallest bucket), docs/architecture.md:141 (inputs travel as one copy) — reference
project paths.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..models.qwen3_moe import AttnMeta, Qwen3MoeModel
from ..ops import functional as F
from ..ops import native as N
from .scheduler import Batch
from .types import SamplingParams

DECODE_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)
# US_DECODE_MERGE=1 merges the decode attention's splits inside the attention kernel (the CTA
# that arrives last); measured 4 us per layer slower than the second launch behind
# programmatic dependent launch at 64 x 1024 keys, so the second launch is the default.
DECODE_MERGE_IN_KERNEL = __import__("os").environ.get("US_DECODE_MERGE", "0") == "1"


class DeviceStepError(RuntimeError):
    """The device status word was set during a step (``code``: see ``ops.native.STATUS_NAMES``)."""

    def __init__(self, code: int):
        self.code = code
        super().__init__(f"device status {code:#x}: {N.STATUS_NAMES.get(code, 'unknown')}")


class InputBlock:
    """Named views over one pinned host buffer and its fixed device twin."""

    def __init__(self, fields: list, device):
        self.device = torch.device(device)
        off = 0
        self.layout = {}
        for name, dtype, shape in fields:
            n = 1
            for s in shape:
                n *= s
            nbytes = n * torch.empty(0, dtype=dtype).element_size()
            off = (off + 15) & ~15
            self.layout[name] = (off, nbytes, dtype, shape)
            off += nbytes
        self.nbytes = (off + 15) & ~15
        pin = self.device.type == "cuda"
        self.host = torch.zeros(self.nbytes, dtype=torch.uint8, pin_memory=pin)
        self.dev = torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device)
        self.h = {k: self.host[o:o + nb].view(dt).view(shape)
                  for k, (o, nb, dt, shape) in self.layout.items()}
        self.d = {k: self.dev[o:o + nb].view(dt).view(shape)
                  for k, (o, nb, dt, shape) in self.layout.items()}
        self.hn = {k: v.numpy() for k, v in self.h.items()}

    def upload(self) -> int:
        self.dev.copy_(self.host, non_blocking=True)
        return self.nbytes


@dataclass
class DecodeGraph:
    graph: object
    variant: str
    bucket: int
    logits: Optional[torch.Tensor]
    sampled: torch.Tensor
    launches: int = 0


@dataclass
class DecodeStream:
    """Decode steps of one fixed set of rows, issued one at a time and read back one at a
    time (see ``CausalLmRunner.decode_begin``)."""
    rows: list
    n: int
    B: int
    blk: object
    graph: object
    variant: str
    launched: int = 0
    collected: int = 0
    limit: int = 0              # steps the rows have cache pages for
    draining: bool = False      # no further step is issued; the ones in flight are read
    events: list = field(default_factory=list)


class CausalLmRunner:
    def __init__(self, model: Qwen3MoeModel, num_pages: int, page_size: int = 16,
                 max_num_seqs: int = 128, max_model_len: int = 4096, use_graphs: bool = True,
                 history_steps: int = 64):
        self.model = model
        self.device = model.device
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_num_seqs = max_num_seqs
        self.max_model_len = max_model_len
        self.max_pages = (max_model_len + page_size - 1) // page_size
        self.kv_caches = model.new_kv_caches(num_pages, page_size)
        self.use_graphs = use_graphs and self.device.type == "cuda"
        self.buckets = [b for b in DECODE_BUCKETS if b < max_num_seqs] + [max_num_seqs]
        self.history_steps = history_steps
        # always-on counters of the places where the host waits for the device, by site
        # (reference: the blocking-call counters of the engine's profiling layer)
        self.blocking = {"decode_readback": 0, "stream_readback": 0, "to_host": 0}
        self.blocking_s = 0.0
        self._blocks: dict = {}
        self._graphs: dict = {}
        self._pool = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._readback = None
        # Called before every forward with (kind, rows, count): the disaggregated layout
        # hooks its step announcer in here so expert ranks can join (parallel/join.py).
        self.announce = lambda kind, rows, count=1: None
        self._scratch: dict = {}
        self._status_host = None
        if self.device.type == "cuda":
            N.kernels().us_status_ptr()       # allocate the status word before any capture
            from ..parallel import symm as _symm      # registers the status entry points
            self._status_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)

    # ---------------------------------------------------------------- blocks --
    def _decode_block(self, B: int) -> InputBlock:
        blk = self._blocks.get(B)
        if blk is None:
            i32, f32, i64 = torch.int32, torch.float32, torch.int64
            blk = InputBlock([
                ("input_ids", i32, (B,)), ("positions", i32, (B,)), ("slots", i32, (B,)),
                ("seq_lens", i32, (B,)), ("live", i32, (1,)), ("step", i32, (1,)),
                ("page_table", i32, (B, self.max_pages)),
                ("temperature", f32, (B,)), ("top_p", f32, (B,)), ("min_p", f32, (B,)),
                ("top_k", i32, (B,)), ("seeds", i64, (B,)), ("sample_pos", i64, (B,)),
            ], self.device)
            blk.history = torch.full((self.history_steps, B), -1, dtype=torch.int32,
                                     device=self.device)
            blk.readback = torch.empty((self.history_steps, B), dtype=torch.int32,
                                       pin_memory=self.device.type == "cuda")
            self._blocks[B] = blk
        return blk

    def bucket_for(self, n: int) -> int:
        for b in self.buckets:
            if n <= b:
                return b
        raise ValueError(f"no decode bucket holds {n} rows (largest {self.buckets[-1]})")

    # ----------------------------------------------------------- decode body --
    def _decode_body(self, blk: InputBlock, B: int, variant: str):
        """The one forward function: eager, rehearsal and capture all run this."""
        d = blk.d
        max_len = self.max_model_len
        splits = F.decode_splits(B, self.model.Hkv, max_len) if self.device.type == "cuda" else 1
        if self._persist_attention(B):
            splits = F.PERSIST_SPLITS
        scratch, counters = self._attn_scratch(B, splits)
        meta = AttnMeta(kind="decode", slots=d["slots"], page_table=d["page_table"],
                        seq_lens=d["seq_lens"], splits=splits, live=d["live"], scratch=scratch,
                        counters=counters)
        hidden = self.model.forward(d["input_ids"], d["positions"], meta, self.kv_caches)
        logits = None
        if variant == "greedy" and hasattr(self.model, "greedy_tokens"):
            sampled = self.model.greedy_tokens(hidden)      # sharded heads trade candidates only
        else:
            logits = self.model.logits(hidden)
        if variant == "greedy":
            if logits is not None:
                sampled = F.argmax(logits)
        elif variant == "sampled":
            if logits.is_cuda:
                F.logits_shape_(logits, temp=d["temperature"])
            else:
                logits = F.R.logits_shape(logits, temp=d["temperature"])
            sampled = F.sample_from_logits(logits, d["top_k"], d["top_p"], d["min_p"], d["seeds"],
                                           d["sample_pos"])
        else:                       # "logits": shaping and the draw happen outside
            return logits, None
        if sampled.device != self.device:
            sampled = sampled.to(self.device)
        # Device-side advance so the next step can run without the host.
        F.decode_advance_(sampled, d["input_ids"], d["positions"], d["seq_lens"], d["slots"],
                          d["page_table"], self.page_size, live=d["live"], history=blk.history,
                          step=d["step"])
        d["sample_pos"].add_(1)
        return logits, sampled

    def _persist_attention(self, B: int) -> bool:
        """Whether this runner's decode steps use the persistent attention kernel."""
        m = self.model
        if self.device.type != "cuda":
            return False
        kc = next((k for k, _ in (self.kv_caches or []) if k is not None), None)
        if kc is None or kc.dtype != torch.bfloat16:
            return False
        # with few (sequence, kv head) pairs a CTA would stream only a few tiles and the
        # kernel's fixed cost (tile list, merge of the cut pairs) outweighs its ring: the split
        # kernel stays (measured at 1100 keys: 64 pairs 24.6 us split four ways against 27.6 us
        # persistent, 128 pairs 35.8 us either way alone but a 2-GPU decode step 10.56 against
        # 10.85 ms, 256 pairs a 1-GPU step 14.65 against 14.29 ms, 512 pairs 84.9 against 80.0 us)
        if B * m.Hkv < F.PERSIST_MIN_PAIRS:
            return False
        return F.decode_persist_ok(B, m.Hq, m.Hkv, m.D, kc.shape[1],
                                   int(getattr(m.cfg, "sliding_window", 0) or 0))

    def _attn_scratch(self, B: int, splits: int):
        """Split-KV partials and arrival counters of the decode attention, one pair per
        (bucket, splits), shared by every layer (allocated outside any capture)."""
        m = self.model
        if self.device.type == "cuda" and splits == F.PERSIST_SPLITS:
            key = (B, splits)
            got = self._scratch.get(key)
            if got is None:
                got = F.decode_persist_scratch(B, m.Hkv, self.device)
                self._scratch[key] = got
            return got
        if self.device.type != "cuda" or splits <= 1 or m.D != 128:
            return None, None
        key = (B, splits)
        got = self._scratch.get(key)
        if got is None:
            got = F.decode_scratch(B, m.Hq, m.Hkv, m.D, splits, self.device)
            if not DECODE_MERGE_IN_KERNEL:
                got = (got[0], None)
            self._scratch[key] = got
        return got

    def check_device_status(self) -> None:
        """Raises when the status word copied behind the step's results is set: a bounded
        device wait ran out (a peer more than the budget late, or gone), so the step's
        tokens are not to be trusted.  The word is cleared so the next engine starts clean."""
        code = int(self._status_host[0]) if self._status_host is not None else 0
        if code:
            self._status_host[0] = 0
            N.kernels().us_status_clear_async(N.stream())
            raise DeviceStepError(code)

    def _decode_kind(self, kind: str, B: int) -> str:
        """Announcement kind of a decode-step forward: expert ranks must know when the step runs
        as two half-batches (they then serve two windows per layer)."""
        micro = bool(getattr(self.model, "microbatch_now", False)) and \
            bool(getattr(self.model, "micro_exchanges", None)) and B >= 2 and B % 2 == 0
        return kind + "+micro" if micro else kind

    def _queue_status_copy(self) -> None:
        if self._status_host is not None:
            N.kernels().us_status_copy_async(N.ptr(self._status_host), N.stream())

    def _graph(self, B: int, variant: str) -> Optional[DecodeGraph]:
        if not self.use_graphs:
            return None
        # a union's micro-batched steps issue other kernels than its plain steps of the same size
        key = (B, variant, bool(getattr(self.model, "microbatch_now", False)))
        g = self._graphs.get(key)
        if g is not None:
            return g
        blk = self._decode_block(B)
        # Rehearse on a side stream (loads modules, sizes workspaces), then capture.
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        saved = blk.dev.clone()
        # Inert inputs: no row is live, no cache slot is written.
        blk.dev.zero_()
        blk.d["slots"].fill_(-1)
        torch.cuda.synchronize()
        self.announce(self._decode_kind("eager", B), B)
        with torch.cuda.stream(s):
            self._decode_body(blk, B, variant)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        blk.dev.copy_(saved)
        graph = torch.cuda.CUDAGraph()
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        before = N.launch_count
        self.announce(self._decode_kind("capture", B), B)
        with torch.cuda.graph(graph, pool=self._pool):
            logits, sampled = self._decode_body(blk, B, variant)
        launches = N.launch_count - before
        blk.dev.copy_(saved)
        torch.cuda.synchronize()
        N.raise_on_device_error()
        g = DecodeGraph(graph, variant, B, logits, sampled, launches)
        self._graphs[key] = g
        return g

    def warm_up(self, variants=("greedy",), buckets=None) -> None:
        """Captures largest first so smaller graphs reuse the big ones' memory."""
        for B in sorted(buckets or self.buckets, reverse=True):
            for v in variants:
                self._graph(B, v)

    # ---------------------------------------------------------------- decode --
    def _fill_decode(self, blk: InputBlock, rows: list, B: int) -> None:
        """Column assembly of a decode batch into the pinned input block (numpy
        views over the pinned memory; one pass over the rows)."""
        h = blk.hn
        n = len(rows)
        ps = self.page_size
        h["live"][0] = n
        h["step"][0] = 0
        ids, pos, slots, temp, top_k, top_p, min_p, seeds = [], [], [], [], [], [], [], []
        pt = h["page_table"]
        # A row of the page table is rewritten only when its request or its page list
        # changed; a list that grew gets its new tail (page lists only ever append, and a
        # preempted or imported request owns a new list object).
        held = blk.__dict__.setdefault("_pt_rows", {})
        for i, req in enumerate(rows):
            p_ = req.num_tokens - 1
            ids.append(req.output_ids[-1] if req.output_ids else req.prompt_ids[-1])
            pos.append(p_)
            pages = req.pages
            slots.append(pages[p_ // ps] * ps + p_ % ps)
            was = held.get(i)
            n_p = len(pages)
            if was is not None and was[0] is pages and was[1] <= n_p:
                if was[1] < n_p:
                    pt[i, was[1]:n_p] = pages[was[1]:]
            else:
                pt[i, :n_p] = pages
            held[i] = (pages, n_p)
            p: SamplingParams = req.params
            greedy = p.greedy
            temp.append(1.0 if greedy else p.temperature)
            top_k.append(1 if greedy else (p.top_k if p.top_k > 0 else 0))
            top_p.append(p.top_p)
            min_p.append(p.min_p)
            sd = req.seed
            seeds.append(sd - (1 << 64) if sd >= (1 << 63) else sd)
        h["input_ids"][:n] = ids
        h["positions"][:n] = pos
        h["seq_lens"][:n] = pos
        h["seq_lens"][:n] += 1
        h["slots"][:n] = slots
        h["temperature"][:n] = temp
        h["top_k"][:n] = top_k
        h["top_p"][:n] = top_p
        h["min_p"][:n] = min_p
        h["seeds"][:n] = seeds
        h["sample_pos"][:n] = pos
        h["sample_pos"][:n] += 1
        if n < B:
            h["input_ids"][n:] = 0
            h["positions"][n:] = 0
            h["seq_lens"][n:] = 0
            h["slots"][n:] = -1
            h["temperature"][n:] = 1.0
            h["top_k"][n:] = 1
            h["top_p"][n:] = 1.0
            h["min_p"][n:] = 0.0

    # ---------------------------------------------------------------- KV tiers --
    def enable_host_tier(self, slots: int) -> None:
        """Host-memory copies of evicted prefix pages: one [slots, page, heads, dim] pair per
        layer this rank owns, pinned on a GPU deployment."""
        self.host_kv = []
        for kc, vc in self.kv_caches:
            if kc is None:
                self.host_kv.append((None, None))
                continue
            shape = (slots,) + tuple(kc.shape[1:])
            hk = torch.zeros(shape, dtype=kc.dtype)
            hv = torch.zeros(shape, dtype=vc.dtype)
            if self.device.type == "cuda":
                hk, hv = hk.pin_memory(), hv.pin_memory()
            if getattr(kc, "page_scale", None) is not None:      # E4M3 pages travel with scales
                hk.page_scale = torch.zeros(slots, dtype=torch.float32)
                hv.page_scale = torch.zeros(slots, dtype=torch.float32)
            self.host_kv.append((hk, hv))

    def apply_kv_moves(self, offloads: list, fetches: list) -> None:
        """Copies decided by the block manager, in order: device pages about to be reused go
        to their host slots, then host slots come back into freshly pinned device pages.
        Runs on the compute stream before the step that reuses the pages."""
        if not offloads and not fetches:
            return
        dev = self.device
        if offloads:
            pages = torch.tensor([p for p, _ in offloads], dtype=torch.long, device=dev)
            slots = torch.tensor([s for _, s in offloads], dtype=torch.long)
            for (kc, vc), (hk, hv) in zip(self.kv_caches, self.host_kv):
                if kc is None:
                    continue
                hk[slots] = kc.index_select(0, pages).to("cpu")
                hv[slots] = vc.index_select(0, pages).to("cpu")
                if getattr(kc, "page_scale", None) is not None:
                    hk.page_scale[slots] = kc.page_scale.index_select(0, pages).to("cpu")
                    hv.page_scale[slots] = vc.page_scale.index_select(0, pages).to("cpu")
            self.d2h_bytes += sum(2 * len(offloads) * kc[0].numel() * kc.element_size()
                                  for kc, _ in self.kv_caches if kc is not None)
        if fetches:
            slots = torch.tensor([s for s, _ in fetches], dtype=torch.long)
            pages = torch.tensor([p for _, p in fetches], dtype=torch.long, device=dev)
            for (kc, vc), (hk, hv) in zip(self.kv_caches, self.host_kv):
                if kc is None:
                    continue
                kc.index_copy_(0, pages, hk[slots].to(dev, non_blocking=True))
                vc.index_copy_(0, pages, hv[slots].to(dev, non_blocking=True))
                if getattr(kc, "page_scale", None) is not None:
                    kc.page_scale.index_copy_(0, pages, hk.page_scale[slots].to(dev))
                    vc.page_scale.index_copy_(0, pages, hv.page_scale[slots].to(dev))
            self.h2d_bytes += sum(2 * len(fetches) * kc[0].numel() * kc.element_size()
                                  for kc, _ in self.kv_caches if kc is not None)

    def release_graphs(self) -> None:
        """Drops every captured graph (do this before tearing down a process
        group whose collectives the graphs captured)."""
        self._graphs.clear()
        self._pool = None

    @staticmethod
    def variant_for(rows: list) -> str:
        if any(r.params.needs_shaping or r.params.logprobs for r in rows):
            return "logits"
        return "greedy" if all(r.params.greedy for r in rows) else "sampled"

    def decode(self, rows: list, steps: int = 1, capacity: Optional[int] = None):
        """Runs ``steps`` decode steps for ``rows`` (requests); returns
        (tokens [steps, n] on the host, logprob info or None).  ``capacity``: the row count
        the step was agreed to run at (an expert union steps with one capacity on every
        member); rows past ``len(rows)`` are padding.  With no rows at all the forward is a
        *join*: every kernel of the step is issued with zero live rows."""
        n = len(rows)
        B = capacity if capacity is not None else self.bucket_for(n)
        assert n <= B
        blk = self._decode_block(B)
        variant = self.variant_for(rows) if rows else "greedy"
        assert steps == 1 or variant != "logits"
        assert steps <= self.history_steps
        self._fill_decode(blk, rows, B)
        g = self._graph(B, variant) if B <= self.buckets[-1] or B in self._graphs else None
        self.h2d_bytes += blk.upload()
        logits = sampled = None
        self.announce(self._decode_kind("replay" if g is not None else "eager", B), B, steps)
        for _ in range(steps):
            if g is not None:
                g.graph.replay()
                N.launch_count += g.launches
                logits, sampled = g.logits, g.sampled
            else:
                logits, sampled = self._decode_body(blk, B, variant)
        info = None
        if variant == "logits":
            sampled, info = self._shape_and_sample(logits[:n], rows)
            out = sampled.view(1, n)
        elif self.device.type == "cuda":
            # one D2H copy of the step results into a fixed pinned buffer
            host = blk.readback[:steps]
            host.copy_(blk.history[:steps], non_blocking=True)
            self._queue_status_copy()          # read with the tokens, no extra synchronisation
            self._wait(torch.cuda.current_stream().synchronize, "decode_readback")
            self.check_device_status()
            self.d2h_bytes += steps * n * 4 + 4
            out = host[:, :n]
        else:
            out = blk.history[:steps, :n].clone()
        return out, info

    # ------------------------------------------------ decode steps in flight --
    def decode_begin(self, rows: list) -> "DecodeStream":
        """Uploads the step state of ``rows`` once; ``decode_launch`` then issues one decode
        step at a time (the device advances positions, slots and input tokens itself) and
        ``decode_collect`` reads a step's tokens once its own copy has landed - so the host
        can issue step k + 1 before it has read step k."""
        n = len(rows)
        B = self.bucket_for(n)
        blk = self._decode_block(B)
        variant = self.variant_for(rows)
        assert variant != "logits"
        self._fill_decode(blk, rows, B)
        g = self._graph(B, variant) if B <= self.buckets[-1] or B in self._graphs else None
        self.h2d_bytes += blk.upload()
        return DecodeStream(rows=list(rows), n=n, B=B, blk=blk, graph=g, variant=variant)

    def decode_launch(self, st: "DecodeStream") -> None:
        k = st.launched
        assert k < self.history_steps
        self.announce(self._decode_kind("replay" if st.graph is not None else "eager", st.B), st.B, 1)
        if st.graph is not None:
            st.graph.graph.replay()
            N.launch_count += st.graph.launches
        else:
            self._decode_body(st.blk, st.B, st.variant)
        if self.device.type == "cuda":
            st.blk.readback[k:k + 1].copy_(st.blk.history[k:k + 1], non_blocking=True)
            self._queue_status_copy()
            ev = torch.cuda.Event()
            ev.record()
            st.events.append(ev)
        st.launched += 1

    def decode_collect(self, st: "DecodeStream", k: int) -> list:
        """Tokens of step ``k`` (one per row of the stream), on the host."""
        assert k < st.launched
        if self.device.type == "cuda":
            self._wait(st.events[k].synchronize, "stream_readback")
            self.check_device_status()
            self.d2h_bytes += st.n * 4 + 4
            return st.blk.readback[k, :st.n].tolist()
        return st.blk.history[k, :st.n].tolist()

    def _to_host(self, t: torch.Tensor) -> torch.Tensor:
        host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        host.copy_(t, non_blocking=True)
        self._queue_status_copy()
        self._wait(torch.cuda.current_stream().synchronize, "to_host")
        self.check_device_status()
        self.d2h_bytes += host.numel() * host.element_size()
        return host

    def _wait(self, fn, site: str) -> None:
        """A host wait on the device, counted by site with the time it took."""
        import time as _time
        t0 = _time.perf_counter()
        fn()
        self.blocking[site] += 1
        self.blocking_s += _time.perf_counter() - t0

    # ------------------------------------------------ shaping outside graphs --
    def _shape_and_sample(self, logits: torch.Tensor, rows: list):
        """Rows with penalties, bias, bans or logprobs: vLLM order on the device,
        then the same draw kernel.  Logprobs are taken on the raw distribution."""
        dev = logits.device
        n, V = logits.shape
        raw = logits
        shaped = logits.clone()
        need_counts = any(r.params.repetition_penalty != 1.0 or r.params.frequency_penalty != 0.0
                          or r.params.presence_penalty != 0.0 for r in rows)
        ban = torch.zeros(n, V, dtype=torch.uint8)
        any_ban = False
        counts = torch.zeros(n, V, dtype=torch.int16) if need_counts else None
        pmask = torch.zeros(n, V, dtype=torch.uint8) if need_counts else None
        bo, bi, bv = [0], [], []
        eos = getattr(self, "eos_token_id", None)
        for i, r in enumerate(rows):
            p = r.params
            if p.allowed_token_ids:
                ban[i] = 1
                ban[i, torch.tensor(p.allowed_token_ids)] = 0
                any_ban = True
            for w in (p.bad_words_ids or []):
                if len(w) == 1:
                    ban[i, w[0]] = 1
                    any_ban = True
                elif len(w) > 1 and r.all_ids[-(len(w) - 1):] == list(w[:-1]):
                    ban[i, w[-1]] = 1
                    any_ban = True
            if len(r.output_ids) < p.min_tokens:
                for t in ([eos] if eos is not None else []) + list(p.stop_token_ids):
                    ban[i, t] = 1
                    any_ban = True
            for tok, val in (p.logit_bias or {}).items():
                bi.append(int(tok))
                bv.append(float(val))
            bo.append(len(bi))
            if need_counts:
                if r.output_ids:
                    counts[i] = torch.bincount(torch.tensor(r.output_ids), minlength=V)[:V].to(torch.int16)
                pmask[i, torch.tensor(r.prompt_ids)] = 1
        f32 = lambda xs: torch.tensor(xs, dtype=torch.float32, device=dev)
        temp = f32([1.0 if r.params.greedy else r.params.temperature for r in rows])
        kw = dict(ban_mask=ban.to(dev) if any_ban else None,
                  out_counts=counts.to(dev) if need_counts else None,
                  prompt_mask=pmask.to(dev) if need_counts else None,
                  rep=f32([r.params.repetition_penalty for r in rows]) if need_counts else None,
                  freq=f32([r.params.frequency_penalty for r in rows]) if need_counts else None,
                  pres=f32([r.params.presence_penalty for r in rows]) if need_counts else None,
                  temp=temp)
        if dev.type == "cuda":
            csr = None
            if bi:
                csr = (torch.tensor(bo, dtype=torch.int32, device=dev),
                       torch.tensor(bi, dtype=torch.int32, device=dev), f32(bv))
            F.logits_shape_(shaped, bias_csr=csr, **kw)
        else:
            bias = [[(bi[j], bv[j]) for j in range(bo[i], bo[i + 1])] for i in range(n)] if bi else None
            shaped = F.R.logits_shape(shaped, bias=bias, **kw)
        top_k = torch.tensor([1 if r.params.greedy else max(r.params.top_k, 0) for r in rows],
                             dtype=torch.int32, device=dev)
        top_p = f32([r.params.top_p for r in rows])
        min_p = f32([r.params.min_p for r in rows])
        seeds = torch.tensor([r.seed - (1 << 64) if r.seed >= (1 << 63) else r.seed for r in rows],
                             dtype=torch.int64, device=dev)
        pos = torch.tensor([r.num_tokens for r in rows], dtype=torch.int64, device=dev)
        sampled = F.sample_from_logits(shaped, top_k, top_p, min_p, seeds, pos)
        sampled = sampled.to(dev)
        info = None
        if any(r.params.logprobs for r in rows):
            lse, lp, rank = F.logprob_stats(raw, sampled)
            kmax = max([r.params.top_logprobs for r in rows] + [0])
            top = None
            if kmax > 0:
                tv, ti = torch.topk(raw.float(), kmax, dim=-1)
                top = ((tv - lse[:, None]).cpu(), ti.cpu())
            lp_c, rank_c = lp.cpu(), rank.cpu()
            info = {}
            for i, r in enumerate(rows):
                if not r.params.logprobs:
                    continue
                tops = []
                if top is not None:
                    k = r.params.top_logprobs
                    tops = [(int(top[1][i, j]), float(top[0][i, j])) for j in range(k)]
                info[r.request_id] = (float(lp_c[i]), int(rank_c[i]), tops)
        if dev.type == "cuda":
            host = self._to_host(sampled)
        else:
            host = sampled.cpu()
        return host, info

    # --------------------------------------------------------------- prefill --
    def join(self, capacity: int) -> None:
        """An idle member's part of an agreed step: the whole forward with zero live rows."""
        self.decode([], 1, capacity=capacity)

    def prefill(self, chunks: list, capacity: Optional[int] = None):
        """Eager varlen prefill of the scheduled chunks; returns (tokens for the
        chunks that sample, in chunk order, on the host; logprob info).  ``capacity`` pads
        the rows to an agreed count (padding rows write no cache slot and route nowhere)."""
        dev = self.device
        ps = self.page_size
        ids, pos, slots, cu_q, cu_k, ctx, last_rows, sample_rows = [], [], [], [0], [0], [], [], []
        max_q = max_k = 0
        for c in chunks:
            req = c.request
            toks = req.all_ids[c.start:c.start + c.length]
            ids.extend(toks)
            pos.extend(range(c.start, c.start + c.length))
            for p_ in range(c.start, c.start + c.length):
                slots.append(req.pages[p_ // ps] * ps + p_ % ps)
            cu_q.append(cu_q[-1] + c.length)
            cu_k.append(cu_k[-1] + c.start + c.length)
            ctx.append(c.start)
            max_q = max(max_q, c.length)
            max_k = max(max_k, c.start + c.length)
            if c.sample:
                last_rows.append(cu_q[-1] - 1)
                sample_rows.append(req)
        T_real = len(ids)
        live = None
        if capacity is not None:
            assert T_real <= capacity, (T_real, capacity)
            pad = capacity - T_real
            ids, pos, slots = ids + [0] * pad, pos + [0] * pad, slots + [-1] * pad
            live = torch.tensor([T_real], dtype=torch.int32, device=dev)
        T = len(ids)
        i32 = torch.int32
        packed = torch.tensor(ids + pos + slots + cu_q + cu_k, dtype=i32,
                              pin_memory=dev.type == "cuda")
        d = packed.to(dev, non_blocking=True)
        self.h2d_bytes += packed.numel() * 4
        nq = len(cu_q)
        page_table = None
        if any(c > 0 for c in ctx):
            page_table = torch.zeros(len(chunks), self.max_pages, dtype=i32)
            for i, c in enumerate(chunks):
                page_table[i, :len(c.request.pages)] = torch.tensor(c.request.pages, dtype=i32)
            page_table = page_table.to(dev)
        meta = AttnMeta(kind="prefill", slots=d[2 * T:3 * T], cu_q=d[3 * T:3 * T + nq],
                        cu_k=d[3 * T + nq:3 * T + 2 * nq], max_q=max_q, max_k=max_k,
                        context_lens=ctx, page_table=page_table, live=live, rows_real=T_real)
        if page_table is not None and dev.type == "cuda":
            from ..ops.attention import context_tables
            meta.ctx_tables = context_tables(ctx, cu_q, cu_k, dev)
            self.h2d_bytes += 4 * len(cu_q) + 8 * T_real
        self.announce("eager", T)
        hidden = self.model.forward(d[:T], d[T:2 * T], meta, self.kv_caches)
        tap = getattr(self, "hidden_tap", None)
        if tap is not None:          # a drafter that feeds on the target's states (MTP head)
            for i, c in enumerate(chunks):
                tap(c.request, c.start, hidden[cu_q[i]:cu_q[i + 1]])
        if not sample_rows:
            return None, None, []
        rows_idx = torch.tensor(last_rows, dtype=i32, device=dev)
        last = F.gather_rows(hidden, rows_idx)
        logits = self.model.logits(last)
        if self.variant_for(sample_rows) == "greedy":
            toks = F.argmax(logits)
            host = self._to_host(toks) if dev.type == "cuda" else toks
            return host, None, sample_rows
        host, info = self._shape_and_sample(logits, sample_rows)
        return host, info, sample_rows

    # ----------------------------------------------------------------- verify --
    def verify(self, rows: list, drafts: list, want_hidden: bool = False):
        """Speculative verification: request ``rows[i]`` runs its last token followed by
        ``drafts[i]`` (positions num_tokens - 1 ...) in one causal chunk over its cached
        context; returns the greedy token after every position, one list per request (and
        with ``want_hidden`` the hidden rows of those positions, for drafters that feed on
        the target's state)."""
        dev, ps = self.device, self.page_size
        ids, pos, slots, cu_q, cu_k, ctx = [], [], [], [0], [0], []
        max_q = max_k = 0
        for req, dr in zip(rows, drafts):
            start = req.num_tokens - 1
            toks = [req.all_ids[-1]] + [int(t) for t in dr]
            ids.extend(toks)
            pos.extend(range(start, start + len(toks)))
            for p_ in range(start, start + len(toks)):
                slots.append(req.pages[p_ // ps] * ps + p_ % ps)
            cu_q.append(cu_q[-1] + len(toks))
            cu_k.append(cu_k[-1] + start + len(toks))
            ctx.append(start)
            max_q = max(max_q, len(toks))
            max_k = max(max_k, start + len(toks))
        T = len(ids)
        i32 = torch.int32
        packed = torch.tensor(ids + pos + slots + cu_q + cu_k, dtype=i32,
                              pin_memory=dev.type == "cuda")
        d = packed.to(dev, non_blocking=True)
        self.h2d_bytes += packed.numel() * 4
        nq = len(cu_q)
        page_table = torch.zeros(len(rows), self.max_pages, dtype=i32)
        for i, req in enumerate(rows):
            page_table[i, :len(req.pages)] = torch.tensor(req.pages, dtype=i32)
        meta = AttnMeta(kind="prefill", slots=d[2 * T:3 * T], cu_q=d[3 * T:3 * T + nq],
                        cu_k=d[3 * T + nq:3 * T + 2 * nq], max_q=max_q, max_k=max_k,
                        context_lens=ctx, page_table=page_table.to(dev))
        if dev.type == "cuda":
            from ..ops.attention import context_tables
            meta.ctx_tables = context_tables(ctx, cu_q, cu_k, dev)
            self.h2d_bytes += 4 * len(cu_q) + 8 * T
        self.announce("eager", T)
        hidden = self.model.forward(d[:T], d[T:2 * T], meta, self.kv_caches)
        toks = F.argmax(self.model.logits(hidden))
        host = (self._to_host(toks) if dev.type == "cuda" else toks).tolist()
        self.d2h_bytes += T * 4
        out = [host[cu_q[i]:cu_q[i + 1]] for i in range(len(rows))]
        if want_hidden:       # the target's states of the verified positions, per request
            return out, [hidden[cu_q[i]:cu_q[i + 1]] for i in range(len(rows))]
        return out

    # ---------------------------------------------------------------- execute --
    def execute(self, batch: Batch, capacity: Optional[int] = None):
        """Returns (sampled {request_id: token}, logprobs {request_id: info})."""
        sampled, lps = {}, {}
        if batch.kind == "decode":
            rows = [c.request for c in batch.chunks]
            toks, info = self.decode(rows, 1, capacity=capacity)
            for i, r in enumerate(rows):
                sampled[r.request_id] = int(toks[0, i])
            lps = info or {}
        else:
            toks, info, rows = self.prefill(batch.chunks, capacity=capacity)
            for i, r in enumerate(rows):
                sampled[r.request_id] = int(toks[i])
            lps = info or {}
        return sampled, lps
