"""Prefill / decode disaggregation on CPU engines: a request that moves after its first
token produces what one engine produces."""
import pytest
import torch

from uniserve_v1_b200.engine.engine import LLMEngine
from uniserve_v1_b200.engine.handoff import (Handoff, PrefillDecodePair, export_request,
                                             import_request, reshard_heads)
from uniserve_v1_b200.engine.types import SamplingParams
from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel


def _engines(n):
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    mk = lambda: LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=160,
                           use_graphs=False)
    return [mk() for _ in range(n)]


def test_prefill_decode_pair_matches_one_engine():
    single, pre, dec = _engines(3)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (7, 33, 16)]
    params = [SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True),
              SamplingParams(temperature=0.8, top_p=0.9, seed=11, max_tokens=12, ignore_eos=True),
              SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)]
    ref = single.generate(prompts, params)
    for through_bytes in (False, True):
        pre, dec = _engines(2)
        pair = PrefillDecodePair(pre, dec, through_bytes=through_bytes)
        rids = [pair.add_request(p, sp, request_id=f"req-{i + 1}")
                for i, (p, sp) in enumerate(zip(prompts, params))]
        outs = {r: [] for r in rids}
        while pair.has_work():
            for o in pair.step():
                outs[o.request_id].extend(o.new_token_ids)
        assert [outs[r] for r in rids] == ref
        assert pair.moved == 2 and pair.moved_bytes > 0     # the one-token request ends in place
        assert pre.blocks.num_free == dec.blocks.num_free == _engines(1)[0].blocks.num_free
        assert not pre.scheduler.running and not dec.scheduler.running   # nothing leaks
        assert dec.scheduler.stats["prefill_tokens"] <= 2   # the decode side computed no prompt


def test_handoff_frames_and_head_ranges():
    pre, dec = _engines(2)
    rid = pre.add_request(list(range(5, 45)), SamplingParams(temperature=0.0, max_tokens=4,
                                                            ignore_eos=True))
    while not pre.scheduler.requests[rid].output_ids:
        pre.step()
    h = export_request(pre, rid, release=False)
    assert h.num_computed == 40 and h.kv[0][0].shape[:2] == (3, 16)
    back = Handoff.from_bytes(h.to_bytes())
    assert back.prompt_ids == h.prompt_ids and torch.equal(back.kv[1][1], h.kv[1][1])
    # two exporting ranks with one head each feed an importer that owns both
    k = h.kv[0][0]
    whole = reshard_heads([(1, k[:, :, 1:2]), (0, k[:, :, 0:1])], 0, 2)
    assert torch.equal(whole, k)
    assert torch.equal(reshard_heads([(0, k)], 1, 1), k[:, :, 1:2])
    halves = []
    for lo in (0, 1):
        part = Handoff(**{**h.__dict__, "head_lo": lo,
                          "kv": [(a[:, :, lo:lo + 1], b[:, :, lo:lo + 1]) for a, b in h.kv]})
        halves.append(part)
    import_request(dec, halves)
    out = []
    while dec.has_work():
        for o in dec.step():
            out.extend(o.new_token_ids)
    ref = []
    while pre.has_work():
        for o in pre.step():
            ref.extend(o.new_token_ids)
    assert out == ref and len(out) == 3


def test_frame_is_explicit_and_validated():
    """The framed state is a JSON header plus raw tensor bytes: it round-trips, a pickle
    stream or a truncated body is refused, and fields that do not fit the importing engine
    (token outside the vocabulary, wrong page size, too many KV heads, more computed
    positions than tokens, page tensors of the wrong shape) are refused before any page is
    written."""
    import dataclasses
    import pickle
    import pytest
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.handoff import (Handoff, HandoffError, export_request,
                                                  import_request)
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    mk = lambda: LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=256, use_graphs=False)
    a, b = mk(), mk()
    rid = a.add_request(list(range(5, 40)), SamplingParams(temperature=0.0, max_tokens=6,
                                                           ignore_eos=True, logit_bias={7: 1.5},
                                                           stop_token_ids=(3,)))
    while not a.scheduler.requests[rid].output_ids:
        a.step()
    h = export_request(a, rid)
    blob = h.to_bytes()
    assert blob[:4] == b"USHO" and b"torch" not in blob[:200]
    g = Handoff.from_bytes(blob)
    assert g.prompt_ids == h.prompt_ids and g.num_computed == h.num_computed
    assert all(torch.equal(x[0], y[0]) and torch.equal(x[1], y[1]) for x, y in zip(g.kv, h.kv) if x)
    for bad in (pickle.dumps({"request_id": "x"}), blob[:40], b"USHO\x01" + b"\xff" * 8, b""):
        with pytest.raises(HandoffError):
            Handoff.from_bytes(bad)
    free = b.blocks.num_free
    for change in ({"prompt_ids": [10 ** 9] + g.prompt_ids[1:]}, {"page_size": g.page_size * 2},
                   {"heads_total": g.heads_total + 64}, {"num_computed": 10 ** 6},
                   {"head_lo": g.heads_total}, {"kv": [None] * (len(g.kv) + 1)},
                   {"kv": [(k[:1], v[:1]) if k is not None else None
                           for k, v in (p or (None, None) for p in g.kv)]}):
        with pytest.raises(HandoffError):
            import_request(b, dataclasses.replace(g, **change))
    assert b.blocks.num_free == free
    import_request(b, g)                         # the honest state still imports
    while b.has_work():
        b.step()


def test_copy_manifests_cover_every_layout_pair_and_route_a_handoff():
    """Resharding plans between tensor-parallel degrees (with replicated heads above the head
    count): every destination head written once from a holder; replicated sources are spread;
    routed through a real hand-off, an importer gets exactly the shards it needs."""
    from uniserve_v1_b200.engine.manifest import CopyManifest, head_range
    for heads in (1, 2, 4, 8):
        for src in (1, 2, 4, 8, 16):
            for dst in (1, 2, 4, 8, 16):
                m = CopyManifest.plan(heads, src, dst)
                m.check()
    m = CopyManifest.plan(4, 2, 4)              # each source rank feeds two destination ranks
    assert [m.sources_of(d) for d in range(4)] == [[0], [0], [1], [1]]
    m = CopyManifest.plan(4, 4, 1)
    assert m.sources_of(0) == [0, 1, 2, 3] and sum(c.heads for c in m.copies) == 4
    m = CopyManifest.plan(2, 8, 2)              # the source replicates each head four times
    assert len(m.copies) == 2 and {c.src_rank for c in m.copies} == {0, 7} or \
        {c.src_rank // 4 for c in m.copies} == {0, 1}
    assert head_range(2, 8, 5) == (1, 1) and head_range(8, 2, 1) == (4, 4)
    assert CopyManifest.plan(8, 2, 4).bytes_moved(pages=3, page_size=16, head_dim=128, layers=2) \
        == 8 * 2 * 3 * 16 * 128 * 2 * 2
    # a TP1 export cut into the two shards a TP2 exporter would send, routed to a TP1 importer
    pre, dec = _engines(2)
    rid = pre.add_request(list(range(5, 45)), SamplingParams(temperature=0.0, max_tokens=4,
                                                            ignore_eos=True))
    while not pre.scheduler.requests[rid].output_ids:
        pre.step()
    h = export_request(pre, rid, release=False)
    H = h.heads_total
    shards = {}
    for r in range(2):
        lo, n = head_range(H, 2, r)
        shards[r] = Handoff(**{**h.__dict__, "head_lo": lo,
                               "kv": [None if p is None else (p[0][:, :, lo:lo + n], p[1][:, :, lo:lo + n])
                                      for p in h.kv]})
    routed = CopyManifest.plan(H, 2, 1).route(shards)
    assert list(routed) == [0] and len(routed[0]) == 2
    new = import_request(dec, routed[0])
    ref = pre.generate([list(range(5, 45))], SamplingParams(temperature=0.0, max_tokens=4,
                                                            ignore_eos=True))[0]
    out = list(dec.scheduler.requests[new].output_ids)
    while dec.has_work():
        for o in dec.step():
            out.extend(o.new_token_ids)
    assert out == ref


# ------------------------------------------------- between tensor-parallel degrees --
def _tp_rank(rank, world, port, q, mode, body):
    """One rank of a 2-way tensor-parallel replicated engine.  mode "lend": compute the
    prompt and the first token, lend the request (every rank its KV heads).  mode "take":
    continue a request that a single-rank engine lent."""
    import os
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.parallel.context import ParallelContext
    from uniserve_v1_b200.server import multirank as MR
    r, w, dev, control = MR.init_rank()
    ctx = ParallelContext.from_world(tensor=world, expert_over_tensor=True)
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32, ctx).init_random(seed=0)
    eng = LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=128, use_graphs=False)
    bus = MR.CommandBus(control, r)
    import torch.distributed as dist

    def leave():            # an orderly end: no rank closes its sockets under the other
        dist.barrier()
        dist.destroy_process_group()

    if r != 0:
        MR.follower_loop(eng, bus)
        leave()
        return
    rep = MR.ReplicatedEngine(eng, bus)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    if mode == "lend":
        rid = rep.add_request(_PROMPT, sp)
        first = []
        while not first:
            for o in rep.step():
                first.extend(o.new_token_ids)
        blob = rep.export_request(rid)
        assert rid not in eng.scheduler.requests           # lent: gone on this side
        rep.shutdown()
        q.put((first, blob))
        leave()
        return
    rid = rep.import_request("moved-1", body)
    toks = []
    while rep.has_work():
        for o in rep.step():
            toks.extend(o.new_token_ids)
    try:
        rep.import_request("moved-2", body[:-7])              # a cut body: every rank refuses it
        refused = False
    except Exception:
        refused = True
    rep.shutdown()
    q.put((toks, refused))
    leave()


_PROMPT = [3, 17, 91, 250, 8, 8, 41, 700, 12, 5, 66, 301, 2, 19, 77, 123, 9, 4, 1000, 55]


def _spawn_tp(mode, body=None):
    import socket
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_tp_rank, args=(r, 2, port, q, mode, body)) for r in range(2)]
    for p in procs:
        p.start()
    out = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return out


def test_handoff_between_tensor_parallel_degrees_over_bytes():
    """A request moves, as bytes, from a 2-rank tensor-parallel deployment to a single-rank
    one and the other way round: the lender's ranks each frame the KV heads they hold, the
    frames travel as one body, the taker's ranks re-cut the heads for themselves.  Either way
    the tokens are those of one engine that did everything."""
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.handoff import (HandoffError, export_request, handoffs_from_bytes,
                                                 import_request, pack_frames, unpack_frames)
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)

    def single():
        model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
        return LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=128, use_graphs=False)

    whole = single().generate([_PROMPT], sp)[0]

    # two ranks lend, one rank takes
    first, blob = _spawn_tp("lend")
    frames = unpack_frames(blob)
    assert len(frames) == 2 and first == whole[:len(first)]
    hs = handoffs_from_bytes(blob)
    assert sorted(h.head_lo for h in hs) == [0, 1] and all(h.heads_total == 2 for h in hs)
    eng = single()
    for h in hs:
        h.validate_for(eng)
    import_request(eng, hs)
    rest = []
    while eng.has_work():
        for o in eng.step():
            rest.extend(o.new_token_ids)
    assert first + rest == whole

    # one rank lends, two ranks take
    eng = single()
    rid = eng.add_request(_PROMPT, sp)
    first = []
    while not first:
        for o in eng.step():
            first.extend(o.new_token_ids)
    body = export_request(eng, rid).to_bytes()
    toks, refused = _spawn_tp("take", body)
    assert first + toks == whole and refused

    # frames that do not cover the heads, or describe different requests, are refused
    with pytest.raises(HandoffError, match="in no frame"):
        handoffs_from_bytes(pack_frames([frames[0], frames[0]]))
    other = hs[1]
    other.request_id = "someone-else"
    with pytest.raises(HandoffError, match="different requests"):
        handoffs_from_bytes(pack_frames([frames[0], other.to_bytes()]))
