"""Expert-union serving on CPU ranks (gloo): data-parallel attention with expert
parallelism (every rank schedules its own requests and holds a share of the experts) and
the disaggregated layout (attention ranks + an experts-only rank).  Loads are uneven, one
attention member gets no request at all (it joins every step), prefill and decode steps of
different members meet in one agreed capacity, and every request's tokens equal those of
one unsharded engine."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _prompts():
    g = torch.Generator().manual_seed(3)
    return [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (9, 41, 20, 5, 33)]


def _worker(rank, world, port, q, afd, micro=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.engine.union import UnionFront, UnionMember, capacity_class, member_loop
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.parallel.context import ParallelContext
    from uniserve_v1_b200.parallel.expert_exchange import HostExpertExchange
    assert capacity_class(0, 64) == 0 and capacity_class(3, 64) == 4 and capacity_class(64, 64) == 64
    assert capacity_class(300, 8192) == 512 and capacity_class(70, 100) == 100
    cfg = Qwen3MoeConfig.tiny()
    sources = tuple(range(world - 1)) if afd else tuple(range(world))
    experts = (world - 1,) if afd else tuple(range(world))
    ctx = ParallelContext(world_rank=rank, world_size=world)
    ctx.source_ranks, ctx.expert_ranks = sources, experts
    model = Qwen3MoeModel(cfg, "cpu", torch.float32, ctx).init_random(seed=0)
    model.exchange = HostExpertExchange(dist.group.WORLD, rank, world, 64, cfg.num_experts_per_tok,
                                        cfg.hidden_size, cfg.num_experts, sources, experts)
    eng = None
    if rank in sources:
        eng = LLMEngine(model, num_pages=96, max_num_seqs=4, max_model_len=128, use_graphs=False,
                        max_num_batched_tokens=32)
    if micro:       # decode steps as two interleaved half-batches, an exchange each
        model.micro_exchanges = [
            HostExpertExchange(dist.group.WORLD, rank, world, 32, cfg.num_experts_per_tok,
                               cfg.hidden_size, cfg.num_experts, sources, experts) for _ in (0, 1)]
    member = UnionMember(dist.group.WORLD, rank, world, sources, experts, engine=eng, model=model,
                         capacity_limit=64, microbatches=2 if micro else 1)
    if rank != 0:
        ticks = member_loop(member, 0)
        q.put((rank, member.stats, ticks))
        dist.barrier()
        dist.destroy_process_group()
        return
    front = UnionFront(member, 0)
    # every request lands on one member only: the other attention members never get one
    front.load = {r: (0 if r == 0 else 10 ** 6) for r in front.load} if afd else front.load
    if not afd:
        front.load[world - 1] = 10 ** 6          # the last member stays idle: it only joins
    sp = SamplingParams(temperature=0.0, max_tokens=7, ignore_eos=True)
    rids = [front.add_request(p, sp) for p in _prompts()[:3]]
    got = {r: [] for r in rids}
    late = None
    steps = 0
    while front.has_work():
        for o in front.step():
            got.setdefault(o.request_id, []).extend(o.new_token_ids)
        steps += 1
        if steps == 4 and late is None:         # requests that arrive while others decode
            late = [front.add_request(p, sp) for p in _prompts()[3:]]
    try:
        front.add_request([5000], sp)
        bad = False
    except ValueError:
        bad = True
    front.shutdown()
    q.put((0, {"tokens": [got[r] for r in rids + late], "where": dict(front.where),
               "stats": front.union_stats(), "rejects": bad}, steps))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("afd,micro", [(False, False), (True, False), (False, True), (True, True)])
def test_union_serving_matches_one_engine(afd, micro):
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    sp = SamplingParams(temperature=0.0, max_tokens=7, ignore_eos=True)
    ref = LLMEngine(model, num_pages=96, max_num_seqs=8, max_model_len=128,
                    use_graphs=False).generate(_prompts(), sp)
    world = 3 if afd else 4            # the tiny model's 8 experts divide over 1 or 4 ranks
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, afd, micro)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(world):
        rank, data, n = q.get(timeout=300)
        res[rank] = (data, n)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    lead, steps = res[0]
    assert lead["tokens"] == ref, (lead["tokens"], ref)
    assert lead["rejects"] and not lead["where"]
    # the idle attention member took part in every step without a batch of its own
    idle = res[1 if afd else world - 1][0]
    assert idle["steps"] == 0 and idle["joins"] > 0
    if afd:
        assert res[world - 1][0]["joins"] == lead["stats"]["steps"] + lead["stats"]["joins"]
    else:
        busy = res[1][0]
        assert busy["steps"] > 0
    assert len(lead["stats"]["capacities"]) >= 2          # prefill and decode classes met
    # steps in which every member decodes (or idles) ran as two half-batches
    assert (lead["stats"].get("micro_steps", 0) > 0) == micro
