"""Tensor- and expert-parallel sharding on CPU ranks (gloo): a model split over
two or four ranks (four: KV heads replicated twice) must reproduce the unsharded model."""
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


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.parallel.context import ParallelContext
    ctx = ParallelContext.from_world(tensor=world, expert_over_tensor=True)
    assert ctx.tp_size == world and ctx.ep_size == world and ctx.tp_rank == rank
    cfg = Qwen3MoeConfig.tiny()
    model = Qwen3MoeModel(cfg, "cpu", torch.float32, ctx).init_random(seed=0)
    assert model.E_local == cfg.num_experts // world
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (9, 20)]
    eng = LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=128, use_graphs=False)
    out = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    if rank == 0:
        q.put(out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_tp_ep_matches_single_rank(world):
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (9, 20)]
    ref = LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=128,
                    use_graphs=False).generate(
        prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert out == ref


def _serve_rank(rank, world, port, q):
    """Leader (rank 0) drives a replicated engine; the follower mirrors its commands."""
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
    if r != 0:
        steps = MR.follower_loop(eng, bus)
        q.put(("follower", steps))
        return
    rep = MR.ReplicatedEngine(eng, bus)
    sp = SamplingParams(temperature=0.8, top_p=0.9, seed=11, max_tokens=6, ignore_eos=True)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (9, 20, 5)]
    ids = [rep.add_request(p, sp) for p in prompts[:2]]
    outs, steps, added = {i: [] for i in ids}, 0, False
    while rep.has_work():
        for o in rep.step():
            outs.setdefault(o.request_id, []).extend(o.new_token_ids)
        steps += 1
        if steps == 2 and not added:          # a request admitted mid-flight, one aborted
            ids.append(rep.add_request(prompts[2], sp))
            rep.abort(ids[0])
            added = True
    rep.shutdown()
    q.put(("leader", steps, [outs.get(i, []) for i in ids]))


def test_replicated_engine_keeps_ranks_in_lock_step():
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_serve_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict()
    for _ in range(2):
        m = q.get(timeout=90)
        got[m[0]] = m[1:]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    steps, outs = got["leader"]
    assert got["follower"][0] == steps
    # the two untouched requests equal what a single-rank engine samples
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    eng = LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=128, use_graphs=False)
    sp = SamplingParams(temperature=0.8, top_p=0.9, seed=11, max_tokens=6, ignore_eos=True)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (9, 20, 5)]
    ref = eng.generate(prompts, sp)
    assert outs[1] == ref[1] and outs[2] == ref[2]
    assert len(outs[0]) < 6 and outs[0] == ref[0][:len(outs[0])]      # aborted early


def _pp_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.parallel.context import ParallelContext
    ctx = ParallelContext.from_world(layer=world)
    cfg = Qwen3MoeConfig.tiny()
    cfg.num_hidden_layers = 4
    model = Qwen3MoeModel(cfg, "cpu", torch.float32, ctx).init_random(seed=0)
    own = [i for i, lw in enumerate(model.layers) if lw is not None]
    assert own == list(range(rank * 2, rank * 2 + 2))
    caches = model.new_kv_caches(4, 16)
    assert all((caches[i][0] is not None) == (i in own) for i in range(4))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (9, 20)]
    eng = LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=128, use_graphs=False)
    out = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    q.put((rank, out))
    dist.barrier()
    dist.destroy_process_group()


def test_pipeline_stages_match_single_rank():
    """Two pipeline stages (two layers each, hand-off of block output and residual by
    point-to-point messages) generate what the unsplit model generates, on both ranks."""
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    cfg = Qwen3MoeConfig.tiny()
    cfg.num_hidden_layers = 4
    model = Qwen3MoeModel(cfg, "cpu", torch.float32).init_random(seed=0)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (9, 20)]
    ref = LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=128,
                    use_graphs=False).generate(
        prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    outs = dict(q.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert outs[0] == ref and outs[1] == ref
