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
