"""Distributed weight data parallelism on CPU ranks (gloo): every rank is a whole attention
replica with its own prompts and a resident half of the experts; a layer's other experts are
read from the peer.  Tokens equal those of one unsharded engine; no token crosses ranks."""
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


def _prompts(rank):
    g = torch.Generator().manual_seed(10 + rank)
    return [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (9, 30)]


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.parallel.context import ParallelContext
    from uniserve_v1_b200.parallel.dwdp import attach_weight_peers
    cfg = Qwen3MoeConfig.tiny()
    ctx = ParallelContext.from_world(expert=world)
    model = Qwen3MoeModel(cfg, "cpu", torch.float32, ctx).init_random(seed=0)
    resident = model.layers[0].w13.shape[0]
    peers = attach_weight_peers(model, dist.group.WORLD, rank, world)
    assert resident == cfg.num_experts // world and model.E_local == cfg.num_experts
    eng = LLMEngine(model, num_pages=96, max_num_seqs=4, max_model_len=128, use_graphs=False)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    # the host form gathers shards collectively, so the ranks step in lock-step here: the same
    # prompt lengths on every rank, different tokens
    outs = eng.generate(_prompts(rank), sp)
    q.put((rank, outs, peers.bytes_read))
    dist.barrier()
    dist.destroy_process_group()


def test_dwdp_ranks_read_expert_shards_and_match_one_engine():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict()
    for _ in range(world):
        rank, outs, nbytes = q.get(timeout=300)
        got[rank] = outs
        assert nbytes > 0
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    eng = LLMEngine(model, num_pages=96, max_num_seqs=4, max_model_len=128, use_graphs=False)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    for rank in range(world):
        assert eng.generate(_prompts(rank), sp) == got[rank], rank
