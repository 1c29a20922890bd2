"""Two GPUs, one process each: the peer-memory collectives against NCCL / a local
sum, and the sharded model under CUDA graphs against the single-GPU engine."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _cfg():
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig
    return Qwen3MoeConfig(vocab_size=2048, hidden_size=512, num_hidden_layers=2,
                          num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                          num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256,
                          eos_token_id=2047, max_position_embeddings=1024)


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeModel
    from uniserve_v1_b200.ops import native as N
    from uniserve_v1_b200.ops import reference as R
    from uniserve_v1_b200.parallel.context import ParallelContext
    from uniserve_v1_b200.parallel.symm import attach_fused
    ctx = ParallelContext.from_world(tensor=world, expert_over_tensor=True)
    fc = attach_fused(ctx, dev, hidden=512)
    result = {}
    # 1. push-form all-reduce + residual + norm, three rounds (epochs and slot parity advance);
    #    odd rounds hand the kernel expert rows to un-permute instead of finished partial rows
    T, H, k = 48, 512, 4
    w = torch.ones(H, dtype=torch.bfloat16, device=dev) * 1.5
    residual = None
    ref_res = None
    ok = True
    budget = 1e-4        # FP32 sums in another order; grows by what the routed rounds may add
    for it in range(4):
        fc.begin_forward()
        g = torch.Generator(device=dev).manual_seed(100 * it + rank)
        if it % 2 == 0:
            mine = (torch.randn(T, H, generator=g, device=dev) * 0.5).to(torch.bfloat16)
            y, residual = fc.allreduce_add_rmsnorm(mine, residual, w, 1e-6)
        else:
            rows = (torch.randn(T * k, H, generator=g, device=dev) * 0.5).to(torch.bfloat16)
            perm = torch.randperm(T * k, generator=g, device=dev).to(torch.int32).view(T, k)
            perm[:, rank % k] = -1                       # a route that is not local
            wts = torch.rand(T, k, generator=g, device=dev)
            y, residual = fc.allreduce_add_rmsnorm(None, residual, w, 1e-6,
                                                   routed=(rows, perm, wts))
            pick = rows.float()[perm.clamp_min(0).long()] * (perm >= 0)[..., None] * wts[..., None]
            mine = pick.sum(1).to(torch.bfloat16)
            # the kernel adds a token's k rows in its own order before it rounds the partial
            # row to bf16 for the push: one bf16 unit round-off per rank, relative to the
            # largest partial value
            top = mine.float().abs().max()
            dist.all_reduce(top, op=dist.ReduceOp.MAX)
            budget += world * 2.0 ** -8 * float(top)
        total = mine.float().clone()
        dist.all_reduce(total)          # NCCL reference sum of the bf16 partials in fp32
        ref_res = total if ref_res is None else ref_res + total
        y_ref = (ref_res * torch.rsqrt(ref_res.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float())
        torch.cuda.synchronize()
        ok &= bool(torch.allclose(residual, ref_res, atol=budget, rtol=1e-4))
        ok &= bool(torch.allclose(y.float(), y_ref, atol=3e-2 + 2 * budget, rtol=3e-2))
    result["fused_norm"] = ok
    # every rank formed the same sum in the same order: bitwise equal results
    mine_sum = residual.double().sum().item()
    sums = [None] * world
    dist.all_gather_object(sums, mine_sum)
    result["same_on_every_rank"] = len(set(sums)) == 1
    # 1b. one site reused back to back while a peer is late: a host sleep before the late
    #     rank's launch, never a device-side stall; slot parity keeps the earlier data intact
    import time
    one = type(fc)(ctx.axis("tensor").group, rank, world, dev, H, sites=3)
    ok = True
    res1 = None
    ref1 = None
    for it in range(6):
        g = torch.Generator(device=dev).manual_seed(500 + 10 * it + rank)
        mine = (torch.randn(T, H, generator=g, device=dev) * 0.5).to(torch.bfloat16)
        if rank == (it % world) and it % 2:
            torch.cuda.synchronize()
            time.sleep(0.05)
        y, res1 = one.allreduce_add_rmsnorm(mine, res1, w, 1e-6)
        total = mine.float().clone()
        dist.all_reduce(total)
        ref1 = total if ref1 is None else ref1 + total
        torch.cuda.synchronize()
        ok &= bool(torch.allclose(res1, ref1, atol=1e-4, rtol=1e-4))
    result["one_site_reuse"] = ok and one.ring == 1
    dist.barrier()
    one.close()
    # 1c. greedy tokens of a vocabulary-sharded head: only (value, column) pairs travel
    V, per = 1000, (1000 + world - 1) // world
    gl = torch.Generator(device=dev).manual_seed(77)
    full = torch.randn(T, per * world, generator=gl, device=dev)
    full[:, V:] = 100.0                                   # pad columns must never win
    full[3, 17] = full[3, 700] = 50.0                     # a tie: the lower column wins
    lo = rank * per
    mine = full[:, lo:lo + per].contiguous()
    got = fc.argmax(mine, max(0, min(V, lo + per) - lo), lo)
    torch.cuda.synchronize()
    result["argmax"] = bool(torch.equal(got.long(), full[:, :V].argmax(-1))) and int(got[3]) == 17
    # 2. generic all-reduce through the heap, twice on the same site in a row
    x = torch.full((16, 512), float(rank + 1), dtype=torch.bfloat16, device=dev)
    fc.begin_forward()
    s = fc.all_reduce(x)
    fc.begin_forward()
    for _ in range(fc.ring):
        s2 = fc.all_reduce(x * 2)
    torch.cuda.synchronize()
    result["allreduce"] = bool((s.float() == sum(range(1, world + 1))).all()) and \
        bool((s2.float() == 2 * sum(range(1, world + 1))).all())
    # 3. sharded engine with graphs == what rank 0 would compute alone
    model = Qwen3MoeModel(_cfg(), dev, torch.bfloat16, ctx).init_random(seed=0)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (9, 33, 20)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    out = LLMEngine(model, num_pages=128, max_num_seqs=4, max_model_len=256,
                    use_graphs=True).generate(prompts, sp)
    torch.cuda.synchronize()
    result["status"] = N.read_status()
    result["tokens"] = out
    # 4. prefill chunks above the one-shot limit: reduce-scatter in the GEMM epilogue, all-gather
    #    from the norm kernel, no library collective in the layer loop
    from uniserve_v1_b200.parallel.tp_fused import attach_fused_tp
    ft = attach_fused_tp(model, 1024)
    long_prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (300, 700, 41)]
    eng2 = LLMEngine(model, num_pages=256, max_num_seqs=4, max_model_len=1024, use_graphs=True,
                     max_num_batched_tokens=1024)
    result["long_tokens"] = eng2.generate(long_prompts, SamplingParams(temperature=0.0, max_tokens=6,
                                                                       ignore_eos=True))
    torch.cuda.synchronize()
    result["fused_prefills"] = ft.calls
    result["status2"] = N.read_status()
    if rank == 0:
        q.put(result)
    dist.barrier()
    ft.close()
    fc.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_collectives_and_sharded_engine(world):
    _need(world)
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeModel
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = q.get(timeout=600)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert res["fused_norm"] and res["allreduce"] and res["status"] == 0, res
    assert res["same_on_every_rank"] and res["one_site_reuse"] and res["argmax"], res
    model = Qwen3MoeModel(_cfg(), "cuda:0", torch.bfloat16).init_random(seed=0)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (9, 33, 20)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    single = LLMEngine(model, num_pages=128, max_num_seqs=4, max_model_len=256).generate(prompts, sp)
    # bf16 partial sums are rounded differently when split over ranks: require the
    # first tokens to agree and most of the rest.
    agree = sum(a == b for s_, t in zip(single, res["tokens"]) for a, b in zip(s_, t))
    total = sum(len(s_) for s_ in single)
    firsts = sum(s_[0] == t[0] for s_, t in zip(single, res["tokens"]))
    # more ranks, more differently rounded partial sums: near-ties of the random model flip
    need_first, need_all = (len(single), 0.7) if world == 2 else (len(single) - 1, 0.5)
    assert firsts >= need_first, (single, res["tokens"])
    assert agree >= need_all * total, (single, res["tokens"])
    # the fused tensor-parallel prefill served those long prompts, and gives the single GPU's tokens
    assert res["fused_prefills"] >= 1 and res["status2"] == 0, res
    long_prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (300, 700, 41)]
    single_long = LLMEngine(model, num_pages=256, max_num_seqs=4, max_model_len=1024,
                            max_num_batched_tokens=1024).generate(
        long_prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    firsts = sum(s_[0] == t[0] for s_, t in zip(single_long, res["long_tokens"]))
    agree = sum(a == b for s_, t in zip(single_long, res["long_tokens"]) for a, b in zip(s_, t))
    assert firsts >= len(single_long) - 1 and agree >= 0.5 * 18, (single_long, res["long_tokens"])


def _h3_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from uniserve_v1_b200.models.minimax_h3 import Denoiser, H3Config, H3Transformer, dmd_ladder
    from uniserve_v1_b200.ops import native as N
    from uniserve_v1_b200.parallel.context import ParallelContext
    from uniserve_v1_b200.parallel.ulysses import FusedUlysses
    ctx = ParallelContext.from_world(ulysses=world)
    cfg = H3Config.tiny()
    cfg.num_heads = 4
    cfg.hidden_size = 256      # attention width 4 x 128 = 512 differs from the stream width
    cfg.refiner_heads = 4
    g = torch.Generator().manual_seed(5)
    text = torch.randn(9, cfg.text_dim, generator=g)

    def run(fused):
        model = H3Transformer(cfg, dev, torch.bfloat16, ctx).init_random(seed=0)
        den = Denoiser(model, dmd_ladder((999, 500), 10.0), dmd_ladder((999, 500), 3.0))
        st = den.prepare(seed=42, latent_frames=3, lat_h=8, lat_w=16, n_audio=20, text_features=text)
        fu = None
        if fused:
            fu = FusedUlysses(ctx, dev, st.layout.rows, model.heads_local, cfg.head_dim)
            model.ulysses = fu
        den.run(st)
        torch.cuda.synchronize()
        status = N.read_status()
        if fu is not None:
            dist.barrier()
            fu.close()
        return st.video.cpu(), st.audio.cpu(), status

    v0, a0, s0 = run(False)
    v1, a1, s1 = run(True)
    if rank == 0:
        q.put({"base": (v0, a0), "fused": (v1, a1), "status": (s0, s1)})
    dist.barrier()
    dist.destroy_process_group()


def test_h3_fused_ulysses_matches_all_to_all_and_single_gpu():
    _need(2)
    from uniserve_v1_b200.models.minimax_h3 import Denoiser, H3Config, H3Transformer, dmd_ladder
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_h3_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = q.get(timeout=600)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert res["status"] == (0, 0)
    vb, ab = res["base"]
    vf, af = res["fused"]
    torch.testing.assert_close(vf, vb, atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(af, ab, atol=1e-3, rtol=1e-3)
    cfg = H3Config.tiny()
    cfg.num_heads = 4
    cfg.hidden_size = 256      # attention width 4 x 128 = 512 differs from the stream width
    cfg.refiner_heads = 4
    model = H3Transformer(cfg, "cuda:0", torch.bfloat16).init_random(seed=0)
    den = Denoiser(model, dmd_ladder((999, 500), 10.0), dmd_ladder((999, 500), 3.0))
    g = torch.Generator().manual_seed(5)
    text = torch.randn(9, cfg.text_dim, generator=g)
    st = den.prepare(seed=42, latent_frames=3, lat_h=8, lat_w=16, n_audio=20, text_features=text)
    den.run(st)
    torch.testing.assert_close(vb, st.video.cpu(), atol=3e-2, rtol=3e-2)


def _push_tail_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import ctypes
    import math
    from uniserve_v1_b200.ops import native as N
    from uniserve_v1_b200.ops.flash import flash_attn_varlen
    from uniserve_v1_b200.parallel.context import ParallelContext
    from uniserve_v1_b200.parallel import ulysses as U
    ctx = ParallelContext.from_world(ulysses=world)
    T, hl, D = 3072, 13, 128          # 12 query pairs x 13 heads = 156 items: one wave and 8 more
    fu = U.FusedUlysses(ctx, dev, T, hl, D)
    ro, inner = T // world, world * hl * D

    def qkv_of(r):
        g = torch.Generator(device="cpu").manual_seed(50 + r)
        return [(torch.randn(T, hl, D, generator=g) * 0.5).to(torch.bfloat16).to(dev) for _ in range(3)]

    qr, kr, vr = qkv_of(rank)
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    scale = 1 / math.sqrt(D)
    ok = True
    for it in range(2):
        fu.fc.barrier(U.SITE_B1)       # nobody still reads the buffers of the round before
        N.call("us_flash_attn_push", N.ptr(qr), N.ptr(kr), N.ptr(vr), N.ptr(cu), N.ptr(cu), T, T,
               hl, hl, qr.stride(0), kr.stride(0), vr.stride(0), scale, fu._ptrs(U.SITE_ATT), world,
               ro, rank * hl * D, inner, N.stream())
        fu.fc.barrier(U.SITE_B2)
        got = fu.fc.site_tensor(U.SITE_ATT, ro, inner).clone()
        torch.cuda.synchronize()
        for r in range(world):          # every rank's heads arrived in its column block
            q2, k2, v2 = qkv_of(r)
            ref = flash_attn_varlen(q2, k2, v2, cu, cu, T, T, scale, False)
            mine = ref[rank * ro:(rank + 1) * ro].reshape(ro, hl * D)
            ok &= bool(torch.equal(got[:, r * hl * D:(r + 1) * hl * D], mine))
    torch.cuda.synchronize()
    q.put((rank, ok, N.read_status()))
    dist.barrier()
    fu.close()
    dist.destroy_process_group()


def test_flash_push_with_split_last_wave_between_real_peers():
    """The sequence-parallel return from the attention epilogue on a shape whose last partial
    wave of (pair, head) items is split over the keys: those rows reach their owners from the
    merge kernel.  Every rank checks the column block of every rank bit for bit against the
    plain kernel."""
    _need(2)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_push_tail_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=600) for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, ok, status in res:
        assert ok and status == 0, (rank, ok, status)


def _ep_worker(rank, world, port, q, afd):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from uniserve_v1_b200.ops import functional as F
    from uniserve_v1_b200.ops import native as N
    from uniserve_v1_b200.ops import reference as R
    from uniserve_v1_b200.parallel.expert_exchange import ExpertExchange
    T, k, H, E, I = 24, 4, 512, 16, 256
    src = (0,) if afd else (0, 1)
    exp = (1,) if afd else (0, 1)
    ex = ExpertExchange(dist.group.WORLD, rank, world, dev, T, k, H, E, I, src, exp)
    g = torch.Generator(device="cpu").manual_seed(7)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.03).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.03).to(torch.bfloat16)
    norm_w = torch.ones(H, dtype=torch.bfloat16, device=dev)
    ok = True
    for it in range(3):                                    # epochs advance across layers
        gt = torch.Generator(device="cpu").manual_seed(100 * it + rank)
        x = (torch.randn(T, H, generator=gt) * 0.5).to(torch.bfloat16).to(dev)
        logits = torch.randn(T, E, generator=gt).to(dev)
        residual = torch.randn(T, H, generator=gt).to(dev)
        live = torch.tensor([T - 3], dtype=torch.int32, device=dev)
        if ex.is_source:
            ids, wts = F.topk_softmax(logits, k, True, live=live)
            ex.dispatch(x, ids, wts, live)
        if ex.is_expert:
            lo = ex.e_lo
            ex.experts(w13[lo:lo + ex.experts_per_rank].to(dev).contiguous(),
                       w2[lo:lo + ex.experts_per_rank].to(dev).contiguous(), T)
        if ex.is_source:
            res2 = residual.clone()
            y, res2 = ex.combine_add_rmsnorm(ids, live, res2, norm_w, 1e-6)
            torch.cuda.synchronize()
            moe = R.moe_experts(x.cpu(), ids.cpu(), wts.cpu(), w13, w2).float()
            ref_res = residual.cpu() + moe
            ref_y = ref_res * torch.rsqrt(ref_res.pow(2).mean(-1, keepdim=True) + 1e-6)
            ok &= bool(torch.allclose(res2.cpu(), ref_res, atol=3e-2, rtol=3e-2))
            ok &= bool(torch.allclose(y.float().cpu(), ref_y, atol=5e-2, rtol=5e-2))
    torch.cuda.synchronize()
    q.put((rank, ok, N.read_status()))
    dist.barrier()
    ex.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("afd", [False, True])
def test_expert_exchange_dispatch_combine(afd):
    """EP (every rank is source and expert) and AFD (rank 0 attention, rank 1 experts)."""
    _need(2)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker, args=(r, 2, port, q, afd)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=600) for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, ok, status in res:
        assert ok and status == 0, res


def _tp_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from uniserve_v1_b200.ops import native as N
    from uniserve_v1_b200.parallel import tp_fused as TP
    rows, H, I, eps = 384, 512, 1024, 1e-6
    g = torch.Generator().manual_seed(11)
    x = torch.randn(rows, H, generator=g)
    w13 = torch.randn(2 * I, H, generator=g) * 0.05
    w2 = torch.randn(H, I, generator=g) * 0.05
    nw = 1.0 + 0.1 * torch.randn(H, generator=g)
    bf = lambda t: t.to(dev).to(torch.bfloat16)
    tp = TP.FusedTP(dist.group.WORLD, rank, world, dev, rows, H)
    ro, Il = rows // world, I // world
    lo = rank * ro
    # own rows: residual x, normalised rows into the heap
    res = x[lo:lo + ro].to(dev).clone()
    xn = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * nw
    tp.gathered(TP.SITE_NORM_A).copy_(bf(xn))       # as left by the producers of every rank
    # weight shards: value rows then gate rows of this rank's slice of I
    w13_l = bf(torch.cat([w13[rank * Il:(rank + 1) * Il], w13[I + rank * Il:I + (rank + 1) * Il]]))
    w2_l = bf(w2[:, rank * Il:(rank + 1) * Il]).contiguous()
    outs = []
    for it in range(2):     # twice: the barriers' epochs advance
        r = res.clone()
        y = tp.mlp(r, TP.SITE_NORM_A, w13_l, w2_l, bf(nw), TP.SITE_NORM_B, eps)
        torch.cuda.synchronize()
        torch.cuda.synchronize()
        dist.barrier()                               # the peers' rows have landed too
        full = tp.gathered(TP.SITE_NORM_B).float().cpu()
        outs.append((r.cpu(), y.float().cpu(), full))
    status = N.read_status()
    gathered = [None] * world
    dist.all_gather_object(gathered, outs[-1])
    same = torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    # every rank holds all rows: its copy equals the concatenation of the owners' rows
    own = [None] * world
    dist.all_gather_object(own, outs[-1][1])
    same = same and torch.equal(outs[-1][2], torch.cat(own, 0))
    if rank == 0:
        q.put({"status": status, "parts": gathered, "same": same})
    dist.barrier()
    tp.close()
    dist.destroy_process_group()


def test_tp_gather_gemm_and_reduce_scatter_gemm_match_reference():
    """Column-parallel GEMM reading the peers' rows + row-parallel GEMM pushing
    partial rows to their owners + slot reduction fused with residual/RMSNorm,
    against the unsharded FP32 computation."""
    _need(2)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = q.get(timeout=600)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert res["status"] == 0
    assert res["same"]
    rows, H, I, eps = 384, 512, 1024, 1e-6
    g = torch.Generator().manual_seed(11)
    x = torch.randn(rows, H, generator=g)
    w13 = torch.randn(2 * I, H, generator=g) * 0.05
    w2 = torch.randn(H, I, generator=g) * 0.05
    nw = 1.0 + 0.1 * torch.randn(H, generator=g)
    r16 = lambda t: t.to(torch.bfloat16).float()
    xn = r16(x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * nw)
    up, gate = xn @ r16(w13[:I]).t(), xn @ r16(w13[I:]).t()
    hid = r16(up * torch.nn.functional.silu(gate))
    want_res = x + hid @ r16(w2).t()
    want_y = want_res / torch.sqrt((want_res * want_res).mean(-1, keepdim=True) + eps) * r16(nw)
    got_res = torch.cat([p[0] for p in res["parts"]], 0)
    got_y = torch.cat([p[1] for p in res["parts"]], 0)
    torch.testing.assert_close(got_res, want_res, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(got_y, want_y, atol=3e-2, rtol=3e-2)


def _dwdp_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeModel
    from uniserve_v1_b200.ops import native as N
    from uniserve_v1_b200.parallel.context import ParallelContext
    from uniserve_v1_b200.parallel.dwdp import attach_weight_peers
    cfg = _cfg()
    ctx = ParallelContext.from_world(expert=world)
    model = Qwen3MoeModel(cfg, dev, torch.bfloat16, ctx).init_random(seed=0)
    peers = attach_weight_peers(model, dist.group.WORLD, rank, world)
    eng = LLMEngine(model, num_pages=128, max_num_seqs=4, max_model_len=256, use_graphs=False)
    g = torch.Generator().manual_seed(20 + rank)
    # the ranks are independent replicas: different numbers of prompts and steps
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist()
               for n in ((9, 33, 20) if rank == 0 else (50,))]
    sp = SamplingParams(temperature=0.0, max_tokens=6 + 4 * rank, ignore_eos=True)
    outs = eng.generate(prompts, sp)
    torch.cuda.synchronize()
    status = N.read_status()
    dist.barrier()                      # nobody frees its shards while a peer may read them
    q.put((rank, prompts, outs, peers.bytes_read, status))
    dist.barrier()
    peers.close()
    dist.destroy_process_group()


def test_dwdp_reads_expert_shards_from_the_peer():
    """Distributed weight data parallelism on two GPUs: each rank is a whole replica with half
    the experts resident; a layer's other half is copied from the peer's heap while the
    previous layer runs.  The ranks run different work and each gives the tokens of an
    unsharded engine."""
    _need(2)
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeModel
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_dwdp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=600) for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    model = Qwen3MoeModel(_cfg(), "cuda:0", torch.bfloat16).init_random(seed=0)
    eng = LLMEngine(model, num_pages=128, max_num_seqs=4, max_model_len=256, use_graphs=False)
    for rank, prompts, outs, nbytes, status in got:
        assert status == 0 and nbytes > 0
        sp = SamplingParams(temperature=0.0, max_tokens=6 + 4 * rank, ignore_eos=True)
        want = eng.generate(prompts, sp)
        same = sum(a == b for x, y in zip(want, outs) for a, b in zip(x, y))
        total = sum(len(x) for x in want)
        # the experts' GEMMs see another expert count per launch (all experts, not half):
        # tiles and rounding can differ, a near-tie may flip
        assert same >= 0.9 * total, (rank, want, outs)
