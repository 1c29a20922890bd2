"""MiniMax-H3-shaped transformer on CPU: layout, schedules, addressable noise and
Ulysses sequence parallelism (two gloo ranks reproduce one rank)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from uniserve_v1_b200.models.minimax_h3 import (Denoiser, H3Config, H3Transformer, build_layout,
                                                dmd_ladder, uniform_schedule)
from uniserve_v1_b200.ops.diffusion import philox_normal


def test_schedules_and_layout():
    lad = dmd_ladder(shift=10.0)
    assert len(lad) == 9 and lad[-1] == 0.0 and all(a > b for a, b in zip(lad, lad[1:]))
    assert abs(lad[0] - 10 * 0.999 / (1 + 9 * 0.999)) < 1e-12
    base = uniform_schedule(50, 12.0)
    assert base[0] == 1.0 and base[-1] == 0.0 and len(base) <= 51
    cfg = H3Config.tiny()
    lay = build_layout(cfg, 5, 6, 8, 10, 7, sp=2)
    assert lay.n_video == 5 * 3 * 4 and lay.used == 60 + 10 + 7 and lay.rows % 128 == 0
    assert lay.mod_index[0] == 0 and lay.mod_index[60] == 3 * 1 + 2 and lay.mod_index[70] == 1
    assert lay.coords[:, 13].tolist() == [1.0, 0.0, 1.0]
    # full-size geometry: 124 frames at 1344x768 -> 37 latent frames x 1008 tokens
    full = H3Config()
    lf, lh, lw = full.latent_shape(124, 1344, 768)
    assert (lf, lh, lw) == (40, 48, 84) or lf * (lh // 2) * (lw // 2) > 0


def test_noise_is_addressable():
    a = philox_normal((4, 50), 11, 0)
    b = philox_normal((200,), 11, 0)
    assert torch.equal(a.view(-1), b)
    assert not torch.equal(philox_normal((200,), 11, 1), b)
    assert abs(float(philox_normal((100000,), 3).std()) - 1.0) < 0.02


def _run(ctx=None, steps=2, conditions=False):
    cfg = H3Config.tiny()
    model = H3Transformer(cfg, "cpu", torch.float32, ctx).init_random(seed=0)
    den = Denoiser(model, dmd_ladder((999, 500), 10.0), dmd_ladder((999, 500), 3.0))
    g = torch.Generator().manual_seed(5)
    text = torch.randn(9, cfg.text_dim, generator=g)
    conds = None
    if conditions:       # a last-frame keyframe, a reference image and a reference track
        conds = [(-1, torch.randn(cfg.latent_channels, 1, 4, 8, generator=g) * 30),
                 (None, torch.randn(cfg.latent_channels, 1, 4, 8, generator=g) * 30),
                 (None, torch.randn(10, cfg.audio_channels, generator=g) * 30)]
    st = den.prepare(seed=42, latent_frames=2, lat_h=4, lat_w=8, n_audio=6, text_features=text,
                     conditions=conds)
    den.run(st)
    return st.video, st.audio


def test_denoiser_single_rank_runs():
    v, a = _run()
    assert torch.isfinite(v).all() and torch.isfinite(a).all()
    v2, a2 = _run()
    assert torch.equal(v, v2) and torch.equal(a, a2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q, axis="ulysses", conditions=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from uniserve_v1_b200.parallel.context import ParallelContext
    if axis == "hybrid":
        ctx = ParallelContext.from_world(ulysses=2, gather=world // 2)
    else:
        ctx = ParallelContext.from_world(**{axis: world})
    v, a = _run(ctx, conditions=conditions)
    if rank == 0:
        q.put((v, a))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("axis", ["ulysses", "gather"])
def test_sequence_parallel_2_with_conditions_matches_single_rank(axis):
    """Condition rows (keyframe, reference image, reference track) follow the text rows; split
    over two ranks the clip is the one a single rank makes, and not the unconditioned one."""
    v1, a1 = _run(conditions=True)
    v0, _ = _run()
    effect = float((v1 - v0).abs().max())
    assert effect > 0
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, axis, True)) for r in range(2)]
    for p in procs:
        p.start()
    v2, a2 = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    torch.testing.assert_close(v2, v1, atol=2e-4, rtol=2e-4)
    torch.testing.assert_close(a2, a1, atol=2e-4, rtol=2e-4)
    assert float((v2 - v1).abs().max()) < 0.1 * effect       # the conditions are what is compared


@pytest.mark.parametrize("axis", ["ulysses", "gather", "layer"])
def test_sequence_parallel_2_matches_single_rank(axis):
    """Rows split over two ranks: heads travelling around attention (Ulysses) or K / V
    rows all-gathered with every head local (gather); or the blocks split over two
    stages (layer) with the rows handed from stage to stage."""
    v1, a1 = _run()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, axis)) for r in range(2)]
    for p in procs:
        p.start()
    v2, a2 = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    torch.testing.assert_close(v2, v1, atol=2e-4, rtol=2e-4)
    torch.testing.assert_close(a2, a1, atol=2e-4, rtol=2e-4)


def test_hybrid_sequence_placement_4_matches_single_rank():
    """Two gather places of two Ulysses members each: a place's rows meet on both members
    for half of the heads, keys and values of that half are gathered across the places."""
    v1, a1 = _run()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 4, port, q, "hybrid")) for r in range(4)]
    for p in procs:
        p.start()
    v2, a2 = q.get(timeout=300)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    torch.testing.assert_close(v2, v1, atol=2e-4, rtol=2e-4)
    torch.testing.assert_close(a2, a1, atol=2e-4, rtol=2e-4)


def test_attention_width_differs_from_stream_width():
    """The served shape has 56 x 128 = 7168 attention channels on a 5376-wide stream."""
    cfg = H3Config.tiny()
    cfg.num_heads = 3                      # 384 attention channels, hidden 256
    model = H3Transformer(cfg, "cpu", torch.float32).init_random(seed=0)
    assert model.blocks[0].qkv.shape == (3 * 384, 256)
    assert model.blocks[0].to_out.shape == (256, 384)
    den = Denoiser(model, dmd_ladder((999, 500), 10.0), dmd_ladder((999, 500), 3.0))
    g = torch.Generator().manual_seed(5)
    text = torch.randn(9, cfg.text_dim, generator=g)
    st = den.prepare(seed=1, latent_frames=2, lat_h=4, lat_w=4, n_audio=6, text_features=text)
    den.run(st)
    assert torch.isfinite(st.video).all() and torch.isfinite(st.audio).all()


def test_sparse_attention_student_reduces_to_dense_when_every_tile_is_kept():
    """With every video tile kept and a zero compression gate the sparse layer is the
    dense layer (same weights, 128-row layout unit)."""
    def run(sparsity):
        cfg = H3Config.tiny()
        cfg.vsa_sparsity = sparsity
        model = H3Transformer(cfg, "cpu", torch.float32).init_random(seed=0)
        return cfg, model
    cfg_s, sparse = run(1e-9)
    cfg_d, dense = run(0.0)
    D, hl = cfg_s.head_dim, sparse.heads_local
    for bs, bd in zip(sparse.blocks, dense.blocks):
        w = bs.qkv.view(4, hl * D, -1)
        w[3].zero_()                                   # gate projection off
        bd.qkv = w[:3].reshape(3 * hl * D, -1).clone()
        bd.to_out, bd.ff1, bd.ff2 = bs.to_out, bs.ff1, bs.ff2
    dense.proj_in, dense.audio_proj_in = sparse.proj_in, sparse.audio_proj_in
    dense.context_embedder, dense.refiner = sparse.context_embedder, sparse.refiner
    dense.proj_out, dense.audio_proj_out = sparse.proj_out, sparse.audio_proj_out
    dense.time_w1, dense.time_w2 = sparse.time_w1, sparse.time_w2
    outs = []
    for m in (sparse, dense):
        den = Denoiser(m, dmd_ladder((999, 500), 10.0), dmd_ladder((999, 500), 3.0))
        g = torch.Generator().manual_seed(5)
        text = torch.randn(9, m.cfg.text_dim, generator=g)
        st = den.prepare(seed=1, latent_frames=4, lat_h=16, lat_w=16, n_audio=6,
                         text_features=text)
        den.run(st)
        outs.append(st.video)
    assert st.layout.tile_sizes is None and outs[0].shape == outs[1].shape
    torch.testing.assert_close(outs[0], outs[1], atol=2e-2, rtol=2e-2)


def test_fp8_feed_forward_stays_close_to_bf16():
    outs = []
    for f8 in (False, True):
        cfg = H3Config.tiny()
        cfg.mlp_fp8 = f8
        model = H3Transformer(cfg, "cpu", torch.float32).init_random(seed=0)
        assert (model.blocks[0].ff1.dtype == torch.uint8) == f8
        den = Denoiser(model, dmd_ladder((999, 500), 10.0), dmd_ladder((999, 500), 3.0))
        g = torch.Generator().manual_seed(5)
        text = torch.randn(9, cfg.text_dim, generator=g)
        st = den.prepare(seed=1, latent_frames=2, lat_h=4, lat_w=4, n_audio=6, text_features=text)
        den.run(st)
        outs.append(st.video)
    assert float((outs[0] - outs[1]).norm() / outs[0].norm()) < 1e-2


def _video_rank(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    from uniserve_v1_b200.models.h3_vae import (AudioVaeConfig, AudioVaeDecoder, VideoVaeConfig,
                                                VideoVaeDecoder)
    from uniserve_v1_b200.parallel.context import ParallelContext
    from uniserve_v1_b200.server import multirank as MR
    from uniserve_v1_b200.server.video_rules import VideoPlan
    from uniserve_v1_b200.server.video_service import VideoJob, VideoService
    r, w, dev, control = MR.init_rank()
    ctx = ParallelContext.from_world(ulysses=world) if world > 1 else None
    svc = _tiny_service(ctx)
    if world == 1:
        q.put(svc.generate(VideoJob("a stream in a forest", _plan())))
        return
    bus = MR.CommandBus(control, r)
    if r > 0:
        done = MR.video_follower_loop(svc, bus)
        q.put(("follower", done))
        return
    rep = MR.ReplicatedVideoService(svc, bus)
    mp4 = svc.generate(VideoJob("a stream in a forest", _plan()))
    rep.shutdown()
    q.put(("leader", mp4))


def _plan():
    from uniserve_v1_b200.server.video_rules import VideoPlan
    return VideoPlan("t2va", 256, 256, 39, 24, 1000, 8)


def _tiny_service(ctx):
    from uniserve_v1_b200.models.h3_vae import (AudioVaeConfig, AudioVaeDecoder, VideoVaeConfig,
                                                VideoVaeDecoder)
    from uniserve_v1_b200.server.video_service import VideoService
    cfg = H3Config.tiny()
    cfg.vae_spatial = 64
    tr = H3Transformer(cfg, "cpu", torch.float32, ctx).init_random(0)
    vc = VideoVaeConfig.tiny()
    vc.latent_channels, vc.spatial = cfg.latent_channels, 64
    vv = VideoVaeDecoder(vc, "cpu", torch.float32).init_random(1)
    av = AudioVaeDecoder(AudioVaeConfig(latent_channels=cfg.audio_channels, decoder_dim=128,
                                        rates=(5, 5, 2, 2, 2, 2, 2), kernels=(9, 9, 4, 4, 4, 4, 4),
                                        res_kernels=(3,), res_dilations=(1,)), "cpu").init_random(2)
    return VideoService(tr, vv, av, sizes=["256x256"], max_seconds=5)


def test_two_rank_video_request_equals_single_rank():
    """A video request served by a leader and a follower (sequence-parallel transformer,
    temporal units of the VAE dealt over the ranks, planes gathered on the leader) yields
    the MP4 a single rank yields."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_video_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=180) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got["follower"] == 1
    one = _tiny_service(None).generate(
        __import__("uniserve_v1_b200.server.video_service", fromlist=["VideoJob"]).VideoJob(
            "a stream in a forest", _plan()))
    two = got["leader"]
    assert two[4:8] == b"ftyp" and len(two) == len(one)
    a = torch.frombuffer(bytearray(one), dtype=torch.uint8).float()
    b = torch.frombuffer(bytearray(two), dtype=torch.uint8).float()
    assert (a - b).abs().mean() < 0.5      # same pictures up to reduction-order noise
