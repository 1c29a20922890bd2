#!/usr/bin/env python
"""Headline benchmark of both served families, one JSON line.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

The line's headline is the **FastH3 8-step clip latency** (seconds, lower is better,
strong scaling): the MiniMax-H3 / FastH3-shaped video + audio transformer (50 blocks,
hidden 5376, 56 heads x 128, FFN 14336) on a 124-frame 1344 x 768 clip (37 latent frames,
38.7k packed rows) with a 1000-token prompt, bf16, random-init weights, Ulysses sequence
parallelism over the N ranks with the all-to-alls fused into the projection GEMM and the
attention epilogue.  A *step* is one denoising step; K steps are timed on the device
(CUDA events, max over ranks) and ``value`` = 8 x the mean step.  ``e2e`` is one whole
request through ``VideoService.generate`` (prompt features copied from pinned host memory,
latent preparation, 8 steps, both VAE decoders, colour conversion, plane read-back, MP4
mux).  At N >= 4 the key ``baseline_shape`` adds the synthetic 121-frame / 8x-spatial
shape (31 x 48 x 84 = 124,992 video tokens).

The nested ``qwen3_moe`` record is the second half of the metric: Qwen3-30B-A3B-shaped
chat serving (48 layers, 128 experts top-8, bf16, paged KV with 16-token pages), 64
concurrent requests of 1024 random prompt ids.  It holds the device-timed decode step
(tokens/s of all concurrent requests from CUDA-graph replays), the same through
``LLMEngine.step`` with its per-step host copies (``e2e``), and ``workload``: 64 requests
x (1024 in, 256 out) from the first ``add_request`` to the last token, prefill included.

N > 1 is launched under ``torch.distributed.run`` (one rank per GPU).
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

BASELINE_TOK_S = 64 / 20.5e-3   # reference: 64 concurrent, 20.5 ms/step on 1xGB200 (docs/configuration.md:468)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, period_ms: int = 200):
        self.gpu = gpu_index
        self.period_ms = period_ms
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms), "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def reference_arm(args) -> int:
    """The reference is a Rust workspace: the offline pip install of its tree
    yields only package metadata (no `uniserve` executable: it needs cargo /
    rustc 1.96 and setuptools-rust, absent from this image), and serving also
    needs Hugging Face checkpoints, FFmpeg 8.1 and NCCL >= 2.30.4."""
    ref = Path(__file__).resolve().parent / "baseline" / "_ref"
    exe = list(ref.glob("bin/uniserve")) if ref.exists() else []
    why = ("reference is a Rust serving binary; offline pip install of the reference tree produced "
           "metadata only (no cargo/rustc, no setuptools-rust), so no `uniserve` executable, "
           "checkpoints, FFmpeg 8.1 or NCCL>=2.30.4 exist to run it")
    if exe:
        why = "reference executable present but cannot serve without checkpoints and its Build Server toolchain"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


BASELINE_CLIP_S = 8.194         # reference: FastH3 8-step, Ulysses8, bf16, 5 s clip on 8xH200 (docs/minimax_h3/evaluation.md:169)


class Job:
    """Rank, device, process group and the helpers every record shares."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.args = args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.t_start = time.time()
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.dev)

    def mark(self, what: str) -> None:
        """Progress trace (one file per rank) when BENCH_TRACE names a directory."""
        d = os.environ.get("BENCH_TRACE")
        if d:
            with open(os.path.join(d, f"bench_rank{self.rank}.log"), "a") as f:
                f.write(f"{time.time() - self.t_start:8.2f}s {what}\n")

    def barrier(self, group=None) -> None:
        import torch
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier(group=group)
        torch.cuda.synchronize()

    def max_over_ranks(self, x: float, group=None) -> float:
        import torch
        import torch.distributed as dist
        if self.world > 1:
            t = torch.tensor([x], device=self.dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            return float(t.item())
        return x

    def timed(self, fn, group=None):
        """Runs ``fn`` between a barrier + synchronize on both sides; returns (device ms as
        the max over ranks, host wall seconds as the max over ranks, fn's result)."""
        import torch
        self.barrier(group)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        ev0.record()
        out = fn()
        ev1.record()
        self.barrier(group)
        wall = time.perf_counter() - t0
        return (self.max_over_ranks(ev0.elapsed_time(ev1), group),
                self.max_over_ranks(wall, group), out)


def release_device_memory() -> None:
    import torch
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()


# ------------------------------------------------------------------- FastH3 --
def fasth3_record(job: Job) -> dict:
    """FastH3 8-step clip latency; see the module docstring for what is timed."""
    import torch
    from uniserve_v1_b200.models.h3_vae import (AudioVaeConfig, AudioVaeDecoder, VideoVaeConfig,
                                                VideoVaeDecoder)
    from uniserve_v1_b200.models.minimax_h3 import H3Config, H3Transformer
    from uniserve_v1_b200.ops import native
    from uniserve_v1_b200.parallel.context import ParallelContext
    from uniserve_v1_b200.server.video_rules import VideoPlan
    from uniserve_v1_b200.server.video_service import VideoJob, VideoService

    args, world, rank, dev = job.args, job.world, job.rank, job.dev
    tiny = args.model == "tiny"
    cfg = H3Config.tiny() if tiny else H3Config()
    if tiny:
        cfg.num_heads = 8
        cfg.hidden_size = 1024
    if args.layers:
        cfg.num_layers = args.layers
    cfg.mlp_fp8 = bool(args.mlp_fp8)
    frames = args.frames or (22 if tiny else 124)
    width, height = (256, 256) if tiny else (1344, 768)
    n_text = args.prompt_len or (64 if tiny else 1000)
    ctx = ParallelContext.from_world(ulysses=world) if world > 1 else ParallelContext.single()
    t0 = time.time()
    model = H3Transformer(cfg, dev, torch.bfloat16, ctx).init_random(seed=0)
    vcfg = VideoVaeConfig.tiny() if tiny else VideoVaeConfig()
    if tiny:
        vcfg.latent_channels, vcfg.spatial = cfg.latent_channels, cfg.vae_spatial
    acfg = AudioVaeConfig.tiny() if tiny else AudioVaeConfig()
    if tiny:
        acfg.latent_channels = cfg.audio_channels
    video_vae = VideoVaeDecoder(vcfg, dev).init_random(seed=1)
    audio_vae = AudioVaeDecoder(acfg, dev).init_random(seed=2)
    svc = VideoService(model, video_vae, audio_vae)
    svc.text.max_tokens = n_text
    den = svc.denoiser
    fused = world > 1 and os.environ.get("US_NO_FUSED", "0") != "1"
    g = torch.Generator().manual_seed(7)
    K, W = args.steps, args.warmup
    nsteps = den.steps

    def measure(lf, lh, lw, n_audio, n_txt, k, w, sample_clocks):
        """Device time of ``k`` denoising steps after ``w`` warm-up steps on one clip."""
        feats = torch.randn(n_txt, cfg.text_dim, generator=g).pin_memory().to(dev)
        st = den.prepare(1000, lf, lh, lw, n_audio, feats)
        if fused:
            from uniserve_v1_b200.parallel.ulysses import FusedUlysses
            if model.ulysses is not None:
                model.ulysses.close()
            model.ulysses = FusedUlysses(ctx, dev, st.layout.rows, model.heads_local, cfg.head_dim)
        for i in range(w):
            st.step = i % nsteps
            den.step(st)
        sampler = ClockSampler(job.local, period_ms=100)
        if rank == 0 and sample_clocks:
            sampler.start()
            time.sleep(0.3)
        launches0 = native.launch_count

        def run():
            for i in range(k):
                st.step = i % nsteps
                den.step(st)
        ms, _, _ = job.timed(run)
        clocks = sampler.stop() if (rank == 0 and sample_clocks) else None
        native.raise_on_device_error()
        return ms, clocks, native.launch_count - launches0, st

    lf, lh, lw = cfg.latent_shape(frames, width, height)
    n_audio = cfg.audio_rows(frames)
    setup_s = time.time() - t0
    job.mark("fasth3 weights ready")
    ms, clocks, launches, st = measure(lf, lh, lw, n_audio, n_text, K, W, True)
    value = ms / K * nsteps / 1e3
    rows, used = st.layout.rows, st.layout.used
    job.mark("fasth3 steps timed")

    phase_ms = None
    if os.environ.get("BENCH_PROBES", "0") == "1":
        # one more step with fence probes around every phase of every block (diagnostic:
        # outside the timed region; the probes are tiny launches of their own)
        from uniserve_v1_b200.engine.profiling import ProbeRing
        from uniserve_v1_b200.tools.profile import device_ranges
        model.probe = ProbeRing(8192, dev)
        st.step = 0
        den.step(st)
        got = model.probe.collect()
        model.probe = None
        agg = {}
        for _, base, _, a, b, _ in device_ranges([(0,) + r for r in got]):
            agg[base] = agg.get(base, 0.0) + (b - a) / 1e6
        phase_ms = {k: round(v, 3) for k, v in sorted(agg.items())}

    e2e = None
    if not args.no_e2e:
        plan = VideoPlan("t2va", width, height, frames, 24, 1000, nsteps)
        prompt = "".join(chr(97 + (i * 7) % 26) for i in range(n_text))
        vjob = VideoJob(prompt, plan)
        svc.time_phases = os.environ.get("BENCH_PHASES", "0") == "1"
        # warm the request path once (one denoising step): decoder kernels loaded, pinned
        # buffers allocated - the timed request then is a steady-state one
        svc.generate(VideoJob(prompt, VideoPlan("t2va", width, height, frames, 24, 1000, 1)))
        job.mark("fasth3 request path warm")
        h0, d0 = svc.h2d_bytes, svc.d2h_bytes
        e2e_ms, wall, mp4 = job.timed(lambda: svc.generate(vjob))
        e2e = {"value": e2e_ms / 1e3, "unit": "s", "host_wall_s": round(wall, 3),
               "h2d_bytes_per_step": svc.h2d_bytes - h0, "d2h_bytes_per_step": svc.d2h_bytes - d0,
               "mp4_bytes": len(mp4),
               "phases_s": {k: round(v, 3) for k, v in vjob.timings.items()} or None,
               "step": "one whole request (bytes are per request)",
               "includes": "prompt features H2D from pinned memory, latent prepare, 8 steps, "
                           "video+audio VAE decode, colour conversion, plane read-back, MP4 mux"}
        job.mark("fasth3 request timed")

    baseline_shape = None
    want_big = (world >= 4 and not tiny and not args.layers) or args.baseline_shape
    if want_big and not args.no_baseline_shape:
        # the synthetic shape: 121 frames, 8x spatial / 4x temporal compression, 2x2 patches
        # -> 31 latent frames of 48 x 84 tokens; 5 s of audio latents; 512 text rows
        blf, blh, blw = (31, 96, 168) if not tiny else (5, 16, 16)
        kb, wb = (4, 3) if not tiny else (2, 3)
        bms, _, _, bst = measure(blf, blh, blw, 2 * 5 * cfg.audio_latents_per_second, 512
                                 if not tiny else 32, kb, wb, False)
        baseline_shape = {"value": bms / kb * nsteps / 1e3, "unit": "s", "steps": kb,
                          "warmup": wb, "ms_per_step": bms / kb,
                          "latent": [blf, blh // 2, blw // 2], "rows": bst.layout.rows,
                          "video_tokens": blf * (blh // 2) * (blw // 2), "text_tokens": 512,
                          "note": "121 frames at 1344x768 under 8x spatial / 4x temporal "
                                  "compression with 2x2 patches; the served VAE is 16x spatial, "
                                  "so this shape is measured on the transformer alone"}
        del bst
        job.mark("fasth3 baseline shape timed")

    par = "single GPU" if world == 1 else \
        f"ulysses{world} ({'all-to-all fused into the projection GEMMs' if fused else 'NCCL all_to_all'})"
    rec = {
        "metric": "FastH3 8-step clip latency", "value": value, "unit": "s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K,
        "higher_is_better": False, "scaling": "strong",
        "vs_baseline": value / (7.448 if args.mlp_fp8 else BASELINE_CLIP_S),
        "dtype": "bf16 + fp8 (e4m3) feed-forward projections" if args.mlp_fp8 else "bf16",
        "data": "synthetic (Philox N(0,1) latents, N(0,1) text features, uniform-random prompt "
                "ids, random-init N(0,0.02) weights)",
        "config": {"model": "MiniMax-H3/FastH3-shaped DiT" if not tiny else "tiny",
                   "layers": cfg.num_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_heads, "ffn": cfg.ffn_size, "frames": frames,
                   "size": f"{width}x{height}", "latent": [lf, lh, lw],
                   "rows": rows, "rows_used": used,
                   "global_batch": 1, "seq_len": used, "text_tokens": n_text,
                   "step": "one denoising step of the clip; value = 8 steps",
                   "parallelism": par,
                   "l2": "inputs larger than L2 (weights read per step >> 126 MB)",
                   "baseline": "8.194 s on 8xH200 (reference docs, whole request)"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
        "launches_per_step": launches // max(K, 1), "setup_s": round(setup_s, 1),
    }
    if baseline_shape:
        rec["baseline_shape"] = baseline_shape
    if phase_ms:
        rec["phase_ms_of_one_step"] = phase_ms
    if args.layers:
        rec["profile_only"] = True
    if model.ulysses is not None:
        model.ulysses.close()
        model.ulysses = None
    return rec


# ---------------------------------------------------------------- Qwen3-MoE --
def qwen3_record(job: Job) -> dict:
    """Qwen3-MoE output tokens/s; see the module docstring for what is timed."""
    import torch
    import torch.distributed as dist
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.ops import native
    from uniserve_v1_b200.parallel.context import ParallelContext

    args, world, rank, dev = job.args, job.world, job.rank, job.dev
    mark = job.mark
    layout = args.layout if world > 1 else "tp-ep"
    model_name = args.model if args.model in ("qwen3-30b-a3b", "qwen3-235b-a22b", "tiny") \
        else "qwen3-30b-a3b"
    cfg = Qwen3MoeConfig.qwen3_30b_a3b() if model_name == "qwen3-30b-a3b" else \
        Qwen3MoeConfig.qwen3_235b_a22b() if model_name == "qwen3-235b-a22b" else Qwen3MoeConfig(
        vocab_size=2048, hidden_size=512, num_hidden_layers=2, num_attention_heads=8,
        num_key_value_heads=2, head_dim=128, num_experts=16, num_experts_per_tok=4,
        moe_intermediate_size=256, eos_token_id=2047, max_position_embeddings=8192)
    if args.layers:
        cfg.num_hidden_layers = args.layers
    ctx = ParallelContext.single()
    sync_group, n_attn, is_attention = None, world, True
    exchange, control, announcer = None, None, None
    micro = []
    if world > 1:
        sync_group = dist.group.WORLD
        if layout == "tp-ep":
            ctx = ParallelContext.from_world(tensor=world, expert_over_tensor=True)
            mark("groups ready")
            if os.environ.get("US_NO_FUSED", "0") != "1":
                from uniserve_v1_b200.parallel.symm import attach_fused
                attach_fused(ctx, dev, hidden=cfg.hidden_size)
        else:
            from uniserve_v1_b200.parallel.expert_exchange import ExpertExchange
            ctx = ParallelContext.from_world(tensor=1)
            if layout == "afd":
                assert world % 2 == 0, "the afd layout splits the ranks in two halves"
                n_attn = world // 2
                ctx.source_ranks = tuple(range(n_attn))
                ctx.expert_ranks = tuple(range(n_attn, world))
                is_attention = rank < n_attn
                attn_group = dist.new_group(list(range(n_attn)))
                control = dist.new_group([0] + list(range(n_attn, world)), backend="gloo")
                sync_group = attn_group
            else:
                ctx.source_ranks = ctx.expert_ranks = tuple(range(world))
            exchange = ExpertExchange(dist.group.WORLD, rank, world, dev, 8192,
                                      cfg.num_experts_per_tok, cfg.hidden_size, cfg.num_experts,
                                      cfg.moe_intermediate_size, ctx.source_ranks,
                                      ctx.expert_ranks)
            if args.microbatches >= 2:
                micro = [ExpertExchange(dist.group.WORLD, rank, world, dev, 256,
                                        cfg.num_experts_per_tok, cfg.hidden_size, cfg.num_experts,
                                        cfg.moe_intermediate_size, ctx.source_ranks,
                                        ctx.expert_ranks) for _ in (0, 1)]
        mark("heap attached")

    if args.concurrency:
        C = args.concurrency
    else:
        C = 128 // n_attn if layout == "afd" else 64       # requests on this rank
    if layout == "afd" and args.concurrency:
        C = args.concurrency // n_attn
    tiny = model_name == "tiny"
    prompt_len = args.prompt_len or (512 if layout == "afd" else 1024)
    out_len = args.output_len or (1024 if layout == "afd" else 256)
    if tiny and not args.prompt_len:
        prompt_len, out_len = 96, 24
    K, W = max(args.steps, 64 if not tiny else args.steps), args.warmup
    total_steps = 2 * (K + W) + 8
    max_len = prompt_len + max(total_steps, out_len) + 16
    per_rank = layout != "tp-ep"
    total_c = C * (n_attn if per_rank else 1)

    t0 = time.time()
    model = Qwen3MoeModel(cfg, dev, torch.bfloat16, ctx,
                          expert_quant=args.expert_quant).init_random(seed=0)
    model.exchange = exchange
    if micro:
        model.micro_exchanges = micro
        model.microbatch_now = True        # every decode step of this run is micro-batched
    if world > 1 and layout == "tp-ep" and os.environ.get("US_NO_FUSED", "0") != "1":
        from uniserve_v1_b200.parallel.tp_fused import attach_fused_tp
        attach_fused_tp(model, 8192)          # prefill chunks: fused reduce-scatter / all-gather
    mark("weights ready")

    if not is_attention:
        # Expert rank of the disaggregated layout: join every announced forward.
        from uniserve_v1_b200.parallel.join import ExpertJoinLoop
        joins = ExpertJoinLoop(model, control, 0).run()
        torch.cuda.synchronize()
        native.raise_on_device_error()
        mark(f"joined {joins} forwards")
        return {}

    eng = LLMEngine(model, max_num_seqs=C, max_model_len=max_len,
                    max_num_batched_tokens=8192, enable_prefix_cache=False)
    if layout == "afd":
        from uniserve_v1_b200.parallel.join import StepAnnouncer
        announcer = StepAnnouncer(control, 0, rank == 0)
        eng.runner.announce = announcer
    g = torch.Generator().manual_seed(1234 + (rank if per_rank else 0))

    def new_prompts():
        return [torch.randint(0, cfg.vocab_size, (prompt_len,), generator=g).tolist()
                for _ in range(C)]
    sp = SamplingParams(temperature=0.0, max_tokens=total_steps + 4, ignore_eos=True)
    ids = [eng.add_request(p, sp) for p in new_prompts()]
    # Prefill every prompt (outside this timed region); ends with all rows decoding.
    while eng.scheduler.waiting or any(not r.output_ids for r in eng.scheduler.running):
        eng.step()
    torch.cuda.synchronize()
    setup_s = time.time() - t0
    first_tokens = [eng.scheduler.requests[i].output_ids[0] for i in ids[:8]]
    mark("prefill done")

    # ---- end to end through the public API: every step copies its input block
    # from pinned host memory and reads the sampled tokens back. ----
    e2e = None
    if not args.no_e2e:
        for _ in range(W):
            eng.step()
        mark("e2e warm-up done")
        h0, d0 = eng.runner.h2d_bytes, eng.runner.d2h_bytes

        def steps():
            for _ in range(K):
                eng.step()
        ms, _, _ = job.timed(steps, sync_group)
        e2e = {"value": total_c * K / (ms / 1e3), "unit": "output tokens/s",
               "ms_per_step": ms / K,
               "h2d_bytes_per_step": (eng.runner.h2d_bytes - h0) // K,
               "d2h_bytes_per_step": (eng.runner.d2h_bytes - d0) // K}
    mark("e2e done")

    # ---- device-timed decode steps: graph replays back to back, the device
    # advances its own step state; weights (57 GB) exceed L2, no flush needed. ----
    rows = list(eng.scheduler.running)
    for r in rows:
        need = eng.scheduler._pages_needed(r, r.num_tokens + K + W + 2)
        r.pages.extend(eng.blocks.allocate(need))
    runner = eng.runner
    B = runner.bucket_for(len(rows))
    blk = runner._decode_block(B)
    runner._fill_decode(blk, rows, B)
    graph = runner._graph(B, "greedy")
    blk.upload()
    runner.announce(runner._decode_kind("replay", B), B, W)
    for _ in range(W):
        graph.graph.replay()
    sampler = ClockSampler(job.local, period_ms=50)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches0 = native.launch_count
    runner.announce(runner._decode_kind("replay", B), B, K)

    def replays():
        for _ in range(K):
            graph.graph.replay()
            native.launch_count += graph.launches
    ms, _, _ = job.timed(replays, sync_group)
    clocks = sampler.stop() if rank == 0 else None
    mark("timed region done")
    native.raise_on_device_error()
    launches = native.launch_count - launches0
    value = total_c * K / (ms / 1e3)
    ctx_lo = rows[0].num_tokens

    # ---- the whole workload: C requests x (prompt_len in, out_len out) from the first
    # add_request to the last token, prefill included, through the engine's public calls ----
    workload = None
    if not args.no_workload:
        for rid in ids:
            eng.abort(rid)
        while eng.has_work():
            eng.step()
        prompts = new_prompts()
        spw = SamplingParams(temperature=0.0, max_tokens=out_len, ignore_eos=True)
        h0, d0 = eng.runner.h2d_bytes, eng.runner.d2h_bytes
        stats0 = dict(eng.scheduler.stats)

        def serve_all():
            rids = [eng.add_request(p, spw) for p in prompts]
            t_first = None
            n_steps = 0
            while eng.has_work():
                eng.step()
                n_steps += 1
                if t_first is None and all(eng.scheduler.requests[r].output_ids for r in rids):
                    t_first = time.perf_counter()
            return rids, t_first, n_steps
        t_begin = time.perf_counter()
        wms, wall, (rids, t_first, n_steps) = job.timed(serve_all, sync_group)
        done = sum(len(eng.scheduler.requests[r].output_ids) for r in rids)
        done_all = done * (n_attn if per_rank else 1)
        workload = {"value": done_all / (wms / 1e3), "unit": "output tokens/s",
                    "requests": total_c, "prompt_tokens": prompt_len, "output_tokens": out_len,
                    "device_s": wms / 1e3, "host_wall_s": round(wall, 3),
                    "time_to_all_first_tokens_s": round((t_first or t_begin) - t_begin, 3),
                    "engine_steps": n_steps, "tokens_out": done_all,
                    "prefill_tokens": eng.scheduler.stats.get("prefill_tokens", 0)
                    - stats0.get("prefill_tokens", 0),
                    "h2d_bytes": eng.runner.h2d_bytes - h0, "d2h_bytes": eng.runner.d2h_bytes - d0,
                    "includes": "add_request, chunked prefill, every decode step with its "
                                "host->device input copy and token read-back"}
        native.raise_on_device_error()
        mark("workload done")

    # ---- N > 1: the sharded model's first tokens against the same model on one rank
    # (two layers of the same shape, so both fit beside the benchmarked model) ----
    tp_check = None
    if world > 1 and layout == "tp-ep" and not args.no_tp_check:
        import dataclasses
        small = dataclasses.replace(cfg, num_hidden_layers=2)
        sp8 = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
        gp = torch.Generator().manual_seed(99)
        ps = [torch.randint(0, cfg.vocab_size, (48,), generator=gp).tolist() for _ in range(4)]
        outs = []
        for c in (ctx, ParallelContext.single()):
            m2 = Qwen3MoeModel(small, dev, torch.bfloat16, c).init_random(seed=5)
            e2 = LLMEngine(m2, num_pages=64, max_num_seqs=4, max_model_len=128,
                           enable_prefix_cache=False)
            outs.append(e2.generate(ps, sp8))
            e2.runner.release_graphs()
            del e2, m2
        flat = [(a, b) for x, y in zip(*outs) for a, b in zip(x, y)]
        tp_check = {"layers": 2, "prompts": 4, "tokens_compared": len(flat),
                    "tokens_equal": sum(a == b for a, b in flat),
                    "first_token_equal": sum(x[0] == y[0] for x, y in zip(*outs))}
        native.raise_on_device_error()
        mark("tp check done")

    par = {"tp-ep": "tp1" if world == 1 else f"tp{world}-attention+ep{world}",
           "dp-ep": f"dp{world}-attention+ep{world} (dispatch/combine over peer memory)",
           "afd": f"afd: attention dp{n_attn} + experts ep{world - n_attn}"}[layout]
    rec = {
        "metric": "Qwen3-MoE output tokens/s", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K,
        "higher_is_better": True, "scaling": "weak" if layout == "dp-ep" else "strong",
        "vs_baseline": value / BASELINE_TOK_S if model_name == "qwen3-30b-a3b" else None,
        "dtype": "bf16" if not args.expert_quant else "fp8 (e4m3, 128x128 blocks) experts + bf16 attention",
        "data": "synthetic (uniform-random prompt ids, random-init N(0,0.02) weights)",
        "config": {"model": {"qwen3-30b-a3b": "Qwen3-30B-A3B-shaped",
                             "qwen3-235b-a22b": "Qwen3-235B-A22B-shaped"}.get(model_name, "tiny"),
                   "layers": cfg.num_hidden_layers, "hidden": cfg.hidden_size,
                   "experts": cfg.num_experts, "top_k": cfg.num_experts_per_tok,
                   "global_batch": total_c, "seq_len": prompt_len,
                   "context_during_timing": [ctx_lo, ctx_lo + K + W],
                   "page_size": 16, "step": "one decode step of all concurrent requests",
                   "parallelism": par, "layout": layout, "microbatches": args.microbatches,
                   "l2": "inputs larger than L2 (weights read per step >> 126 MB)",
                   "baseline": "64 concurrent, 20.5 ms/step on 1xGB200 (reference docs)"},
        "clocks": clocks, "e2e": e2e, "workload": workload, "gpu_launches": launches,
        "launches_per_step": graph.launches, "setup_s": round(setup_s, 1),
        "first_tokens": first_tokens,
    }
    if tp_check:
        rec["tp_check"] = tp_check
    if args.layers:
        rec["profile_only"] = True
    mark("record ready")
    # Graphs that captured collectives must go before their communicator.
    if announcer is not None:
        announcer.stop()
    eng.runner.release_graphs()
    del graph
    if ctx.fused is not None:
        torch.cuda.synchronize()
        ctx.fused.close()
        ctx.fused = None
    return rec


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="all", choices=["all", "qwen3-moe", "fasth3"],
                    help="all (default): the FastH3 clip latency as the headline with the "
                         "Qwen3-MoE record nested; or one of the two alone")
    ap.add_argument("--frames", type=int, default=0, help="fasth3: frame count (rule 17n + 5)")
    ap.add_argument("--mlp-fp8", action="store_true",
                    help="fasth3: feed-forward projections in FP8 (per-tensor weights, per-row "
                         "dynamic activations); the line then reports dtype bf16 + fp8 MLPs")
    ap.add_argument("--baseline-shape", action="store_true",
                    help="fasth3: also time the synthetic 124,992-token shape (default at N >= 4)")
    ap.add_argument("--no-baseline-shape", action="store_true")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--concurrency", type=int, default=0,
                    help="qwen3-moe: concurrent requests (default 64; per rank in the dp-ep "
                         "layout; 128 in total in the afd layout)")
    ap.add_argument("--prompt-len", type=int, default=0)
    ap.add_argument("--output-len", type=int, default=0,
                    help="qwen3-moe: output tokens per request of the whole-workload run")
    ap.add_argument("--model", default="default",
                    choices=["default", "qwen3-30b-a3b", "qwen3-235b-a22b", "tiny"],
                    help="tiny: small shapes of both families (plumbing check, not a benchmark)")
    ap.add_argument("--expert-quant", default=None, choices=["fp8_block"],
                    help="block-scaled FP8 expert weights (128 x 128 blocks); the value is then "
                         "reported with dtype fp8 experts + bf16 attention")
    ap.add_argument("--microbatches", type=int, default=1,
                    help="dp-ep / afd layouts: 2 = decode steps as two interleaved half-batches")
    ap.add_argument("--layout", default="tp-ep", choices=["tp-ep", "dp-ep", "afd"],
                    help="qwen3-moe: tp-ep: attention heads split over all ranks, whole experts "
                         "per rank, all-reduce fused into the norms (strong scaling, the default); "
                         "dp-ep: data-parallel attention + expert-parallel dispatch/combine "
                         "(weak scaling: `concurrency` requests per rank); "
                         "afd: attention on the first half of the ranks, experts on the second")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-workload", action="store_true")
    ap.add_argument("--no-tp-check", action="store_true")
    ap.add_argument("--layers", type=int, default=0,
                    help="profiling only: cut the layer count (the printed line is then marked "
                         "profile_only and is not a benchmark value)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)

    job = Job(args)
    line = None
    if args.workload in ("all", "fasth3"):
        line = fasth3_record(job)
        release_device_memory()
    if args.workload in ("all", "qwen3-moe"):
        q = qwen3_record(job)
        if line is None:
            line = q
        else:
            line["metric"] = "FastH3 8-step clip latency (s); Qwen3-MoE output tokens/s nested"
            line["qwen3_moe"] = q
            line["gpu_launches"] = line["gpu_launches"] + q.get("gpu_launches", 0)
    if job.rank == 0 and line:
        print(json.dumps(line))
    job.mark("line printed")
    if job.world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        job.mark("exit")
        os._exit(0)     # skip communicator teardown: nothing is left to save
    return 0


if __name__ == "__main__":
    sys.exit(main())
