"""Micro-benchmarks of the hot kernels with roofline fractions.

    python -m uniserve_v1_b200.tools.opbench flash --rows 37710 --heads 7
    python -m uniserve_v1_b200.tools.opbench gemm --rows 37710 --m 5376 --k 5376
    python -m uniserve_v1_b200.tools.opbench gated --rows 37710 --m 14336 --k 5376
    python -m uniserve_v1_b200.tools.opbench decode --batch 64 --ctx 1024

Timing: CUDA events on the launching stream, warm-up first, a buffer larger than
L2 is written between timed iterations.  Fractions are "of measured": the
denominators come from ``MEASURED_PEAKS.json`` at the repository root when it
exists (copy bandwidth and cuBLAS bf16 throughput measured on the pool), else
the fallback 6.65 TB/s / 1.59 PFLOP/s ("of fallback").
"""
from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

import torch

from ..ops import functional as F
from ..ops.flash import flash_attn_varlen


def peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"] / 1e3, d["bf16_tflops"], "of measured"
    return 6.65, 1590.0, "of fallback"


def timeit(fn, iters=10, warmup=3):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["prefill", "delta", "flash", "gemm", "gated", "decode", "moe", "fused-norm",
                                   "ulysses", "tp", "moe-fp8", "gemm-fp8", "gemm-fp8t", "ep",
                                   "rank-decode"])
    ap.add_argument("--tp", type=int, default=8, help="rank-decode: ranks of the emulated layout")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--splits", type=int, default=0, help="decode: KV splits (0 = heuristic)")
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--q-heads", type=int, default=32)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--inter", type=int, default=768)
    ap.add_argument("--rows", type=int, default=37710)
    ap.add_argument("--heads", type=int, default=7)
    ap.add_argument("--m", type=int, default=5376)
    ap.add_argument("--k", type=int, default=5376)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--head-dim", type=int, default=128, help="flash: 128 or 64")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--kv", default="bf16", choices=["bf16", "fp8"], help="decode: page type")
    ap.add_argument("--persist", action="store_true",
                    help="decode: the persistent kernel (bf16 pages)")
    a = ap.parse_args()
    tbs, tfl, tag = peaks()
    dev, bf = "cuda", torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: (torch.randn(*s, generator=g, device=dev) * 0.5).to(bf)
    out = {"op": a.op}
    if a.op == "flash":
        T, H, D = a.rows, a.heads, a.head_dim
        q, k, v = rnd(T, H, D), rnd(T, H, D), rnd(T, H, D)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        o = torch.empty_like(q)
        ms = timeit(lambda: flash_attn_varlen(q, k, v, cu, cu, T, T, 1 / math.sqrt(D), a.causal,
                                              out=o), a.iters)
        flops = 4.0 * T * T * D * H * (0.5 if a.causal else 1.0)
        out.update(rows=T, heads=H, head_dim=D, ms=ms, tflops=flops / ms / 1e9, frac=flops / ms / 1e9 / tfl)
    elif a.op == "prefill":
        # One prefill chunk through the engine at the real widths: `--batch` prompts of `--ctx`
        # tokens (one chunk of batch x ctx rows), `--layers` layers.  ms_per_layer is what a
        # 48-layer model pays per chunk; a launch list of this command shows the shares.
        from ..engine.engine import LLMEngine
        from ..engine.types import SamplingParams
        from ..models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
        cfg = Qwen3MoeConfig.qwen3_30b_a3b()
        cfg.num_hidden_layers = a.layers
        model = Qwen3MoeModel(cfg, dev, bf).init_random(seed=0)
        rows = a.batch * a.ctx
        eng = LLMEngine(model, max_num_seqs=a.batch, max_model_len=a.ctx + 64,
                        max_num_batched_tokens=rows, enable_prefix_cache=False)
        gp = torch.Generator().manual_seed(1)
        sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
        times = []
        for it in range(a.iters + 2):
            for _ in range(a.batch):
                eng.add_request(torch.randint(0, cfg.vocab_size, (a.ctx,), generator=gp).tolist(), sp)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            while eng.has_work():
                eng.step()
            e1.record()
            torch.cuda.synchronize()
            if it >= 2:
                times.append(e0.elapsed_time(e1))
        times.sort()
        ms = times[len(times) // 2]
        out.update(rows=rows, layers=a.layers, ms=ms, ms_per_layer=ms / a.layers,
                   tokens_per_s=rows / ms * 1e3 * a.layers / 48,
                   note="tokens_per_s is scaled to 48 layers; embedding, head and sampling "
                        "of the last rows are in ms once")
    elif a.op == "rank-decode":
        # One rank's share of a tensor-parallel + whole-experts decode step, alone on one GPU:
        # the model is built as rank 0 of `--tp` ranks over a detached context whose
        # collectives are local stand-ins (results are meaningless, kernel shapes are the
        # rank's), so the per-rank compute floor of the N-GPU step can be timed and profiled
        # without peers.  --layers cuts the depth; ms_per_layer is what scales.
        from ..engine.engine import LLMEngine
        from ..engine.types import SamplingParams
        from ..models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
        from ..parallel.context import Axis, ParallelContext

        class Detached(ParallelContext):
            def all_reduce(self, x, axis="tensor"):
                return x

            def all_gather_tp_cols(self, x):
                return x.repeat(1, self.tp_size)

        P = a.tp
        ctx = Detached(world_rank=0, world_size=P)
        ctx.axes["tensor"] = Axis(None, 0, P, tuple(range(P)))
        ctx.axes["expert"] = ctx.axes["tensor"]
        ctx.expert_parallel = True
        cfg = Qwen3MoeConfig.qwen3_30b_a3b()
        cfg.num_hidden_layers = a.layers
        model = Qwen3MoeModel(cfg, dev, bf, ctx).init_random(seed=0)
        eng = LLMEngine(model, max_num_seqs=a.batch, max_model_len=a.ctx + 64,
                        enable_prefix_cache=False)
        gp = torch.Generator().manual_seed(1)
        sp = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
        for _ in range(a.batch):
            eng.add_request(torch.randint(0, cfg.vocab_size, (a.ctx,), generator=gp).tolist(), sp)
        while eng.scheduler.waiting or any(not r.output_ids for r in eng.scheduler.running):
            eng.step()
        rows = list(eng.scheduler.running)
        for r in rows:
            r.pages.extend(eng.blocks.allocate(eng.scheduler._pages_needed(r, r.num_tokens + 40)))
        runner = eng.runner
        B = runner.bucket_for(len(rows))
        blk = runner._decode_block(B)
        runner._fill_decode(blk, rows, B)
        graph = runner._graph(B, "greedy")
        blk.upload()
        for _ in range(3):
            graph.graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            graph.graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.iters
        out.update(tp=P, layers=a.layers, batch=a.batch, ctx=a.ctx, ms_per_step=ms,
                   launches=graph.launches, ms_per_layer=ms / a.layers,
                   note="includes embedding, head and sampling once per step")
    elif a.op in ("gemm", "gated"):
        x = rnd(a.rows, a.k)
        w = rnd(a.m * (2 if a.op == "gated" else 1), a.k)
        fn = (lambda: F.linear_gated(x, w)) if a.op == "gated" else (lambda: F.linear(x, w))
        ms = timeit(fn, a.iters)
        flops = 2.0 * a.rows * w.shape[0] * a.k
        byts = 2.0 * (x.numel() + w.numel() + a.rows * a.m)
        out.update(rows=a.rows, m=a.m, k=a.k, ms=ms, tflops=flops / ms / 1e9,
                   frac_compute=flops / ms / 1e9 / tfl, tbs=byts / ms / 1e9,
                   frac_memory=byts / ms / 1e9 / tbs)
    elif a.op == "moe":
        # one MoE layer of a decode step: route, sort, gather, grouped FC1 + FC2, un-permute
        T, E, k, H, I = a.batch, a.experts, a.topk, a.hidden, a.inter
        x = rnd(T, H)
        w13, w2 = rnd(E, 2 * I, H), rnd(E, H, I)
        logits = torch.randn(T, E, generator=g, device=dev)
        ids, wts = F.topk_softmax(logits, k, True)
        ws = F.MoeWorkspace.create(T, k, E, H, I, dev)
        ms = timeit(lambda: F.moe_experts(x, ids, wts, w13, w2, ws=ws), a.iters)
        active = int(torch.unique(ids).numel())
        byts = active * (w13[0].numel() + w2[0].numel()) * 2.0
        out.update(tokens=T, experts=E, active_experts=active, ms=ms, tbs=byts / ms / 1e9,
                   frac_memory=byts / ms / 1e9 / tbs)
    elif a.op == "moe-fp8":
        # the same layer with block-scaled FP8 expert weights (quantise rows, grouped FC1,
        # quantise, grouped FC2)
        from ..ops import fp8 as Q
        T, E, k, H, I = a.batch, a.experts, a.topk, a.hidden, a.inter
        x = rnd(T, H)
        ex = Q.Fp8Experts.from_bf16(rnd(E, 2 * I, H), rnd(E, H, I))
        logits = torch.randn(T, E, generator=g, device=dev)
        ids, wts = F.topk_softmax(logits, k, True)
        ws = F.MoeWorkspace.create(T, k, E, H, I, dev)
        if ws.block_n > 64:
            ws = F.MoeWorkspace.create(T, k, E, H, I, dev, block_n=64)
        ms = timeit(lambda: Q.moe_experts_fp8(x, ids, wts, ex, ws=ws), a.iters)
        active = int(torch.unique(ids).numel())
        byts = active * (ex.w13[0].numel() + ex.w2[0].numel()) * 1.0
        flops = 2.0 * T * k * 3 * I * H
        out.update(tokens=T, experts=E, active_experts=active, block_n=ws.block_n, ms=ms,
                   tbs=byts / ms / 1e9, frac_memory=byts / ms / 1e9 / tbs,
                   tflops=flops / ms / 1e9)
    elif a.op == "gemm-fp8":
        from ..ops import fp8 as Q
        x, w = rnd(a.rows, a.k), rnd(a.m, a.k)
        wq, wsc = Q.quantize_weight_block128(w)
        xq, xs = Q.quantize_rows_block128(x)
        ms = timeit(lambda: Q.linear_fp8_block(None, wq, wsc, xq=xq, x_scale=xs), a.iters)
        msq = timeit(lambda: Q.quantize_rows_block128(x, None, xq, xs), a.iters)
        flops = 2.0 * a.rows * a.m * a.k
        byts = 1.0 * (x.numel() + w.numel()) + 2.0 * a.rows * a.m
        out.update(rows=a.rows, m=a.m, k=a.k, ms=ms, tflops=flops / ms / 1e9,
                   tbs=byts / ms / 1e9, frac_memory=byts / ms / 1e9 / tbs, quantize_ms=msq,
                   quantize_tbs=3.0 * x.numel() / msq / 1e9)
    elif a.op == "ep":
        # one expert-parallel MoE layer with this rank as the only member of both role
        # sets: route + dispatch (peer stores), sort + gather + grouped FC1, FC2 whose
        # epilogue pushes gate-weighted rows to the token owner, combine + residual + norm
        from ..parallel.expert_exchange import ExpertExchange
        T, E, k, H, I = a.batch, a.experts, a.topk, a.hidden, a.inter
        ex = ExpertExchange(None, 0, 1, dev, T, k, H, E, I)
        x = rnd(T, H)
        w13, w2, nw = rnd(E, 2 * I, H), rnd(E, H, I), rnd(H)
        logits = torch.randn(T, E, generator=g, device=dev)
        ids, wts = F.topk_softmax(logits, k, True)
        live = torch.full((1,), T, dtype=torch.int32, device=dev)
        res = torch.zeros(T, H, dtype=torch.float32, device=dev)

        def layer():
            ex.dispatch(x, ids, wts, live)
            ex.experts(w13, w2, T)
            ex.combine_add_rmsnorm(ids, live, res, nw, 1e-6)
        ms = timeit(layer, a.iters)
        active = int(torch.unique(ids).numel())
        byts = active * (w13[0].numel() + w2[0].numel()) * 2.0
        out.update(tokens=T, experts=E, active_experts=active, ms=ms, tbs=byts / ms / 1e9,
                   frac_memory=byts / ms / 1e9 / tbs)
    elif a.op == "gemm-fp8t":
        # per-tensor weights, per-row activations, whole-K accumulation (persistent kernel);
        # the reference quotes 1525 TFLOPS for 32768 x 28672 x 5376 with pre-encoded operands
        from ..ops import fp8 as Q
        from ..ops import native as N_
        x, w = rnd(a.rows, a.k), rnd(a.m, a.k)
        wq, wsc = Q.quantize_weight_tensor(w)
        xq, xs = Q.quantize_rows(x, wsc)
        o = torch.empty(a.rows, a.m, dtype=bf, device=dev)
        run = lambda: N_.call("us_gemm_fp8_rowscale", N_.ptr(wq), N_.ptr(xq), N_.ptr(o), a.m, a.m,
                              a.k, a.rows, a.k, a.k, a.m, 0, 0, 0, 0, N_.ptr(xs), 256, N_.stream())
        ms = timeit(run, a.iters)
        msq = timeit(lambda: Q.quantize_rows(x, wsc), a.iters)
        flops = 2.0 * a.rows * a.m * a.k
        out.update(rows=a.rows, m=a.m, k=a.k, ms=ms, tflops=flops / ms / 1e9, quantize_ms=msq,
                   with_quantize_tflops=flops / (ms + msq) / 1e9)
    elif a.op == "fused-norm":
        # all-reduce + residual + RMSNorm over the peer heap; one rank (its own peer) so a
        # profiler can attach; the 2/8-rank numbers come from bench.py
        from ..ops import native as N_
        from ..parallel.symm import FusedComm
        T, H = a.batch, a.hidden
        fc = FusedComm(None, 0, 1, dev, H, sites=4)
        w = torch.ones(H, dtype=bf, device=dev)
        part = rnd(T, H)
        res = torch.zeros(T, H, dtype=torch.float32, device=dev)
        ms = timeit(lambda: fc.allreduce_add_rmsnorm(part, res, w, 1e-6), a.iters)
        out.update(rows=T, hidden=H, ms=ms)
    elif a.op == "ulysses":
        # the two fused GEMMs of the Ulysses block with this rank as its own peer:
        # QKV projection scattering from the epilogue, to_out pulling its K slices by TMA
        import ctypes
        from ..ops import native as N_
        from ..parallel import ulysses as U
        from ..parallel.symm import FusedComm
        rows, H, hl, D = a.rows, a.m, a.heads, 128
        W = 3 * hl * D
        fc = FusedComm(None, 0, 1, dev, 0, sites=4, site_bytes=rows * max(W, H) * 2)
        x = rnd(rows, H)
        wqkv, wout = rnd(W, H), rnd(H, hl * D)
        ptr_q = (ctypes.c_void_p * 1)(fc.peer_site_ptr(0, 0))
        ptr_a = (ctypes.c_void_p * 1)(fc.peer_site_ptr(0, 1))
        fc.site_tensor(1, rows, hl * D).copy_(rnd(rows, hl * D))
        o = torch.empty(rows, H, dtype=bf, device=dev)
        bn = F._block_n(rows, False)
        ms1 = timeit(lambda: N_.call("us_gemm_wx_scatter", N_.ptr(wqkv), N_.ptr(x), W, H, rows, H,
                                     H, W, ptr_q, W, 0, bn, N_.stream()), a.iters)
        ms2 = timeit(lambda: N_.call("us_gemm_wx_pull", N_.ptr(wout), ptr_a, 1, hl * D, N_.ptr(o),
                                     H, hl * D, rows, hl * D, hl * D, H, 0, bn, N_.stream()),
                     a.iters)
        # the Ulysses return: attention over the scattered heads, rows pushed to their owner
        full = fc.site_tensor(0, rows, W)
        full.copy_(rnd(rows, W))
        qh, kh, vh = full[:, :hl * D], full[:, hl * D:2 * hl * D], full[:, 2 * hl * D:]
        cu = torch.tensor([0, rows], dtype=torch.int32, device=dev)
        ms3 = timeit(lambda: N_.call("us_flash_attn_push", N_.ptr(qh), N_.ptr(kh), N_.ptr(vh),
                                     N_.ptr(cu), N_.ptr(cu), rows, rows, hl, hl, W, W, W,
                                     1.0 / math.sqrt(D), ptr_a, 1, rows, 0, hl * D, N_.stream()),
                     max(2, a.iters // 3))
        out.update(push_ms=ms3, push_tflops=4.0 * rows * rows * hl * D / ms3 / 1e9)
        out.update(rows=rows, hidden=H, heads_local=hl, scatter_ms=ms1,
                   scatter_tflops=2.0 * rows * W * H / ms1 / 1e9, pull_ms=ms2,
                   pull_tflops=2.0 * rows * H * hl * D / ms2 / 1e9)
    elif a.op == "delta":
        # recurrent layer kernels at the Qwen3.5 shape: a decode step of `batch` sequences
        # (state traffic bound) and a prefill of `rows` tokens of one sequence (latency bound)
        from ..ops import gated_delta as GD
        Hk, Hv, Dk, Dv = 16, 32, 128, 128
        B = a.batch
        pool = torch.zeros(B, Hv, Dk, Dv, dtype=torch.float32, device=dev)
        A = -(torch.rand(Hv, device=dev) * 2 + 0.2)
        dtb = torch.rand(Hv, device=dev)

        def run(T, cu, slots):
            q, k, v = rnd(T, Hk, Dk), rnd(T, Hk, Dk), rnd(T, Hv, Dv)
            ar, br = rnd(T, Hv), rnd(T, Hv)
            return timeit(lambda: GD.gated_delta_rule_packed(q, k, v, pool, cu, slots,
                                                             raw=(ar, br, A, dtb)), a.iters)
        cu = torch.arange(B + 1, dtype=torch.int32, device=dev)
        ms_dec = run(B, cu, cu[:B])
        T = min(a.rows, 4096)
        cu1 = torch.tensor([0, T], dtype=torch.int32, device=dev)
        ms_pre = run(T, cu1, cu[:1])
        state_bytes = 2.0 * B * Hv * Dk * Dv * 4
        C = 2 * Hk * Dk + Hv * Dv
        x, w = rnd(T, C), rnd(C, 4)
        st = torch.zeros(1, 3, C, dtype=bf, device=dev)
        ms_conv = timeit(lambda: GD.causal_conv1d(x, w, st, cu=cu1, slots=cu[:1]), a.iters)
        out.update(batch=B, decode_ms=ms_dec, decode_tbs=state_bytes / ms_dec / 1e9,
                   frac_memory=state_bytes / ms_dec / 1e9 / tbs, prefill_tokens=T,
                   prefill_ms=ms_pre, us_per_token=ms_pre * 1e3 / T, conv_ms=ms_conv,
                   conv_tbs=2.0 * T * C * 2 / ms_conv / 1e9)
    elif a.op == "tp":
        # the fused tensor-parallel MLP with this rank as its own (only) peer: gated
        # up-projection gathering its rows by TMA from the heap, down-projection
        # storing its partial rows into the owner's slot, slot sum + residual + norm
        from ..parallel import tp_fused as TP
        rows, H, I = a.rows, a.m, a.inter
        tp = TP.FusedTP(None, 0, 1, dev, rows, H)
        tp.gathered(TP.SITE_NORM_A).copy_(rnd(rows, H))
        w13, w2, nw = rnd(2 * I, H), rnd(H, I), rnd(H)
        res = torch.zeros(rows, H, dtype=torch.float32, device=dev)
        hid = tp.gather_linear(w13, TP.SITE_NORM_A, gated=True)
        ms1 = timeit(lambda: tp.gather_linear(w13, TP.SITE_NORM_A, gated=True), a.iters)
        ms2 = timeit(lambda: tp.reduce_scatter_linear(w2, hid), a.iters)
        ms3 = timeit(lambda: tp.reduce_add_rmsnorm(res, nw, TP.SITE_NORM_B, 1e-6), a.iters)
        out.update(rows=rows, hidden=H, inter_local=I, gather_gated_ms=ms1,
                   gather_gated_tflops=4.0 * rows * I * H / ms1 / 1e9, reduce_scatter_ms=ms2,
                   reduce_scatter_tflops=2.0 * rows * I * H / ms2 / 1e9, reduce_norm_ms=ms3,
                   reduce_norm_tbs=rows * H * (2 + 4 + 4 + 2) / ms3 / 1e9)
    else:
        B, Hq, Hkv, D, page = a.batch, a.q_heads, a.kv_heads, 128, 16
        per = (a.ctx + page - 1) // page
        pages = B * per + 1
        kc, vc = rnd(pages, page, Hkv, D), rnd(pages, page, Hkv, D)
        q = rnd(B, Hq, D)
        pt = (torch.randperm(pages - 1, device=dev)[:B * per].view(B, per) + 1).to(torch.int32)
        sl = torch.full((B,), a.ctx, dtype=torch.int32, device=dev)
        splits = a.splits or F.decode_splits(B, Hkv, a.ctx)
        scratch, counters = F.decode_scratch(B, Hq, Hkv, D, splits, dev)
        if a.persist and a.kv == "bf16":      # one CTA per SM over the launch's tile list
            splits = F.PERSIST_SPLITS
            scratch, counters = F.decode_persist_scratch(B, Hkv, dev)
        ks = vs = None
        esz = 2.0
        if a.kv == "fp8":            # E4M3 pages with one scale per page and plane
            kc = torch.randint(0, 120, kc.shape, dtype=torch.uint8, device=dev)
            vc = torch.randint(0, 120, vc.shape, dtype=torch.uint8, device=dev)
            ks = torch.rand(pages, device=dev) * 0.01 + 0.001
            vs = torch.rand(pages, device=dev) * 0.01 + 0.001
            esz = 1.0
        ms = timeit(lambda: F.paged_decode_attention(q, kc, vc, pt, sl, 1 / math.sqrt(D), splits,
                                                     scratch=scratch, counters=counters,
                                                     k_scale=ks, v_scale=vs),
                    a.iters)
        byts = 2.0 * B * a.ctx * Hkv * D * esz
        out["kv"] = a.kv
        out.update(batch=B, ctx=a.ctx, splits=splits, persistent=bool(a.persist and a.kv == "bf16"), ms=ms, tbs=byts / ms / 1e9,
                   frac_memory=byts / ms / 1e9 / tbs)
    out["roofline"] = tag
    print(json.dumps(out))


if __name__ == "__main__":
    main()
