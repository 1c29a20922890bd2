"""Fused compute+collective kernels timed on real peers.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 \
        --master-port 29511 -m uniserve_v1_b200.tools.opbench_ranks [--ops norm,argmax,...]

One process per GPU.  Every kernel is timed with CUDA events on the launching stream, after
warm-up, a buffer larger than L2 written between iterations; the figure of an iteration is the
MAX over ranks (one all-reduce of the times after the loop), the figure reported is the median
iteration.  Every row gives the bytes that must cross NVLink per rank and the roofline time:
the slower of (FLOPs / measured bf16 GEMM peak) and (NVLink bytes / 770 GB/s, the measured
peer-copy bandwidth per direction), and achieved = roofline time / measured time.  Rows of
latency-bound kernels (a decode step's 64-row all-reduce moves 230 KB) say so: their floor is
the flag round trip, not the link.

No profiler is ever attached to this program: a kernel replay would re-run flag protocols.
Rank 0 prints one JSON object per row and a table at the end.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os

import torch
import torch.distributed as dist

from ..ops import functional as F
from ..ops import native as N
from .opbench import peaks

LINK_GBS = 770.0          # measured peer copy, per direction per GPU


class Bench:
    def __init__(self):
        self.rank = int(os.environ.get("RANK", 0))
        self.world = int(os.environ.get("WORLD_SIZE", 1))
        self.dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
        torch.cuda.set_device(self.dev)
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=self.dev)
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev)
        self.tbs, self.tflops, self.tag = peaks()
        self.rows = []
        self.g = torch.Generator(device=self.dev).manual_seed(1234 + self.rank)

    def rnd(self, *shape, scale=0.25, dtype=torch.bfloat16):
        return (torch.randn(*shape, generator=self.g, device=self.dev) * scale).to(dtype)

    def time(self, fn, iters=20, warmup=5):
        """Median over iterations of the max over ranks, in ms."""
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        ts = torch.zeros(iters, device=self.dev)
        for i in range(iters):
            self.flush.zero_()
            dist.barrier()          # ranks enter each iteration together, as in a served step
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts[i] = e0.elapsed_time(e1)
        dist.all_reduce(ts, op=dist.ReduceOp.MAX)
        return float(ts.sort().values[iters // 2])

    def row(self, name, ms, flops=0.0, link_bytes=0.0, hbm_bytes=0.0, note="", **extra):
        t_c = flops / (self.tflops * 1e12) * 1e3
        t_l = link_bytes / (LINK_GBS * 1e9) * 1e3
        t_m = hbm_bytes / (self.tbs * 1e12) * 1e3
        floor = max(t_c, t_l, t_m)
        r = dict(op=name, ranks=self.world, ms=round(ms, 4), link_mb_per_rank=round(link_bytes / 1e6, 3),
                 roofline_ms=round(floor, 4), bound=("compute" if floor == t_c else
                                                     "nvlink" if floor == t_l else "hbm"),
                 achieved=round(floor / ms, 3) if ms > 0 else None, roofline=self.tag, **extra)
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
        if link_bytes:
            r["link_gbs"] = round(link_bytes / ms / 1e6, 1)
        if note:
            r["note"] = note
        self.rows.append(r)
        if self.rank == 0:
            print(json.dumps(r), flush=True)


# ------------------------------------------------------------------------- ops --
def op_norm(b: Bench, a):
    """Decode all-reduce + residual + RMSNorm (push form), against NCCL all-reduce + the
    separate add-norm kernel."""
    from ..parallel.symm import FusedComm
    T, H, P = a.batch, a.hidden, b.world
    fc = FusedComm(dist.group.WORLD, b.rank, P, b.dev, H, sites=10, max_rows=256)
    w = torch.ones(H, dtype=torch.bfloat16, device=b.dev)
    part = b.rnd(T, H)
    res = torch.zeros(T, H, dtype=torch.float32, device=b.dev)
    ms = b.time(lambda: fc.allreduce_add_rmsnorm(part, res, w, 1e-6), a.iters)
    link = (P - 1) * T * H * 2.0
    b.row("allreduce_add_rmsnorm (push)", ms, link_bytes=link, rows=T, hidden=H,
          note="latency-bound: one flag crossing per step")

    def nccl():
        t = part.clone()
        dist.all_reduce(t)
        F.add_rmsnorm(t, res, w, 1e-6)
    ms2 = b.time(nccl, a.iters)
    b.row("nccl all_reduce + add_rmsnorm", ms2, link_bytes=link, rows=T, hidden=H, note="baseline")
    # routed form: the un-permute of the expert output rides on the all-reduce
    k = a.topk
    y = b.rnd(T * k, H)
    perm = torch.randperm(T * k, device=b.dev, generator=b.g).to(torch.int32).view(T, k)
    wts = torch.rand(T, k, device=b.dev, generator=b.g)
    ms3 = b.time(lambda: fc.allreduce_add_rmsnorm(None, res, w, 1e-6, routed=(y, perm, wts)),
                 a.iters)
    b.row("unpermute + allreduce_add_rmsnorm (push)", ms3, link_bytes=link, rows=T, hidden=H,
          top_k=k)
    V = 151936 // P
    logits = b.rnd(T, V, dtype=torch.float32, scale=1.0)
    ms4 = b.time(lambda: fc.argmax(logits, V, b.rank * V), a.iters)
    b.row("sharded argmax exchange", ms4, link_bytes=(P - 1) * T * 8.0, hbm_bytes=T * V * 4.0,
          rows=T, cols=V)

    def nccl_gather():
        box = torch.empty(P, T, V, dtype=torch.float32, device=b.dev)
        dist.all_gather_into_tensor(box, logits)
        box.permute(1, 0, 2).reshape(T, P * V).argmax(-1)
    ms5 = b.time(nccl_gather, a.iters)
    b.row("nccl all_gather logits + argmax", ms5, link_bytes=(P - 1) * T * V * 4.0, rows=T,
          note="baseline")
    fc.close()


def op_ulysses(b: Bench, a):
    """The three fused steps of a Ulysses attention block at the video shape: QKV projection
    scattering to the head owners, attention pushing rows to the row owners, local to_out."""
    from ..parallel.symm import FusedComm
    P, D = b.world, 128
    heads = a.heads_total
    if heads % P:
        heads = (heads + P - 1) // P * P          # the model pads its heads the same way
    hl = heads // P
    H = a.model_dim
    unit = 128 * P
    rows = (a.rows + unit - 1) // unit * unit
    ro = rows // P
    W = 3 * hl * D
    fc = FusedComm(dist.group.WORLD, b.rank, P, b.dev, hidden=0, sites=6, site_bytes=rows * W * 2)
    x = b.rnd(ro, H)
    wqkv, wout = b.rnd(P * W, H, scale=0.02), b.rnd(H, P * hl * D, scale=0.02)

    def ptrs(site):
        return (ctypes.c_void_p * P)(*[fc.peer_site_ptr(r, site) for r in range(P)])
    p_qkv, p_att = ptrs(0), ptrs(1)
    st = N.stream()
    bn = F._block_n(ro, False)
    from ..parallel import ulysses as _U          # registers the signatures
    del _U

    def scatter():
        N.call("us_gemm_wx_scatter", N.ptr(wqkv), N.ptr(x), P * W, H, ro, H, x.stride(0), W,
               p_qkv, W, b.rank * ro, bn, st)
        fc.barrier(2)
    ms1 = b.time(scatter, a.iters)
    b.row("QKV GEMM + Ulysses scatter (+flag barrier)", ms1, flops=2.0 * ro * P * W * H,
          link_bytes=(P - 1) * ro * W * 2.0, rows_own=ro, hidden=H, heads_local=hl)
    full = fc.site_tensor(0, rows, W)
    full.copy_(b.rnd(rows, W))
    q, k, v = full[:, :hl * D], full[:, hl * D:2 * hl * D], full[:, 2 * hl * D:]
    cu = torch.tensor([0, rows], dtype=torch.int32, device=b.dev)
    inner = P * hl * D
    scale = 1.0 / math.sqrt(D)

    def flash():
        N.call("us_flash_attn_push", N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(cu), N.ptr(cu), rows, rows,
               hl, hl, full.stride(0), full.stride(0), full.stride(0), scale, p_att, P, ro,
               b.rank * hl * D, inner, st)
        fc.barrier(3)
    ms2 = b.time(flash, max(3, a.iters // 4), warmup=2)
    b.row("flash attention + Ulysses return push (+flag barrier)", ms2,
          flops=4.0 * rows * rows * hl * D, link_bytes=(P - 1) * ro * hl * D * 2.0, rows=rows,
          heads_local=hl)
    att = fc.site_tensor(1, ro, inner)
    ms3 = b.time(lambda: F.linear(att, wout), a.iters)
    b.row("to_out GEMM (local after push)", ms3, flops=2.0 * ro * H * inner, rows_own=ro)

    def nccl_a2a():
        src = full[:ro * P].view(P, ro, W)
        dst = torch.empty_like(src)
        dist.all_to_all_single(dst, src.contiguous())
    ms4 = b.time(nccl_a2a, a.iters)
    b.row("nccl all_to_all of the QKV rows", ms4, link_bytes=(P - 1) * ro * W * 2.0,
          note="baseline: the transfer the scatter epilogue hides")
    fc.close()


def op_tp(b: Bench, a):
    """Tensor-parallel MLP on the peer heap: all-gather -> gated GEMM, GEMM -> reduce-scatter,
    slot sum + residual + norm."""
    from ..parallel import tp_fused as TP
    P = b.world
    rows, H, I = a.tp_rows, a.model_dim, a.ffn // P
    unit = 128 * P
    rows = (rows + unit - 1) // unit * unit
    tp = TP.FusedTP(dist.group.WORLD, b.rank, P, b.dev, rows, H)
    tp.gathered(TP.SITE_NORM_A).copy_(b.rnd(rows, H))
    w13, w2, nw = b.rnd(2 * I, H, scale=0.02), b.rnd(H, I, scale=0.02), b.rnd(H)
    res = torch.zeros(rows // P, H, dtype=torch.float32, device=b.dev)
    hid = tp.gather_linear(w13, TP.SITE_NORM_A, gated=True)
    ms1 = b.time(lambda: tp.gather_linear(w13, TP.SITE_NORM_A, gated=True), a.iters)
    b.row("all-gather -> gated up GEMM", ms1, flops=4.0 * rows * I * H,
          link_bytes=(P - 1) * (rows // P) * H * 2.0, rows=rows, hidden=H, inter_local=I)
    ms2 = b.time(lambda: tp.reduce_scatter_linear(w2, hid), a.iters)
    b.row("down GEMM -> reduce-scatter (peer stores)", ms2, flops=2.0 * rows * I * H,
          link_bytes=(P - 1) * (rows // P) * H * 2.0, rows=rows)
    ms3 = b.time(lambda: tp.reduce_add_rmsnorm(res, nw, TP.SITE_NORM_B, 1e-6), a.iters)
    b.row("slot sum + residual + RMSNorm + all-gather stores", ms3,
          hbm_bytes=(rows // P) * H * (2.0 * P + 4 + 4 + 2),
          link_bytes=(P - 1) * (rows // P) * H * 2.0, rows_own=rows // P)

    def nccl():
        full = torch.empty(rows, H, dtype=torch.bfloat16, device=b.dev)
        dist.all_gather_into_tensor(full, tp.own_rows(TP.SITE_NORM_A).contiguous())
        y = F.linear(F.linear_gated(full, w13), w2)
        out = torch.empty(rows // P, H, dtype=torch.bfloat16, device=b.dev)
        dist.reduce_scatter_tensor(out, y)
    ms4 = b.time(nccl, a.iters)
    b.row("nccl all_gather + GEMMs + reduce_scatter", ms4, flops=6.0 * rows * I * H,
          link_bytes=2.0 * (P - 1) * (rows // P) * H * 2.0, note="baseline for the sum of the rows above")
    tp.close()


def op_ep(b: Bench, a):
    """One expert-parallel MoE layer, every rank both attention member and expert holder:
    dispatch by peer stores, grouped FC1/FC2 with the gate-weighted push, combine + norm."""
    from ..parallel.expert_exchange import ExpertExchange
    P = b.world
    T, E, k, H, I = a.batch, a.experts, a.topk, a.hidden, a.inter
    ex = ExpertExchange(dist.group.WORLD, b.rank, P, b.dev, T, k, H, E, I)
    El = E // P
    x = b.rnd(T, H)
    w13, w2, nw = b.rnd(El, 2 * I, H, scale=0.05), b.rnd(El, H, I, scale=0.05), b.rnd(H)
    logits = torch.randn(T, E, generator=b.g, device=b.dev)
    ids, wts = F.topk_softmax(logits, k, True)
    live = torch.full((1,), T, dtype=torch.int32, device=b.dev)
    res = torch.zeros(T, H, dtype=torch.float32, device=b.dev)

    def layer():
        ex.dispatch(x, ids, wts, live)
        ex.experts(w13, w2, T)
        ex.combine_add_rmsnorm(ids, live, res, nw, 1e-6)
    ms = b.time(layer, a.iters)
    away = T * k * (P - 1) / P                    # expected routed rows that leave the rank
    b.row("EP layer: dispatch + FC1 + FC2 push + combine", ms, link_bytes=2.0 * away * H * 2.0,
          hbm_bytes=min(El, T * P * k) * 3.0 * I * H * 2.0, tokens_per_rank=T, experts_local=El)

    def hand_off():
        ex.dispatch(x, ids, wts, live)
    ms2 = b.time(hand_off, a.iters)
    b.row("EP dispatch alone (attention -> expert hand-off)", ms2, link_bytes=away * H * 2.0,
          tokens_per_rank=T, note="latency-bound at decode sizes")
    ex.close()


OPS = {"norm": op_norm, "ulysses": op_ulysses, "tp": op_tp, "ep": op_ep}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="norm,ep,tp,ulysses")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--inter", type=int, default=768)
    ap.add_argument("--rows", type=int, default=38912, help="ulysses: rows of the whole clip")
    ap.add_argument("--heads-total", type=int, default=42)
    ap.add_argument("--model-dim", type=int, default=5376)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--tp-rows", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default=None, help="rank 0 writes the table (markdown) here")
    a = ap.parse_args()
    b = Bench()
    for name in a.ops.split(","):
        OPS[name](b, a)
        N.raise_on_device_error()
        dist.barrier()
    if b.rank == 0:
        lines = ["| op | ranks | ms (max over ranks) | NVLink MB/rank | roofline ms | bound | achieved |",
                 "|---|---|---|---|---|---|---|"]
        for r in b.rows:
            lines.append(f"| {r['op']} | {r['ranks']} | {r['ms']} | {r['link_mb_per_rank']} | "
                         f"{r['roofline_ms']} | {r['bound']} | {r['achieved']} |")
        text = "\n".join(lines)
        print(text)
        if a.out:
            with open(a.out, "w") as f:
                f.write(text + "\n")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
