"""Each CUDA kernel against the plain PyTorch FP32 restatement of the same op."""
import math

import pytest
import torch

from uniserve_v1_b200.ops import functional as F
from uniserve_v1_b200.ops import native as N
from uniserve_v1_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def rnd(*shape, scale=1.0, dtype=BF, seed=None):
    g = torch.Generator(device=DEV)
    g.manual_seed(seed if seed is not None else (hash(shape) & 0xFFFF))
    return (torch.randn(*shape, generator=g, device=DEV) * scale).to(dtype)


def close(a, b, atol, rtol):
    torch.testing.assert_close(a.float(), b.float(), atol=atol, rtol=rtol)


from uniserve_v1_b200.ops.tolerance import Tolerance   # bounds derived per operator

# both sides round their result into bf16 once: one more unit round-off than a single store
BF16_STORE = Tolerance(0.0, 2.0 ** -8)


def teardown_function(_):
    torch.cuda.synchronize()
    N.raise_on_device_error()


@pytest.mark.parametrize("T,H", [(1, 256), (64, 2048), (7, 5376)])
def test_rmsnorm(T, H):
    x, w = rnd(T, H), rnd(H)
    # sum of H squares in FP32, one scale, one product, stored in bf16 on both sides
    tol = Tolerance.rounding(H, out=BF).then(BF16_STORE)
    tol.check(F.rmsnorm(x, w, 1e-6), R.rmsnorm(x, w, 1e-6), "rmsnorm")


def test_add_rmsnorm():
    x, w = rnd(33, 2048), rnd(2048)
    y0, r0 = F.add_rmsnorm(x, None, w, 1e-6)
    ye, re_ = R.add_rmsnorm(x, None, w, 1e-6)
    close(y0, ye, 2e-2, 2e-2)
    close(r0, re_, 1e-6, 1e-6)
    x2 = rnd(33, 2048, seed=5)
    y1, r1 = F.add_rmsnorm(x2, r0, w, 1e-6)
    ye1, re1 = R.add_rmsnorm(x2, re_, w, 1e-6)
    close(y1, ye1, 2e-2, 2e-2)
    close(r1, re1, 1e-5, 1e-5)


def test_modulated_rmsnorm_and_gated_residual():
    T, H = 50, 512
    x, u = rnd(T, H), rnd(T, H, seed=2)
    table = rnd(9 * 6, H, dtype=torch.float32, seed=3) * 0.1
    idx = torch.randint(0, 9, (T,), device=DEV, dtype=torch.int32)
    close(F.modulated_rmsnorm(x, None, table, idx, 6, 0, 1, 1e-6),
          R.modulated_rmsnorm(x, None, table, idx, 6, 0, 1, 1e-6), 2e-2, 2e-2)
    h = x.clone()
    F.gated_residual_(h, u, table, idx, 6, 2)
    close(h, R.gated_residual(x, u, table, idx, 6, 2), 2e-2, 2e-2)


def test_layer_norm():
    x, w, b = rnd(19, 1152), rnd(1152), rnd(1152, seed=4)
    close(F.layer_norm(x, w, b, 1e-5), R.layer_norm(x, w, b, 1e-5), 3e-2, 2e-2)


@pytest.mark.parametrize("rows,M,K", [(1, 128, 64), (16, 256, 128), (5, 384, 2048), (64, 5120, 2048),
                                       (200, 256, 512), (300, 1024, 768), (64, 1000, 264)])
def test_linear_bf16(rows, M, K):
    x, w = rnd(rows, K), rnd(M, K, scale=0.05)
    y = F.linear(x, w)
    ref = R.linear(x, w)
    # K mixed-sign products accumulated in FP32 (tensor memory), both sides stored in bf16
    Tolerance.dot(K, out=BF).then(BF16_STORE).check(y, ref, "linear")


@pytest.mark.parametrize("rows,M,K", [(64, 768, 2048), (64, 2048, 512), (33, 128, 2048),
                                       (7, 1000, 256), (16, 5120, 4096), (1, 24, 768),
                                       (64, 128, 4096), (20, 512, 1536)])
def test_linear_decode_kernel(rows, M, K, monkeypatch):
    """The weight-streaming kernel of decode-size projections (at most 64 rows, K a multiple
    of 256): bf16 and fp32 outputs, bias, a strided activation view, and the same result as
    the tcgen05 kernel it stands in for."""
    monkeypatch.setattr(F, "LINEAR_DECODE_MAX", 1 << 40)
    x, w = rnd(rows, K), rnd(M, K, scale=0.05)
    ref = x.float() @ w.float().t()
    tol = 1e-3 * math.sqrt(K / 64)            # fp32 accumulation of bf16 products
    y32 = F.linear(x, w, out_dtype=torch.float32)
    Tolerance.dot(K, out=torch.float32).check(y32, ref, "decode linear, fp32 out")
    close(y32, ref, tol, 1e-3)
    close(F.linear(x, w), ref, 2e-2 * math.sqrt(K / 64), 2e-2)
    b = rnd(M, dtype=torch.float32, seed=3)
    close(F.linear(x, w, bias=b, out_dtype=torch.float32), ref + b, tol, 1e-3)
    wide = rnd(rows, K + 64, seed=9)
    close(F.linear(wide[:, :K], w, out_dtype=torch.float32), wide[:, :K].float() @ w.float().t(),
          tol, 1e-3)
    monkeypatch.setattr(F, "LINEAR_DECODE", False)
    close(F.linear(x, w, out_dtype=torch.float32), y32, tol, 1e-3)


@pytest.mark.parametrize("rows,M,K", [(2600, 2176, 512), (4100, 1280, 192), (2304, 2048, 1024)])
def test_linear_many_tiles(rows, M, K):
    """More than one wave of tiles: the persistent kernels (CTA pairs by default; an odd
    number of 128-feature tiles leaves one CTA of the last pair without a tile)."""
    x, w = rnd(rows, K), rnd(M, K, scale=0.05)
    close(F.linear(x, w), R.linear(x, w), 2e-2 * math.sqrt(K / 64), 2e-2)
    b = rnd(M, dtype=torch.float32, seed=3)
    y = F.linear(x, w, bias=b, out_dtype=torch.float32)
    close(y, x.float() @ w.float().t() + b, 1e-2 * math.sqrt(K / 64), 5e-3)


def test_linear_gated_many_tiles():
    x, w = rnd(2700, 512), rnd(2 * 1152, 512, scale=0.05)
    close(F.linear_gated(x, w), R.linear_gated(x, w), 3e-2, 3e-2)


def test_linear_fp32_out_bias():
    x, w, b = rnd(40, 512), rnd(300, 512, scale=0.05), rnd(300, dtype=torch.float32)
    y = F.linear(x, w, bias=b, out_dtype=torch.float32)
    ref = (x.float() @ w.float().t()) + b
    close(y, ref, 5e-3, 5e-3)


@pytest.mark.parametrize("rows", [3, 64, 150])
def test_linear_gated(rows):
    x, w = rnd(rows, 1024), rnd(2 * 384, 1024, scale=0.05)
    close(F.linear_gated(x, w), R.linear_gated(x, w), 3e-2, 3e-2)
    close(F.linear_gated(x, w, stepwise=True), R.linear_gated(x, w, stepwise=True), 3e-2, 3e-2)


@pytest.mark.parametrize("T,D", [(37, 128), (700, 128), (37, 64)])
def test_qk_norm_rope_kv(T, D):
    """128-wide heads take the one-token-per-CTA kernel (heads split over CTAs for few tokens,
    whole tokens for many); other widths the one-warp-per-row kernel."""
    Hq, Hkv, page = 8, 2, 16
    qkv = rnd(T, (Hq + 2 * Hkv) * D)
    qw, kw = rnd(D), rnd(D, seed=9)
    pos = torch.randint(0, 5000, (T,), device=DEV, dtype=torch.int32)
    inv = R.rope_inv_freq(D, 1e6, DEV)
    pages = (T + page - 1) // page + 5
    slots = torch.randperm(pages * page, device=DEV)[:T].to(torch.int32)
    slots[3] = -1
    kc = torch.zeros(pages, page, Hkv, D, dtype=BF, device=DEV)
    vc = torch.zeros_like(kc)
    ref = qkv.clone().cpu()
    kc_r, vc_r = kc.clone().cpu(), vc.clone().cpu()
    F.qk_norm_rope_kv_(ref, qw.cpu(), kw.cpu(), pos.cpu(), inv.cpu(), slots.cpu(), kc_r, vc_r,
                       Hq, Hkv, D)
    F.qk_norm_rope_kv_(qkv, qw, kw, pos, inv, slots, kc, vc, Hq, Hkv, D)
    close(qkv.cpu(), ref, 3e-2, 3e-2)
    close(kc.cpu(), kc_r, 3e-2, 3e-2)
    close(vc.cpu(), vc_r, 0, 0)


def test_qk_norm_rope3():
    T, H, D, Fq = 45, 4, 128, 16
    q, k = rnd(T, H * D), rnd(T, H * D, seed=3)
    qw, kw = rnd(D), rnd(D, seed=8)
    coords = torch.rand(3, T, device=DEV) * 40
    inv = R.rope_inv_freq(2 * Fq, 10000.0, DEV)
    qr, kr = R.qk_norm_rope3(q.view(T, H, D), k.view(T, H, D), qw, kw, coords, inv, Fq, 1e-6)
    q2, k2 = q.clone(), k.clone()
    F.qk_norm_rope3_(q, k, qw, kw, coords, inv, H, H, D, Fq)
    close(q.view(T, H, D), qr, 3e-2, 3e-2)
    close(k.view(T, H, D), kr, 3e-2, 3e-2)
    # table-driven fast path (row-strided views of a wider buffer, no q/k norm weights too)
    wide = torch.cat([q2, k2, rnd(T, 64)], 1)
    qv, kv = wide[:, :H * D], wide[:, H * D:2 * H * D]
    F.qk_norm_rope3_(qv, kv, qw, kw, coords, inv, H, H, D, Fq, table=F.rope3_table(coords, inv))
    close(qv.reshape(T, H, D), qr, 3e-2, 3e-2)
    close(kv.reshape(T, H, D), kr, 3e-2, 3e-2)


@pytest.mark.parametrize("Hq,Hkv,D,splits", [(32, 4, 128, 1), (32, 4, 128, 4), (4, 2, 64, 2),
                                              (16, 1, 128, 3)])
def test_paged_decode_attention(Hq, Hkv, D, splits):
    B, page, pages = 5, 16, 200
    lens = torch.tensor([1, 17, 300, 64, 511], dtype=torch.int32, device=DEV)
    q = rnd(B, Hq, D)
    kc, vc = rnd(pages, page, Hkv, D, seed=1), rnd(pages, page, Hkv, D, seed=2)
    pt = torch.randperm(pages - 1, device=DEV)[:B * 32].view(B, 32).to(torch.int32) + 1
    out = F.paged_decode_attention(q, kc, vc, pt, lens, 1 / math.sqrt(D), splits=splits)
    ref = R.paged_decode_attention(q, kc, vc, pt, lens, 1 / math.sqrt(D))
    close(out, ref, 2e-2, 2e-2)
    # scores: D products; probabilities rounded to bf16 before the second product (so each
    # carries u_bf16, amplified by e^|score error| ~ 1 + error); output: up to 511 products,
    # a denominator of as many positive terms, stored in bf16 on both sides
    L = int(lens.max())
    tol = Tolerance.dot(D, out=torch.float32).scaled(float(q.float().abs().max() *
                                                           kc.float().abs().max() * D ** 0.5)) \
        .then(Tolerance.dot(L, out=BF, inputs=BF)).then(Tolerance.rounding(L, out=BF)) \
        .then(BF16_STORE)
    tol.check(out, ref, "paged decode attention")


def test_topk_softmax():
    T, E, k = 70, 128, 8
    logits = rnd(T, E, dtype=torch.float32)
    ids, w = F.topk_softmax(logits, k, True)
    ids_r, w_r = R.topk_softmax(logits, k, True)
    assert torch.equal(ids.cpu(), ids_r.cpu())
    close(w, w_r, 1e-5, 1e-4)
    live = torch.tensor([10], dtype=torch.int32, device=DEV)
    ids2, w2 = F.topk_softmax(logits, k, True, live=live)
    assert (ids2[10:] == -1).all() and (w2[10:] == 0).all()
    assert torch.equal(ids2[:10].cpu(), ids_r[:10].cpu())


@pytest.mark.parametrize("T,E,k,H,I", [(64, 128, 8, 2048, 768), (5, 8, 2, 256, 128),
                                        (300, 16, 4, 512, 256)])
def test_moe_experts(T, E, k, H, I):
    x = rnd(T, H)
    w13, w2 = rnd(E, 2 * I, H, scale=0.03), rnd(E, H, I, scale=0.03, seed=4)
    logits = rnd(T, E, dtype=torch.float32, seed=6)
    ids, w = F.topk_softmax(logits, k, True)
    out = F.moe_experts(x, ids, w, w13, w2)
    ref = R.moe_experts(x, ids, w, w13, w2)
    close(out, ref, 3e-2, 3e-2)
    # expert-parallel window: only experts [E/2, E) are local
    out2 = F.moe_experts(x, ids, w, w13[E // 2:].contiguous(), w2[E // 2:].contiguous(),
                         e_lo=E // 2)
    ref2 = R.moe_experts(x, ids, w, w13[E // 2:], w2[E // 2:], e_lo=E // 2)
    close(out2, ref2, 3e-2, 3e-2)


@pytest.mark.parametrize("T,E,k,H,I", [(2048, 8, 2, 512, 256), (1500, 4, 2, 1024, 384),
                                        (5001, 8, 2, 512, 256)])
def test_moe_experts_prefill_size_on_cta_pairs(T, E, k, H, I, monkeypatch):
    """A few hundred rows per expert: 256-row tiles of the sort kernel's list on the swapped
    CTA-pair kernel (gated FC1 and FC2), with uneven loads - one expert almost empty, ragged
    last tiles - against the FP32 restatement and against the single-CTA kernel.  The largest
    case has more than 8192 routes: the sort runs as a cluster of CTAs."""
    x = rnd(T, H)
    w13, w2 = rnd(E, 2 * I, H, scale=0.03), rnd(E, H, I, scale=0.03, seed=4)
    logits = rnd(T, E, dtype=torch.float32, seed=6)
    logits[:, 1] -= 6.0                                  # expert 1 gets very few rows
    logits[:, 0] += 1.0
    ids, w = F.topk_softmax(logits, k, True)
    ws = F.MoeWorkspace.create(T, k, E, H, I, DEV)
    assert ws.block_n == 256
    out = F.moe_experts(x, ids, w, w13, w2, ws=ws)
    ref = R.moe_experts(x, ids, w, w13, w2)
    close(out, ref, 3e-2, 3e-2)
    monkeypatch.setattr(F, "MOE_PAIR_MIN_ROWS", 1 << 30)
    ws1 = F.MoeWorkspace.create(T, k, E, H, I, DEV)
    assert ws1.block_n == 128
    out1 = F.moe_experts(x, ids, w, w13, w2, ws=ws1)
    close(out, out1, 2e-2, 2e-2)
    # expert-parallel window
    ws2 = F.MoeWorkspace.create(T, k, E // 2, H, I, DEV, block_n=256)
    out2 = F.moe_experts(x, ids, w, w13[E // 2:].contiguous(), w2[E // 2:].contiguous(),
                         e_lo=E // 2, ws=ws2)
    close(out2, R.moe_experts(x, ids, w, w13[E // 2:], w2[E // 2:], e_lo=E // 2), 3e-2, 3e-2)


def test_argmax_and_logprob_stats():
    logits = rnd(9, 151936, dtype=torch.float32)
    am = F.argmax(logits)
    assert torch.equal(am.cpu(), R.argmax(logits).cpu())
    lse, lp, rank = F.logprob_stats(logits, am)
    lse_r, lp_r, rank_r = R.logprob_stats(logits, am)
    close(lse, lse_r, 1e-3, 1e-4)
    close(lp, lp_r, 1e-3, 1e-4)
    assert torch.equal(rank.cpu(), rank_r.cpu())


def test_sample_from_logits_matches_reference_rule():
    B, V = 12, 4096
    logits = rnd(B, V, dtype=torch.float32, scale=3.0)
    top_k = torch.tensor([0, 1, 20, 50, 0, 0, 20, 5, 0, 100, 3, 0], dtype=torch.int32, device=DEV)
    top_p = torch.tensor([1, 1, 1, .9, .5, .95, .95, 1, .1, .8, 1, 1], dtype=torch.float32, device=DEV)
    min_p = torch.tensor([0, 0, 0, 0, 0, 0, .05, 0, 0, 0, 0, .2], dtype=torch.float32, device=DEV)
    seeds = torch.arange(B, dtype=torch.int64, device=DEV) + 1234
    pos = torch.arange(B, dtype=torch.int64, device=DEV) * 7 + 3
    out = F.sample_from_logits(logits, top_k, top_p, min_p, seeds, pos)
    ref = R.sample_from_logits(logits.cpu(), top_k.cpu(), top_p.cpu(), min_p.cpu(), seeds.cpu(),
                               pos.cpu())
    assert torch.equal(out.cpu(), ref), (out.cpu(), ref)
    # same (seed, position, distribution) -> same token, whatever the batch
    out1 = F.sample_from_logits(logits[5:6].contiguous(), top_k[5:6], top_p[5:6], min_p[5:6],
                                seeds[5:6], pos[5:6])
    assert int(out1[0]) == int(out[5])


def test_sampler_distribution():
    V, n = 64, 4000
    base = rnd(1, V, dtype=torch.float32, scale=1.5)
    logits = base.expand(n, V).contiguous()
    seeds = torch.full((n,), 77, dtype=torch.int64, device=DEV)
    pos = torch.arange(n, dtype=torch.int64, device=DEV)
    out = F.sample_from_logits(logits, None, None, None, seeds, pos)
    freq = torch.bincount(out.long(), minlength=V).float() / n
    p = base[0].softmax(-1)
    assert (freq - p).abs().max() < 0.03


def test_logits_shape():
    B, V = 4, 1000
    logits = rnd(B, V, dtype=torch.float32)
    counts = torch.randint(0, 3, (B, V), device=DEV).to(torch.int16)
    pm = (torch.rand(B, V, device=DEV) < 0.1).to(torch.uint8)
    ban = (torch.rand(B, V, device=DEV) < 0.05).to(torch.uint8)
    rep = torch.tensor([1.0, 1.3, 1.1, 1.0], device=DEV)
    fr = torch.tensor([0.0, 0.5, 0.0, 0.2], device=DEV)
    pr = torch.tensor([0.3, 0.0, 0.0, 0.2], device=DEV)
    temp = torch.tensor([1.0, 0.7, 0.0, 2.0], device=DEV)
    bo = torch.tensor([0, 2, 2, 3, 3], dtype=torch.int32, device=DEV)
    bi = torch.tensor([5, 9, 700], dtype=torch.int32, device=DEV)
    bv = torch.tensor([2.0, -1.0, 5.0], device=DEV)
    ref = R.logits_shape(logits, ban, [[(5, 2.0), (9, -1.0)], [], [(700, 5.0)], []], counts, pm,
                         rep, fr, pr, temp)
    out = F.logits_shape_(logits.clone(), ban, (bo, bi, bv), counts, pm, rep, fr, pr, temp)
    close(out, ref, 1e-5, 1e-5)


def test_embedding_gather_advance():
    table = rnd(1000, 256)
    ids = torch.randint(0, 1000, (33,), device=DEV, dtype=torch.int32)
    close(F.embedding(ids, table), table[ids.long()], 0, 0)
    out = F.embedding(ids, table[100:600].contiguous(), 100, 600)
    ok = (ids >= 100) & (ids < 600)
    close(out[ok], table[ids[ok].long()], 0, 0)
    assert (out[~ok] == 0).all()
    idx = torch.tensor([3, -1, 7], dtype=torch.int32, device=DEV)
    g = F.gather_rows(table, idx)
    close(g[0], table[3], 0, 0)
    assert (g[1] == 0).all()


def test_peer_wait_that_runs_out_sets_the_status_and_later_waits_give_up():
    """A wait on a peer flag that nothing ever writes: with the budget set to a few
    milliseconds the kernel returns, the status word reads "peer flag timeout", the next fused
    launch gives up at once (its wait budget is zero while the word is set), the host check
    raises, and after the word is cleared and the heap reset a clean launch passes.  The
    silent peer is a second allocation of this process (a loopback heap of two ranks): no
    GPU waits for longer than the budget and nothing faults."""
    import time
    from uniserve_v1_b200.parallel.symm import FusedComm, set_peer_wait_clocks
    assert N.read_status() == 0
    T, H = 8, 512
    w = torch.ones(H, dtype=BF, device=DEV)
    part = rnd(T, H, seed=90)
    set_peer_wait_clocks(6_000_000)                    # about 3 ms at 1.9 GHz
    lone = FusedComm(None, 0, 2, DEV, H, sites=4, loopback=True)
    try:
        t0 = time.perf_counter()
        lone.allreduce_add_rmsnorm(part, None, w, 1e-6)
        torch.cuda.synchronize()
        first = time.perf_counter() - t0
        assert first < 1.0                             # bounded by the budget, not by 1.5 s
        t0 = time.perf_counter()
        for _ in range(20):                            # every later wait gives up at once
            lone.allreduce_add_rmsnorm(part, None, w, 1e-6)
        lone.barrier(lone.SITE_AUX)
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 0.5
        with pytest.raises(RuntimeError, match="peer flag"):
            N.raise_on_device_error()
        assert N.read_status() == 0                    # the read cleared it
        # the serving path's form: the word copied behind the results, checked without a
        # synchronisation of its own, and cleared for whoever runs next
        from uniserve_v1_b200.engine.runner import DeviceStepError
        host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        lone.allreduce_add_rmsnorm(part, None, w, 1e-6)
        N.kernels().us_status_copy_async(N.ptr(host), N.stream())
        torch.cuda.synchronize()
        assert int(host[0]) == 0x400
        with pytest.raises(DeviceStepError):
            raise DeviceStepError(int(host[0]))
        N.kernels().us_status_clear_async(N.stream())
        torch.cuda.synchronize()
        assert N.read_status() == 0
    finally:
        lone.close()
        set_peer_wait_clocks(0)
    # a clean launch after the failure: one rank, nothing to wait for
    solo = FusedComm(None, 0, 1, DEV, H, sites=4)
    try:
        y, res = solo.allreduce_add_rmsnorm(part, None, w, 1e-6)
        ye, re_ = R.add_rmsnorm(part, None, w, 1e-6)
        torch.cuda.synchronize()
        close(y, ye, 2e-2, 2e-2)
        close(res, re_, 1e-6, 1e-6)
        solo.reset()
        y2, _ = solo.allreduce_add_rmsnorm(part, None, w, 1e-6)
        close(y2, ye, 2e-2, 2e-2)
        lg = rnd(5, 3000, dtype=torch.float32, seed=91)
        assert torch.equal(solo.argmax(lg, 2900, 0).long(), lg[:, :2900].argmax(-1))
    finally:
        solo.close()
    assert N.read_status() == 0


@pytest.mark.parametrize("T,E,k,H", [(64, 128, 8, 2048), (5, 16, 4, 256), (300, 128, 8, 512)])
def test_route_sort_gather_and_unpermute_norm_equal_the_separate_kernels(T, E, k, H):
    """One launch for routing + route sort + row gather, and the un-permute folded into the
    residual add + RMSNorm: same ids, weights, expert outputs and norm as the separate
    kernels; run twice (the grid-wide counters put themselves back)."""
    I = 128
    logits = rnd(T, E, dtype=torch.float32, seed=31)
    x = rnd(T, H, seed=32)
    w13, w2 = rnd(E // 2, 2 * I, H, scale=0.05, seed=33), rnd(E // 2, H, I, scale=0.05, seed=34)
    nw = rnd(H, seed=35)
    res0 = rnd(T, H, dtype=torch.float32, seed=36)
    ids0, w0 = F.topk_softmax(logits, k, True)
    plain = F.moe_experts(x, ids0, w0, w13, w2, e_lo=E // 2)
    y_ref, r_ref = F.add_rmsnorm(plain, res0.clone(), nw, 1e-6)
    ws = F.MoeWorkspace.create(T, k, E // 2, H, I, DEV)
    for _ in range(2):
        ids1, w1 = F.route_sort_gather(logits, x, k, True, ws, E // 2, E // 2)
        assert torch.equal(ids0, ids1) and torch.equal(w0, w1)
        y_perm, perm = F.moe_experts(x, ids1, w1, w13, w2, e_lo=E // 2, ws=ws, pregathered=True,
                                     defer_unpermute=True)
        y, r = F.unpermute_add_rmsnorm(y_perm, perm, w1, res0.clone(), nw, 1e-6)
        close(r, r_ref, 1e-5, 1e-5)
        close(y, y_ref, 2e-2, 2e-2)
    assert int(ws.sync.sum()) == 0
    live = torch.tensor([max(1, T - 3)], dtype=torch.int32, device=DEV)
    ids2, _ = F.route_sort_gather(logits, x, k, True, ws, E // 2, E // 2, live=live)
    assert (ids2[int(live):] == -1).all() and torch.equal(ids2[:int(live)], ids0[:int(live)])


@pytest.mark.parametrize("Hq,Hkv,lens", [
    (32, 4, [1, 17, 300, 64, 511]),                 # 20 pairs of 1 - 4 tiles: fewer tiles than CTAs
    (16, 16, [1100] * 24 + [0, 5]),                 # 9 tiles per pair, a sequence without keys
    (16, 1, [4000, 3, 129, 2050]),                  # pairs cut into many ranges
    (8, 8, [130] * 200),                            # 1600 pairs of 2 tiles: several pairs per range
])
def test_paged_decode_attention_persistent_kernel(Hq, Hkv, lens):
    """One CTA per SM over the tile list of the whole launch: pairs inside a range are written
    directly, pairs cut by a range boundary meet through their arrival counter.  Run twice on
    the same scratch (the counters put themselves back)."""
    B, page, D = len(lens), 16, 128
    per = (max(lens) + page - 1) // page + 1
    pages = B * per + 1
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    q = rnd(B, Hq, D)
    kc, vc = rnd(pages, page, Hkv, D, seed=1), rnd(pages, page, Hkv, D, seed=2)
    pt = (torch.randperm(pages - 1, device=DEV)[:B * per].view(B, per) + 1).to(torch.int32)
    ref = R.paged_decode_attention(q, kc, vc, pt, sl, 1 / math.sqrt(D))
    scratch, counters = F.decode_persist_scratch(B, Hkv, DEV)
    for _ in range(2):
        out = F.paged_decode_attention(q, kc, vc, pt, sl, 1 / math.sqrt(D), F.PERSIST_SPLITS,
                                       scratch=scratch, counters=counters)
        live = sl > 0
        close(out[live], ref[live], 2e-2, 2e-2)
        assert float(out[~live].float().abs().max()) == 0.0 if bool((~live).any()) else True
        assert int(counters.abs().sum()) == 0
    assert N.read_status() == 0


@pytest.mark.parametrize("Hq,Hkv,splits", [(32, 4, 4), (16, 1, 3), (8, 1, 8)])
def test_paged_decode_attention_merges_its_splits_in_the_kernel(Hq, Hkv, splits):
    B, page, pages, D = 5, 16, 200, 128
    lens = torch.tensor([1, 17, 300, 64, 511], dtype=torch.int32, device=DEV)
    q = rnd(B, Hq, D)
    kc, vc = rnd(pages, page, Hkv, D, seed=1), rnd(pages, page, Hkv, D, seed=2)
    pt = torch.randperm(pages - 1, device=DEV)[:B * 32].view(B, 32).to(torch.int32) + 1
    scratch, counters = F.decode_scratch(B, Hq, Hkv, D, splits, DEV)
    ref = R.paged_decode_attention(q, kc, vc, pt, lens, 1 / math.sqrt(D))
    two = F.paged_decode_attention(q, kc, vc, pt, lens, 1 / math.sqrt(D), splits=splits)
    for _ in range(3):                                  # the counters return to zero
        out = F.paged_decode_attention(q, kc, vc, pt, lens, 1 / math.sqrt(D), splits=splits,
                                       scratch=scratch, counters=counters)
        close(out, ref, 2e-2, 2e-2)
        close(out, two, 1e-3, 1e-3)
    assert int(counters.sum()) == 0


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("Hq,Hkv", [(4, 4), (8, 2)])
def test_flash_attn_varlen(causal, Hq, Hkv):
    from uniserve_v1_b200.ops.flash import flash_attn_varlen
    D = 128
    q_lens = [1, 130, 257, 64, 500]
    k_lens = q_lens if not causal else [7, 130, 300, 64, 777]   # keys already cached in front
    if not causal:
        k_lens = [33, 130, 200, 640, 500]
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    cu_k = torch.tensor([0] + list(torch.tensor(k_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    Tq, Tk = sum(q_lens), sum(k_lens)
    # q, k, v as column slices of one wider buffer (row-strided views)
    buf = rnd(max(Tq, Tk), (Hq + 2 * Hkv) * D)
    q = buf[:Tq, :Hq * D].view(Tq, Hq, D)
    k = buf[:Tk, Hq * D:(Hq + Hkv) * D].view(Tk, Hkv, D)
    v = buf[:Tk, (Hq + Hkv) * D:].view(Tk, Hkv, D)
    scale = 1 / math.sqrt(D)
    out = flash_attn_varlen(q, k, v, cu_q, cu_k, max(q_lens), max(k_lens), scale, causal)
    ref = R.varlen_attention(q, k, v, cu_q.cpu(), cu_k.cpu(), scale, causal)
    close(out, ref, 2e-2, 2e-2)


def test_flash_attn_long_sequence():
    from uniserve_v1_b200.ops.flash import flash_attn_varlen
    D, H, T = 128, 2, 4096 + 77
    q, k, v = rnd(T, H, D, seed=1), rnd(T, H, D, seed=2), rnd(T, H, D, seed=3)
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    out = flash_attn_varlen(q, k, v, cu, cu, T, T, 1 / math.sqrt(D), False)
    ref = R.varlen_attention(q, k, v, cu.cpu(), cu.cpu(), 1 / math.sqrt(D), False)
    close(out, ref, 2e-2, 2e-2)


def test_flash_attn_last_partial_wave_split_over_the_keys():
    """12 query pairs x 13 heads are 156 (pair, head) items: one wave of 148 CTAs and 8 more,
    which the launch splits over the keys (6 parts of 4 key blocks), leaves unnormalised with
    their maxima and sums, and merges; K and V lengths differ from Q and are ragged."""
    from uniserve_v1_b200.ops.flash import flash_attn_varlen
    D, H, Tq, Tk = 128, 13, 3072 - 5, 3072 - 37
    q, k, v = rnd(Tq, H, D, seed=1), rnd(Tk, H, D, seed=2), rnd(Tk, H, D, seed=3)
    cu_q = torch.tensor([0, Tq], dtype=torch.int32, device=DEV)
    cu_k = torch.tensor([0, Tk], dtype=torch.int32, device=DEV)
    out = flash_attn_varlen(q, k, v, cu_q, cu_k, Tq, Tk, 1 / math.sqrt(D), False)
    ref = R.varlen_attention(q, k, v, cu_q.cpu(), cu_k.cpu(), 1 / math.sqrt(D), False)
    close(out, ref, 2e-2, 2e-2)
    assert N.read_status() == 0


def test_flash_attn_push_with_a_split_last_wave_equals_the_plain_kernel():
    """The sequence-parallel return (rows stored into their owners' buffers from the epilogue,
    here two buffers of this GPU) on a shape whose last wave is split over the keys: the merge
    kernel does the owner mapping for those rows."""
    import ctypes
    from uniserve_v1_b200.ops.flash import flash_attn_varlen
    from uniserve_v1_b200.parallel import ulysses  # registers the entry point's signature
    D, H, T, P = 128, 13, 3072, 2
    q, k, v = rnd(T, H, D, seed=4), rnd(T, H, D, seed=5), rnd(T, H, D, seed=6)
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    ref = flash_attn_varlen(q, k, v, cu, cu, T, T, 1 / math.sqrt(D), False)
    ro, inner = T // P, 2 * H * D                      # this rank's heads are columns [H*D, 2*H*D)
    bufs = [torch.zeros(ro, inner, dtype=BF, device=DEV) for _ in range(P)]
    ptrs = (ctypes.c_void_p * P)(*[b.data_ptr() for b in bufs])
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    N.call("us_flash_attn_push", N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(cu), N.ptr(cu), T, T, H, H,
           q.stride(0), k.stride(0), v.stride(0), 1 / math.sqrt(D), ptrs, P, ro, H * D, inner, st)
    torch.cuda.synchronize()
    got = torch.cat([b[:, H * D:] for b in bufs], 0).view(T, H, D)
    assert torch.equal(got, ref)
    assert all(float(b[:, :H * D].abs().max()) == 0.0 for b in bufs)
    assert N.read_status() == 0


@pytest.mark.parametrize("single", [True, False])
@pytest.mark.parametrize("causal", [False, True])
def test_flash_attn_both_kernels(single, causal, monkeypatch):
    """The single-tile kernel and the two-tile ping-pong kernel on the same input:
    causal self-attention (the first tile of a pair walks fewer key blocks than
    the second) and a ragged tail (the second tile of the last pair is partial)."""
    import uniserve_v1_b200.ops.flash as FL
    monkeypatch.setattr(FL, "_SINGLE_TILE_ONLY", single)
    D, H = 128, 3
    lens = [1000, 129, 384]
    T = sum(lens)
    q, k, v = rnd(T, H, D, seed=11), rnd(T, H, D, seed=12), rnd(T, H, D, seed=13)
    cu = torch.tensor([0, 1000, 1129, 1513], dtype=torch.int32, device=DEV)
    out = FL.flash_attn_varlen(q, k, v, cu, cu, max(lens), max(lens), 1 / math.sqrt(D), causal)
    ref = R.varlen_attention(q, k, v, cu.cpu(), cu.cpu(), 1 / math.sqrt(D), causal)
    close(out, ref, 2e-2, 2e-2)


def test_fence_probes_stamp_the_stream_in_order():
    from uniserve_v1_b200.engine.profiling import ProbeRing
    ring = ProbeRing(16, DEV)
    x = rnd(4096, 4096)
    ring.mark("work.begin", 7)
    y = F.linear(x, x)
    ring.mark("work.end", 7)
    rows = ring.collect()
    assert [r[0] for r in rows] == ["work.begin", "work.end"]
    assert rows[1][1] > rows[0][1] > 0 and rows[0][3] == 7
    assert (rows[1][1] - rows[0][1]) < 1e9          # a sub-second GEMM
    assert ring.collect() == [] and y.shape == (4096, 4096)


@pytest.mark.parametrize("T,E,k", [(64, 128, 8), (5, 16, 4), (300, 128, 8)])
def test_route_and_sort_equals_the_two_kernels(T, E, k):
    H, I = 256, 128
    logits = rnd(T, E, dtype=torch.float32, seed=21)
    ids0, w0 = F.topk_softmax(logits, k, True)
    ws = F.MoeWorkspace.create(T, k, E // 2, H, I, DEV)
    ids1, w1 = F.route_and_sort(logits, k, True, ws, E // 2, E // 2)
    assert torch.equal(ids0, ids1) and torch.equal(w0, w1)
    x = rnd(T, H, seed=22)
    w13, w2 = rnd(E // 2, 2 * I, H, scale=0.05, seed=23), rnd(E // 2, H, I, scale=0.05, seed=24)
    a = F.moe_experts(x, ids0, w0, w13, w2, e_lo=E // 2)
    b = F.moe_experts(x, ids1, w1, w13, w2, e_lo=E // 2, ws=ws, presorted=True)
    close(a, b, 1e-3, 1e-3)


def _ptr_array(tensors):
    import ctypes
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def test_gemm_peer_modes_with_local_buffers_as_peers():
    """The four peer modes of the GEMM (operand tiles pulled from per-rank K slices or
    per-rank row intervals; output tiles scattered by feature or reduce-scattered by row)
    with local tensors standing in for the peers' buffers."""
    from uniserve_v1_b200.parallel import tp_fused, ulysses  # noqa: F401  (register signatures)
    rows, K, M, P = 320, 512, 384, 2
    x, w = rnd(rows, K, seed=31), rnd(M, K, scale=0.05, seed=32)
    ref = x.float() @ w.float().t()
    st = N.stream()
    # pull: K is the concatenation of two peers' [rows, K / 2] buffers
    parts = [x[:, :K // 2].contiguous(), x[:, K // 2:].contiguous()]
    out = torch.empty(rows, M, dtype=BF, device=DEV)
    N.call("us_gemm_wx_pull", N.ptr(w), _ptr_array(parts), P, K // 2, N.ptr(out), M, K, rows, K,
           K // 2, M, 0, 64, st)
    close(out, ref, 3e-2, 3e-2)
    # gather: the rows are the concatenation of two peers' [rows / 2, K] buffers
    halves = [x[:rows // 2].contiguous(), x[rows // 2:].contiguous()]
    out2 = torch.empty(rows, M, dtype=BF, device=DEV)
    N.call("us_gemm_wx_gather", N.ptr(w), _ptr_array(halves), P, rows // 2, N.ptr(out2), M, M, K,
           rows, K, K, M, 0, 0, 0, 0, 32, st)
    close(out2, ref, 3e-2, 3e-2)
    # scatter: features [p * M / 2, ...) go to peer p at row offset 16
    wide = rnd(256, K, scale=0.05, seed=33)            # 2 x 128 features
    dst = [torch.zeros(rows + 16, 128, dtype=BF, device=DEV) for _ in range(P)]
    N.call("us_gemm_wx_scatter", N.ptr(wide), N.ptr(x), 256, K, rows, K, K, 128, _ptr_array(dst),
           128, 16, 64, st)
    refw = x.float() @ wide.float().t()
    for p_ in range(P):
        close(dst[p_][16:], refw[:, p_ * 128:(p_ + 1) * 128], 3e-2, 3e-2)
        assert float(dst[p_][:16].abs().max()) == 0.0
    # reduce-scatter: rows [p * rows / 2, ...) go to peer p, slot 1 of 2
    slots = [torch.zeros(2, rows // 2, M, dtype=BF, device=DEV) for _ in range(P)]
    N.call("us_gemm_wx_reduce_scatter", N.ptr(w), N.ptr(x), M, K, rows, K, K, M,
           _ptr_array(slots), P, rows // 2, 1, 0, 32, st)
    for p_ in range(P):
        close(slots[p_][1], ref[p_ * (rows // 2):(p_ + 1) * (rows // 2)], 3e-2, 3e-2)
        assert float(slots[p_][0].abs().max()) == 0.0


def test_gemm_output_modes_many_tiles():
    """Scatter by feature block, reduce-scatter by row interval and the row-mapped output on
    problems of more than one wave of tiles (the CTA-pair kernel, one activation row per
    epilogue thread), local tensors standing in for the peers' buffers."""
    from uniserve_v1_b200.parallel import tp_fused, ulysses  # noqa: F401  (register signatures)
    rows, K, P = 2500, 256, 2
    x = rnd(rows, K, seed=41)
    st = N.stream()
    wide = rnd(2048, K, scale=0.05, seed=42)           # 2 x 1024 features
    dst = [torch.zeros(rows + 8, 1024, dtype=BF, device=DEV) for _ in range(P)]
    N.call("us_gemm_wx_scatter", N.ptr(wide), N.ptr(x), 2048, K, rows, K, K, 1024, _ptr_array(dst),
           1024, 8, 256, st)
    refw = x.float() @ wide.float().t()
    for p_ in range(P):
        close(dst[p_][8:], refw[:, p_ * 1024:(p_ + 1) * 1024], 3e-2, 3e-2)
        assert float(dst[p_][:8].abs().max()) == 0.0
    rows2, M = 2560, 2048
    x2, w = rnd(rows2, K, seed=43), rnd(M, K, scale=0.05, seed=44)
    ref = x2.float() @ w.float().t()
    slots = [torch.zeros(2, rows2 // 2, M, dtype=BF, device=DEV) for _ in range(P)]
    N.call("us_gemm_wx_reduce_scatter", N.ptr(w), N.ptr(x2), M, K, rows2, K, K, M,
           _ptr_array(slots), P, rows2 // 2, 1, 0, 256, st)
    for p_ in range(P):
        close(slots[p_][1], ref[p_ * (rows2 // 2):(p_ + 1) * (rows2 // 2)], 3e-2, 3e-2)
        assert float(slots[p_][0].abs().max()) == 0.0


@pytest.mark.parametrize("causal", [False, True])
def test_flash_attn_head_dim_64(causal):
    """64-wide heads on the two-tile kernel (row-strided q / k / v views, GQA 2:1)."""
    from uniserve_v1_b200.ops.flash import flash_attn_varlen
    D, Hq, Hkv = 64, 4, 2
    lens = [300, 70, 513]
    T = sum(lens)
    buf = rnd(T, (Hq + 2 * Hkv) * D, seed=51)
    q = buf[:, :Hq * D].view(T, Hq, D)
    k = buf[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
    v = buf[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    cu = torch.tensor([0, 300, 370, 883], dtype=torch.int32, device=DEV)
    out = flash_attn_varlen(q, k, v, cu, cu, max(lens), max(lens), 1 / math.sqrt(D), causal)
    ref = R.varlen_attention(q, k, v, cu.cpu(), cu.cpu(), 1 / math.sqrt(D), causal)
    close(out, ref, 2e-2, 2e-2)


def test_flash_attn_head_dim_96():
    """96-wide heads (the text refiner's) run on the tensor-core kernel, zero-padded to 128
    channels; a width the kernels do not serve is refused, not computed elsewhere."""
    from uniserve_v1_b200.ops.flash import flash_attn_varlen
    D, H = 96, 3
    lens = [200, 57]
    T = sum(lens)
    q, k, v = rnd(T, H, D, seed=61), rnd(T, H, D, seed=62), rnd(T, H, D, seed=63)
    cu = torch.tensor([0, 200, 257], dtype=torch.int32, device=DEV)
    out = flash_attn_varlen(q, k, v, cu, cu, max(lens), max(lens), 1 / math.sqrt(D), False)
    ref = R.varlen_attention(q, k, v, cu.cpu(), cu.cpu(), 1 / math.sqrt(D), False)
    assert out.shape == (T, H, D)
    close(out, ref, 2e-2, 2e-2)
    with pytest.raises(ValueError):
        flash_attn_varlen(rnd(T, H, 100), rnd(T, H, 100), rnd(T, H, 100), cu, cu, 200, 200, 0.1,
                          False)


# ------------------------------------------------- recurrent token mixers --
@pytest.mark.parametrize("dtype", [BF, torch.float32])
def test_causal_conv1d_packed_batch_and_state(dtype):
    """Three packed sequences (one shorter than the filter) against the FP32 restatement run
    per sequence, outputs and carried state, then a second call that continues from the state."""
    from uniserve_v1_b200.ops import gated_delta as GD
    C, K = 640, 4
    lens = [37, 2, 9]
    w = rnd(C, K, scale=0.5, dtype=dtype)
    pool = rnd(5, K - 1, C, dtype=dtype, seed=3)
    slots = torch.tensor([4, 0, 2], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, 37, 39, 48], dtype=torch.int32, device=DEV)
    wide = rnd(sum(lens), C + 64, dtype=dtype, seed=4)
    x = wide[:, 32:32 + C]                                   # a strided view, as in the model
    before = pool.clone()
    y, _ = GD.causal_conv1d(x, w, pool, cu=cu, slots=slots)
    # K products in FP32, silu, one store: a rounding bound (terms can cancel: relative to max)
    tol = Tolerance.dot(K, out=dtype).then(Tolerance(0.0, 2.0 ** -20, True))
    lo = 0
    for n, s in zip(lens, slots.tolist()):
        ref_y, ref_state = GD.causal_conv1d(x[lo:lo + n].cpu().float(), w.cpu().float(),
                                            before[s].cpu().float())
        tol.check(y[lo:lo + n], ref_y, "causal_conv1d")
        Tolerance.exact().check(pool[s], ref_state.to(dtype), "causal_conv1d state")
        lo += n
    Tolerance.exact().check(pool[1], before[1], "untouched slot")
    # the single-sequence form returns a new state and leaves the caller's alone
    st = before[0].clone()
    y1, st1 = GD.causal_conv1d(x[:5].contiguous(), w, st)
    ref_y, ref_state = GD.causal_conv1d(x[:5].cpu().float(), w.cpu().float(), before[0].cpu().float())
    tol.check(y1, ref_y, "causal_conv1d single")
    Tolerance.exact().check(st, before[0], "caller's state")
    Tolerance.exact().check(st1, ref_state.to(dtype), "returned state")


@pytest.mark.parametrize("Dk,Dv,Hk,Hv,dtype", [(128, 128, 4, 8, BF), (16, 16, 2, 4, torch.float32),
                                               (64, 96, 2, 2, BF)])
def test_gated_delta_rule_kernel(Dk, Dv, Hk, Hv, dtype):
    """Packed sequences (lengths across the 16-token staging boundary, and a decode-size one)
    against the step-by-step FP32 recurrence; gates given and gates formed in the kernel."""
    from uniserve_v1_b200.ops import gated_delta as GD
    lens = [37, 1, 16]
    T = sum(lens)
    q, k, v = rnd(T, Hk, Dk, dtype=dtype, seed=1), rnd(T, Hk, Dk, dtype=dtype, seed=2), \
        rnd(T, Hv, Dv, dtype=dtype, seed=3)
    a_raw, b_raw = rnd(T, Hv, dtype=dtype, seed=4), rnd(T, Hv, dtype=dtype, seed=5)
    A = -(torch.rand(Hv, device=DEV) * 2 + 0.2)
    dt_bias = torch.rand(Hv, device=DEV)
    g = A * torch.nn.functional.softplus(a_raw.float() + dt_bias)
    beta = torch.sigmoid(b_raw.float())
    pool0 = rnd(4, Hv, Dk, Dv, dtype=torch.float32, scale=0.1, seed=6)
    slots = torch.tensor([2, 0, 3], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, 37, 38, 54], dtype=torch.int32, device=DEV)
    rep = Hv // Hk
    # per token two Dk-long FP32 dots whose error feeds the next token; fast exp / rsqrt
    # intrinsics add about 2^-21 per use
    tol = Tolerance.dot(Dk, out=torch.float32).then(Tolerance(0.0, 2.0 ** -19, True)).scaled(max(lens))
    for mode in ("given", "raw"):
        pool = pool0.clone()
        if mode == "given":
            out = GD.gated_delta_rule_packed(q, k, v, pool, cu, slots, g=g.contiguous(),
                                             beta=beta.contiguous())
        else:
            out = GD.gated_delta_rule_packed(q, k, v, pool, cu, slots, raw=(a_raw, b_raw, A, dt_bias))
        lo = 0
        for n, s in zip(lens, slots.tolist()):
            sl = slice(lo, lo + n)
            ref_o, ref_S = GD.gated_delta_rule_steps(
                q[sl].cpu().repeat_interleave(rep, 1), k[sl].cpu().repeat_interleave(rep, 1),
                v[sl].cpu(), g[sl].cpu(), beta[sl].cpu(), pool0[s].cpu())
            tol.check(out[sl], ref_o, f"gated delta rule output ({mode})")
            tol.check(pool[s], ref_S, f"gated delta rule state ({mode})")
            lo += n
        Tolerance.exact().check(pool[1], pool0[1], "untouched slot")
    # the dispatching entry point (one sequence, expanded heads) takes the kernel on a GPU
    qe, ke = q[:37].repeat_interleave(rep, 1), k[:37].repeat_interleave(rep, 1)
    o2, S2 = GD.gated_delta_rule(qe, ke, v[:37], g[:37], beta[:37], pool0[2])
    ref_o, ref_S = GD.gated_delta_rule_chunked(qe.cpu(), ke.cpu(), v[:37].cpu(), g[:37].cpu(),
                                               beta[:37].cpu(), pool0[2].cpu())
    tol.check(o2, ref_o, "gated delta rule vs the chunked form")
    tol.check(S2, ref_S, "state vs the chunked form")


def test_rmsnorm_gated_kernel():
    from uniserve_v1_b200.ops import gated_delta as GD
    T, Hv, Dv = 19, 8, 128
    x = rnd(T, Hv, Dv, dtype=torch.float32, seed=1)
    w = rnd(Dv, seed=2)
    wide = rnd(T, Hv * Dv + 32, seed=3)
    z = wide[:, 16:16 + Hv * Dv].unflatten(1, (Hv, Dv))
    y = GD.rmsnorm_gated(x, w, z, 1e-6)
    assert y.dtype == BF
    ref = GD.rmsnorm_gated(x.cpu().to(BF), w.cpu(), z.cpu(), 1e-6)
    # both round x to bf16 first, the normalised value and its product with w once each
    Tolerance.rounding(Dv, out=BF).then(BF16_STORE).then(BF16_STORE).check(y, ref, "rmsnorm_gated")


def test_hybrid_model_on_the_kernels_matches_restatement():
    """The Qwen3.5-style hybrid model with its linear-attention layers on the recurrent
    kernels against the same bf16 model with those layers on the PyTorch restatement: logits
    of a prompt run in chunks and the recurrent state after it."""
    from uniserve_v1_b200.models.qwen3_5 import Qwen35MoeModel
    from uniserve_v1_b200.ops import gated_delta as GD
    cfg = Qwen35MoeModel.tiny_config()
    model = Qwen35MoeModel(cfg, DEV, BF).init_random(seed=0)
    prompt = torch.tensor([(7 * i + 3) % cfg.vocab_size for i in range(45)], device=DEV)
    runs = {}
    for use in (True, False):
        GD.USE_KERNELS = use
        try:
            st = model.new_state()
            runs[use] = ([model.forward(prompt[lo:lo + 20], st, lo) for lo in (0, 20, 40)], st)
        finally:
            GD.USE_KERNELS = True
    for a, b in zip(runs[True][0], runs[False][0]):
        cos = torch.nn.functional.cosine_similarity(a.float(), b.float(), dim=-1)
        assert float(cos.min()) > 0.995, f"cosine {float(cos.min()):.4f}"
    for i, (a, b) in enumerate(zip(runs[True][1], runs[False][1])):
        if a.rule is not None:
            rel = (a.rule - b.rule).norm() / b.rule.norm()
            assert float(rel) < 0.02, f"layer {i}: recurrent state off by {float(rel):.3f}"


# ----------------------------------------------------------- FP8 KV pages --
def test_kv_write_scaled_matches_the_page_rule():
    """The scaled page write against its CPU restatement through a prefill-sized launch (runs
    of rows per page, a skipped row) and two decode-sized appends, one of which grows a
    page's scale and re-encodes it."""
    page, Hkv, D, pages = 16, 4, 128, 12
    kc = torch.zeros(pages, page, Hkv, D, dtype=torch.uint8, device=DEV)
    vc = torch.zeros_like(kc)
    ks = torch.zeros(pages, dtype=torch.float32, device=DEV)
    vs = torch.zeros_like(ks)
    ref = [t.cpu().clone() for t in (kc, vc, ks, vs)]
    # two sequences: pages (3, 7, 1) rows 0..36 and pages (5,) rows 0..8; one skipped row
    slots = [3 * page + i for i in range(16)] + [7 * page + i for i in range(16)] + \
        [1 * page + i for i in range(5)] + [-1] + [5 * page + i for i in range(9)]
    steps = [(slots, 1.0), ([1 * page + 5, 5 * page + 9], 0.3), ([1 * page + 6, 5 * page + 10], 6.0)]
    for n, (sl, mag) in enumerate(steps):
        T = len(sl)
        wide = rnd(T, (8 + 2 * Hkv) * D, scale=mag, seed=10 + n)
        v3 = wide.view(T, 8 + 2 * Hkv, D)
        k, v = v3[:, 8:8 + Hkv], v3[:, 8 + Hkv:]                 # views of a fused projection
        st = torch.tensor(sl, dtype=torch.int32, device=DEV)
        F.kv_write_scaled(k, v, st, kc, vc, ks, vs)
        R.kv_write_scaled(ref[0], ref[1], ref[2], ref[3], k.cpu(), v.cpu(), st.cpu())
        torch.cuda.synchronize()
        # the scale is one FP32 division of the same maximum on both sides
        Tolerance(0.0, 2.0 ** -22).check(ks, ref[2], f"key scales, step {n}")
        Tolerance(0.0, 2.0 ** -22).check(vs, ref[3], f"value scales, step {n}")
        # bytes: the same rounding of the same quotient up to the last bit of the FP32
        # reciprocal; compare the decoded values within one E4M3 step (2^-3 relative)
        tol = Tolerance(float(ref[2].max()) * 2.0 ** -9, 2.0 ** -3)
        tol.check(R.kv_dequant(kc.cpu(), ks.cpu()), R.kv_dequant(ref[0], ref[2]), f"key pages {n}")
        tol.check(R.kv_dequant(vc.cpu(), vs.cpu()), R.kv_dequant(ref[1], ref[3]), f"value pages {n}")
        same = (kc.cpu() == ref[0]).float().mean()
        assert float(same) > 0.995, f"step {n}: {float(same):.4f} of the key bytes agree"


@pytest.mark.parametrize("B,Hq,Hkv,ctx,splits", [(4, 32, 4, 300, 1), (3, 8, 1, 1100, 3),
                                                 (64, 32, 4, 1040, 1)])
def test_paged_decode_attention_fp8_pages(B, Hq, Hkv, ctx, splits):
    """E4M3 pages with per-page scales against the FP32 restatement over the decoded values:
    what differs is FP16 rounding of Q and P and the accumulation order."""
    D, page = 128, 16
    per = (ctx + page - 1) // page
    pages = B * per + 1
    g = torch.Generator(device=DEV).manual_seed(5)
    kc = torch.randint(0, 256, (pages, page, Hkv, D), dtype=torch.uint8, device=DEV, generator=g)
    vc = torch.randint(0, 256, (pages, page, Hkv, D), dtype=torch.uint8, device=DEV, generator=g)
    nan = lambda t: (t & 0x7F) == 0x7F                       # the two E4M3 NaN encodings
    kc[nan(kc)] = 0
    vc[nan(vc)] = 0
    ks = (torch.rand(pages, device=DEV, generator=g) * 0.004 + 0.0005)
    vs = (torch.rand(pages, device=DEV, generator=g) * 0.01 + 0.001)
    q = rnd(B, Hq, D, seed=6)
    pt = (torch.randperm(pages - 1, device=DEV, generator=g)[:B * per].view(B, per) + 1).to(torch.int32)
    sl = torch.tensor([ctx - (7 * b) % 50 for b in range(B)], dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(D)
    scratch, counters = F.decode_scratch(B, Hq, Hkv, D, splits, DEV)
    out = F.paged_decode_attention(q, kc, vc, pt, sl, scale, splits, scratch=scratch,
                                   counters=counters if splits > 1 else None, k_scale=ks, v_scale=vs)
    ref = R.paged_decode_attention(q.cpu().float(), kc.cpu(), vc.cpu(), pt.cpu(), sl.cpu(), scale, 0,
                                   ks.cpu(), vs.cpu())
    # scores: D products with Q rounded to FP16; probabilities rounded to FP16, ctx of them
    # summed against values that are exact in FP16; one bf16 store
    f16 = torch.float16
    smax = float(q.float().abs().max()) * 448.0 * float(ks.max()) * math.sqrt(D) * scale
    tol = Tolerance.dot(D, out=torch.float32, inputs=f16).scaled(max(1.0, smax)) \
        .then(Tolerance.dot(ctx, out=BF, inputs=f16)).then(BF16_STORE)
    tol.check(out, ref, "fp8 paged decode attention")


def test_kv_gather_and_cached_context_prefill():
    """Pages -> packed rows through the page table (bf16 and E4M3 pages), then a chunked
    prefill through the engine: the second chunk attends to the first through the gather and
    gives the tokens of an unchunked run."""
    page, Hkv, D, pages = 16, 2, 128, 20
    kc, vc = rnd(pages, page, Hkv, D, seed=1), rnd(pages, page, Hkv, D, seed=2)
    pt = torch.tensor([[3, 9, 4, 0], [7, 1, 0, 0]], dtype=torch.int32, device=DEV)
    lens = [37, 20]
    cu = torch.tensor([0, 37, 57], dtype=torch.int32, device=DEV)
    ko, vo = F.kv_gather(kc, vc, pt, cu, 57)
    for s, n in enumerate(lens):
        want = kc[pt[s].long()].reshape(-1, Hkv, D)[:n]
        Tolerance.exact().check(ko[int(cu[s]):int(cu[s]) + n], want, "gathered keys")
        want = vc[pt[s].long()].reshape(-1, Hkv, D)[:n]
        Tolerance.exact().check(vo[int(cu[s]):int(cu[s]) + n], want, "gathered values")
    k8 = torch.randint(0, 120, (pages, page, Hkv, D), dtype=torch.uint8, device=DEV)
    sc = torch.rand(pages, device=DEV) * 0.01 + 0.001
    out_cu = torch.tensor([5, 60], dtype=torch.int32, device=DEV)       # room between sequences
    buf = (torch.zeros(100, Hkv, D, dtype=BF, device=DEV), torch.zeros(100, Hkv, D, dtype=BF, device=DEV))
    F.kv_gather(k8, k8, pt, cu, 57, sc, sc, out=buf, out_cu=out_cu)
    deq = R.kv_dequant(k8.cpu(), sc.cpu())
    for s, n in enumerate(lens):
        want = deq[pt[s].cpu().long()].reshape(-1, Hkv, D)[:n]
        Tolerance(0.0, 2.0 ** -8).check(buf[0][int(out_cu[s]):int(out_cu[s]) + n], want, "fp8 gather")
    assert float(buf[0][:5].abs().max()) == 0.0

    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    import dataclasses
    cfg = dataclasses.replace(Qwen3MoeConfig.tiny(), head_dim=128)     # the FP8 kernel's width
    prompts = [[(5 * i + j) % cfg.vocab_size for i in range(n)] for j, n in enumerate((150, 33, 70))]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    outs = {}
    for name, kw in (("whole", {}), ("chunked", {"max_num_batched_tokens": 64}),
                     ("fp8", {"max_num_batched_tokens": 64, "kv_dtype": "fp8"})):
        model = Qwen3MoeModel(cfg, DEV, BF).init_random(seed=0)
        eng = LLMEngine(model, num_pages=128, max_num_seqs=4, max_model_len=256, **kw)
        outs[name] = eng.generate(prompts, sp)
    agree = lambda a, b: sum(x == y for p, q_ in zip(a, b) for x, y in zip(p, q_)) / 24.0
    assert agree(outs["whole"], outs["chunked"]) >= 0.9, outs
    assert agree(outs["whole"], outs["fp8"]) >= 0.6, outs


def test_engine_sleep_levels_free_memory_and_wake_restores_tokens():
    """Level 1 frees the KV cache and graphs, level 2 parks the weights in pinned host memory;
    after wake the engine gives the tokens it gave before."""
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    cfg = Qwen3MoeConfig.tiny()
    model = Qwen3MoeModel(cfg, DEV, BF).init_random(seed=0)
    eng = LLMEngine(model, num_pages=256, max_num_seqs=4, max_model_len=256)
    prompts = [[(3 * i + j) % cfg.vocab_size for i in range(n)] for j, n in enumerate((17, 40))]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    want = eng.generate(prompts, sp)
    for level in (1, 2):
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        out = eng.sleep(level)
        after = torch.cuda.memory_allocated()
        assert out["freed_bytes"] > 0 and before - after >= 0.9 * out["freed_bytes"]
        if level == 2:
            assert model.embed is None and model.layers[0].qkv is None
        assert eng.step() == [] and not eng.has_work()
        eng.wake()
        assert eng.generate(prompts, sp) == want


@pytest.mark.parametrize("kv", [None, "fp8"])
def test_prefill_decode_handoff_between_gpu_engines(kv):
    """Prefill / decode disaggregation on the GPU: requests move after their first token
    (through the byte framing) into a second engine with its own pages (bf16 or E4M3), which
    continues with decode steps under CUDA graphs and gives one engine's tokens."""
    import dataclasses
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.handoff import PrefillDecodePair
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    cfg = dataclasses.replace(Qwen3MoeConfig.tiny(), head_dim=128)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (7, 33, 16)]
    sp = SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True)

    def engine():
        model = Qwen3MoeModel(cfg, DEV, BF).init_random(seed=0)
        return LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=160, kv_dtype=kv)
    ref = engine().generate(prompts, sp)
    pre, dec = engine(), engine()
    pair = PrefillDecodePair(pre, dec, through_bytes=True)
    rids = [pair.add_request(p, sp, request_id=f"req-{i + 1}") for i, p in enumerate(prompts)]
    outs = {r: [] for r in rids}
    while pair.has_work():
        for o in pair.step():
            outs[o.request_id].extend(o.new_token_ids)
    got = [outs[r] for r in rids]
    assert pair.moved == 3 and dec.scheduler.stats["prefill_tokens"] <= 3
    if kv is None:
        assert got == ref
    else:       # pages are re-quantised on import: near-ties of the random model may flip
        same = sum(a == b for x, y in zip(ref, got) for a, b in zip(x, y))
        assert [x[0] for x in got] == [x[0] for x in ref] and same >= 0.7 * 27, (ref, got)


def test_two_expert_exchanges_live_side_by_side():
    """Exchanges are handles, not a process-wide singleton: two of them (different sizes) are
    alive at once, used alternately, and each gives the MoE layer its local form gives."""
    from uniserve_v1_b200.parallel.expert_exchange import ExpertExchange
    k, H, E, I = 4, 512, 16, 256
    exs = [ExpertExchange(None, 0, 1, DEV, T, k, H, E, I) for T in (24, 40)]
    assert exs[0].h.value != exs[1].h.value
    w13, w2 = rnd(E, 2 * I, H, scale=0.03, seed=1), rnd(E, H, I, scale=0.03, seed=2)
    nw = torch.ones(H, dtype=BF, device=DEV)
    for it in range(3):
        for n, ex in enumerate(exs):
            T = ex.T
            x = rnd(T, H, scale=0.5, seed=10 * it + n)
            logits = rnd(T, E, dtype=torch.float32, seed=100 + 10 * it + n)
            res = rnd(T, H, dtype=torch.float32, seed=200 + 10 * it + n)
            ids, wts = F.topk_softmax(logits, k, True)
            live = torch.full((1,), T, dtype=torch.int32, device=DEV)
            ex.dispatch(x, ids, wts, live)
            ex.experts(w13, w2, T)
            res_ex = res.clone()
            y = ex.combine_add_rmsnorm(ids, live, res_ex, nw, 1e-6)
            y = y[0] if isinstance(y, tuple) else y
            local = F.moe_experts(x, ids, wts, w13, w2)
            y_ref, _ = F.add_rmsnorm(local, res.clone(), nw, 1e-6)
            close(y, y_ref, 4e-2, 4e-2)
    for ex in exs:
        ex.close()


def test_weights_keeper_maps_device_weights_into_another_process(tmp_path):
    """A `keep` process holds the weights in ITS device memory; this process opens the CUDA IPC
    handles, so its model's tensors are the keeper's memory, and generates the tokens of a model
    with its own weights."""
    import json
    import os
    import subprocess
    import sys
    from uniserve_v1_b200.__main__ import _qwen3_model
    from uniserve_v1_b200.config.policy import Package
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.server.weights_keeper import stop_keeper
    pkg_dir = tmp_path / "pkg"
    pkg_dir.mkdir()
    (pkg_dir / "config.toml").write_text('model = "random:tiny"\nserved_model_name = "tiny"\n')
    sock = str(tmp_path / "w.sock")
    r, w = os.pipe()
    os.set_inheritable(w, True)
    proc = subprocess.Popen([sys.executable, "-m", "uniserve_v1_b200", "keep", str(pkg_dir),
                             "--socket", sock, "--ready-fd", str(w)], pass_fds=(w,),
                            cwd=os.path.dirname(os.path.dirname(__file__)))
    os.close(w)
    try:
        info = json.loads(os.read(r, 4096).split(b"\n")[0])
        assert info["state"] == "keeping"
        pkg = Package.load(str(pkg_dir))
        dev = torch.device("cuda", 0)
        prompts = [[(3 * i + j) % 1000 for i in range(n)] for j, n in enumerate((9, 30))]
        sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
        _, own, _ = _qwen3_model(pkg, None, dev, BF, None)
        want = LLMEngine(own, num_pages=64, max_num_seqs=4, max_model_len=128).generate(prompts, sp)
        before = torch.cuda.memory_allocated()
        _, mapped, _ = _qwen3_model(pkg, None, dev, BF, None, sock)
        assert mapped.weights_from["keeper_pid"] == proc.pid
        assert torch.cuda.memory_allocated() - before < own.weight_bytes() // 4   # mapped, not copied
        assert torch.equal(mapped.embed, own.embed)
        got = LLMEngine(mapped, num_pages=64, max_num_seqs=4, max_model_len=128).generate(prompts, sp)
        assert got == want
        del mapped
        assert stop_keeper(sock)
        proc.wait(timeout=60)
    finally:
        os.close(r)
        if proc.poll() is None:
            proc.terminate()


def test_profile_timeline_collector_sees_the_library_kernels(tmp_path):
    """A session with the ``timeline`` collector holds one record per kernel the process ran
    while it was open - also the kernels this package launches through its own library, which
    never pass through PyTorch - beside the fence probes of the step."""
    from uniserve_v1_b200.engine.profiling import StepProfiler
    from uniserve_v1_b200.tools import profile as P
    x, w = rnd(64, 1024), rnd(512, 1024, scale=0.05)
    F.linear(x, w)                                   # library loaded, kernels configured
    torch.cuda.synchronize()
    prof = StepProfiler(DEV)
    path = str(tmp_path / "timeline.sqlite")
    prof.open(path, {"case": "gpu"}, collectors=["fence_timeline", "timeline"])
    with prof.step("decode", 0):
        y = F.linear(x, w)
        big = F.linear(rnd(512, 1024), w)
    torch.cuda.synchronize()
    prof.close()
    s = P.load(path)
    kernels = [k for k in s["kernels"] if k[2] == "kernel"]
    names = " ".join(k[1] for k in kernels)
    assert "gemm_wx" in names or "linear_decode" in names, names[:400]
    assert all(k[5] > 0 for k in kernels)
    assert len(P.device_ranges(s["probes"])) == 1
    assert P.summary([s])["kernels"]
    assert y.shape == (64, 512) and big.shape == (512, 512)
