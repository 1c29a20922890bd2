"""Block-scaled FP8: quantisers and the tcgen05 GEMM against FP32 restatements
built from the same quantised operands."""
import pytest
import torch

from uniserve_v1_b200.ops import fp8 as Q
from uniserve_v1_b200.ops import functional as F
from uniserve_v1_b200.ops import native as N

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator(device=DEV)
    g.manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=DEV) * scale).to(BF)


def teardown_function(_):
    torch.cuda.synchronize()
    N.raise_on_device_error()


def test_quantize_rows_matches_torch_cast():
    x = rnd(77, 512, scale=3.0)
    x[5] = 0                      # an all-zero row keeps scale 1
    q, s = Q.quantize_rows_block128(x)
    qc, sc = Q.quantize_rows_block128(x.cpu())
    torch.testing.assert_close(s[:, :77].cpu(), sc[:, :77], rtol=1e-6, atol=0)
    same = (q.cpu() == qc).float().mean().item()
    assert same > 0.999, same
    back = Q.dequantize_rows_block128(q.cpu(), s.cpu())
    torch.testing.assert_close(back, x.float().cpu(), rtol=0.07, atol=1e-3)


def test_quantize_tensor_static_and_dynamic():
    x = rnd(1000, 96, scale=2.0, seed=3)
    q, s = Q.quantize_tensor(x, scale=0.05)
    want = (x.float() * (1.0 / 0.05)).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    assert (q == want).float().mean().item() > 0.999
    q2, s2 = Q.quantize_tensor(x)
    amax = x.float().abs().max().item()
    assert abs(s2.item() - amax / 448.0) < 1e-6 * amax
    back = q2.view(torch.float8_e4m3fn).float() * s2
    torch.testing.assert_close(back, x.float(), rtol=0.07, atol=amax / 448.0)


@pytest.mark.parametrize("T,K,M,gated", [(5, 256, 128, False), (100, 512, 384, False),
                                         (300, 2048, 768, False), (64, 2048, 768, True),
                                         (130, 768, 2048, False), (17, 512, 256, True)])
def test_linear_fp8_block(T, K, M, gated):
    x = rnd(T, K, seed=1)
    w = rnd(2 * M if gated else M, K, scale=0.05, seed=2)
    wq, ws = Q.quantize_weight_block128(w)
    xq, xs = Q.quantize_rows_block128(x)
    out = Q.linear_fp8_block(None, wq, ws, gated=gated, xq=xq, x_scale=xs)
    xf = Q.dequantize_rows_block128(xq.cpu(), xs.cpu())
    wf = Q.dequantize_weight_block128(wq.cpu(), ws.cpu())
    y = xf @ wf.t()
    if gated:
        y = y[:, :M] * torch.nn.functional.silu(y[:, M:])
    torch.testing.assert_close(out.float().cpu(), y, rtol=2e-2, atol=2e-2)
    # and close to the unquantised product
    yf = x.float().cpu() @ w.float().cpu().t()
    if gated:
        yf = yf[:, :M] * torch.nn.functional.silu(yf[:, M:])
    err = (out.float().cpu() - yf).norm() / yf.norm()
    assert err < 0.08, err


@pytest.mark.parametrize("T,E,k,H,I", [(64, 16, 4, 512, 256), (9, 8, 2, 256, 128),
                                       (200, 8, 2, 512, 384)])
def test_moe_experts_fp8(T, E, k, H, I):
    x = rnd(T, H, seed=5)
    w13, w2 = rnd(E, 2 * I, H, scale=0.05, seed=6), rnd(E, H, I, scale=0.05, seed=7)
    ex = Q.Fp8Experts.from_bf16(w13, w2)
    g = torch.Generator(device=DEV)
    g.manual_seed(8)
    logits = torch.randn(T, E, generator=g, device=DEV)
    ids, wts = F.topk_softmax(logits, k, True)
    out = Q.moe_experts_fp8(x, ids, wts, ex)
    # FP32 restatement with the same quantisation points
    w13f = Q.dequantize_weight_block128(ex.w13.cpu(), ex.w13_scale.cpu())
    w2f = Q.dequantize_weight_block128(ex.w2.cpu(), ex.w2_scale.cpu())
    qd = lambda t: Q.dequantize_rows_block128(*Q.quantize_rows_block128(t.to(BF)))
    xc = qd(x.cpu())
    ref = torch.zeros(T, H)
    for t in range(T):
        for j in range(k):
            e = int(ids[t, j])
            y = w13f[e] @ xc[t]
            h = (y[:I] * torch.nn.functional.silu(y[I:])).to(BF)
            h = qd(h[None])[0]
            ref[t] += float(wts[t, j]) * (w2f[e] @ h).to(BF).float()
    torch.testing.assert_close(out.float().cpu(), ref, rtol=4e-2, atol=4e-2)


@pytest.mark.parametrize("T,K,M,gated", [(300, 512, 384, False), (1000, 1024, 640, True),
                                         (64, 256, 128, False),
                                         # more than one wave of tiles: the CTA-pair kernels
                                         (2600, 256, 2176, False), (2700, 256, 1152, True)])
def test_linear_fp8_per_tensor(T, K, M, gated):
    """Per-tensor weight scale, per-row dynamic activation scale, whole-K accumulation in
    tensor memory: against the FP32 product of the same quantised operands."""
    x = rnd(T, K, seed=41)
    w = rnd(2 * M if gated else M, K, scale=0.05, seed=42)
    wq, ws = Q.quantize_weight_tensor(w)
    out = Q.linear_fp8(x, wq, ws, gated=gated)
    ref = Q.linear_fp8(x.cpu(), wq.cpu(), ws, gated=gated)
    torch.testing.assert_close(out.float().cpu(), ref.float(), rtol=2e-2, atol=2e-2)
    yf = x.float().cpu() @ w.float().cpu().t()
    if gated:
        yf = yf[:, :M] * torch.nn.functional.silu(yf[:, M:])
    err = (out.float().cpu() - yf).norm() / yf.norm()
    assert err < 0.08, err
