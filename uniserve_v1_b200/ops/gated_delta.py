"""Recurrent token mixers of the hybrid Qwen3.5 layers: the stateful causal depthwise
convolution and the gated delta rule.

    conv:   y_t[c] = silu( sum_j w[c, j] * x_{t - (K - 1) + j}[c] ),  state = last K - 1 inputs
    rule:   S <- S * exp(g_t);  d = (v_t - S^T k_t) * beta_t;  S <- S + k_t d^T;  o_t = S^T q_t

with q and k L2-normalised per head and q scaled by 1 / sqrt(d_k).  Both carry their
state across calls, so a prompt can be run in chunks and decoding is one step of the
same functions.  These are the FP32 formulas on PyTorch tensors (any device): a step-by-step
form and a chunked form built from matrix products and one triangular solve per chunk;
dedicated tensor-core kernels for them are not part of this package.

Reference behaviour: crates/ops/kernels/causal_conv1d, crates/ops/kernels/gated_delta_rule,
crates/nn/src/modules/gated_delta_net.rs (reference project paths).
"""
from __future__ import annotations

import torch


def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor | None = None):
    """x [T, C], weight [C, K], state [K - 1, C] (the inputs before x, zeros at the
    start) -> (silu(conv) [T, C], new state)."""
    T, C = x.shape
    K = weight.shape[1]
    if state is None:
        state = torch.zeros(K - 1, C, dtype=x.dtype, device=x.device)
    full = torch.cat([state, x], 0).float()                       # [K - 1 + T, C]
    win = full.unfold(0, K, 1)                                    # [T, C, K]
    y = torch.nn.functional.silu((win * weight.float()[None]).sum(-1))
    return y.to(x.dtype), full[-(K - 1):].to(x.dtype)


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def gated_delta_rule(q, k, v, g, beta, state=None, chunk: int = 64):
    """q, k [T, H, Dk], v [T, H, Dv], g (log decay) and beta [T, H], state [H, Dk, Dv]
    -> (o [T, H, Dv] FP32, new state FP32).  Long inputs run chunk by chunk
    (``gated_delta_rule_chunked``), short ones step by step."""
    if q.shape[0] > 16:
        return gated_delta_rule_chunked(q, k, v, g, beta, state, chunk)
    return gated_delta_rule_steps(q, k, v, g, beta, state)


def gated_delta_rule_chunked(q, k, v, g, beta, state=None, chunk: int = 64):
    """The same recurrence, C positions at a time.  With G the running sum of g inside
    the chunk and S0 the state at its start, the corrections u_t = beta_t (v_t - S_{t-1}^T k_t)
    solve a unit lower-triangular system

        (I + L) U = beta * (V - diag(e^G) K S0),   L[t, j] = beta_t e^{G_t - G_j} (k_t . k_j), j < t

    after which  O = diag(e^G) Q S0 + tril(e^{G_t - G_j} Q K^T) U  and
    S_C = e^{G_C} S0 + (K e^{G_C - G})^T U  are matrix products."""
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    qf = (l2norm(q.float()) * (Dk ** -0.5)).transpose(0, 1)       # [H, T, Dk]
    kf = l2norm(k.float()).transpose(0, 1)
    vf, gf, bf = v.float().transpose(0, 1), g.float().t(), beta.float().t()
    S = torch.zeros(H, Dk, Dv, device=q.device) if state is None else state.float().clone()
    out = torch.empty(H, T, Dv, device=q.device)
    for lo in range(0, T, chunk):
        hi = min(T, lo + chunk)
        C = hi - lo
        Q, K, V, B = qf[:, lo:hi], kf[:, lo:hi], vf[:, lo:hi], bf[:, lo:hi]
        G = gf[:, lo:hi].cumsum(-1)                               # [H, C]
        decay = (G[:, :, None] - G[:, None, :]).tril().exp().tril()       # e^{G_t - G_j}, j <= t
        L = (torch.einsum("htd,hjd->htj", K, K) * decay * B[:, :, None]).tril(-1)
        eye = torch.eye(C, device=q.device).expand(H, C, C)
        rhs = B[:, :, None] * (V - G.exp()[:, :, None] * torch.einsum("htd,hdv->htv", K, S))
        U = torch.linalg.solve_triangular(eye + L, rhs, upper=False, unitriangular=True)
        out[:, lo:hi] = G.exp()[:, :, None] * torch.einsum("htd,hdv->htv", Q, S) + \
            torch.einsum("htj,hjv->htv", torch.einsum("htd,hjd->htj", Q, K) * decay, U)
        tail = (G[:, -1:] - G).exp()                                        # e^{G_C - G_j}
        S = G[:, -1].exp()[:, None, None] * S + torch.einsum("hjd,hjv->hdv", K * tail[:, :, None], U)
    return out.transpose(0, 1).contiguous(), S


def gated_delta_rule_steps(q, k, v, g, beta, state=None):
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    q = l2norm(q.float()) * (Dk ** -0.5)
    k = l2norm(k.float())
    v, g, beta = v.float(), g.float(), beta.float()
    S = torch.zeros(H, Dk, Dv, device=q.device) if state is None else state.float().clone()
    out = torch.empty(T, H, Dv, device=q.device)
    for t in range(T):
        S = S * g[t].exp()[:, None, None]
        mem = torch.einsum("hkv,hk->hv", S, k[t])
        d = (v[t] - mem) * beta[t][:, None]
        S = S + k[t][:, :, None] * d[:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out, S


def rmsnorm_gated(x: torch.Tensor, w: torch.Tensor, gate: torch.Tensor, eps: float):
    """Per-head RMSNorm of x (weight w) times silu(gate)."""
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w
    return (y.float() * torch.nn.functional.silu(gate.float())).to(x.dtype)
