"""Recurrent token mixers of the hybrid Qwen3.5 layers: the stateful causal depthwise
convolution and the gated delta rule.

    conv:   y_t[c] = silu( sum_j w[c, j] * x_{t - (K - 1) + j}[c] ),  state = last K - 1 inputs
    rule:   S <- S * exp(g_t);  d = (v_t - S^T k_t) * beta_t;  S <- S + k_t d^T;  o_t = S^T q_t

with q and k L2-normalised per head and q scaled by 1 / sqrt(d_k).  Both carry their
state across calls, so a prompt can be run in chunks and decoding is one step of the
same functions.  On a GPU the three entry points run the kernels of ``csrc/gated_delta.cu``
(state slice in registers, one pass over HBM per call); the PyTorch restatements below (a
step-by-step form and a chunked form built from matrix products and one triangular solve
per chunk) are the FP32 oracle and the CPU path.

Reference behaviour: crates/ops/kernels/causal_conv1d, crates/ops/kernels/gated_delta_rule,
crates/nn/src/modules/gated_delta_net.rs (reference project paths).
"""
from __future__ import annotations

import torch

from . import native as N

_KERNEL_DK = (16, 32, 64, 128)
USE_KERNELS = True        # False: the PyTorch restatements on every device (A/B, tests)


def _one_sequence(T: int, device):
    return (torch.tensor([0, T], dtype=torch.int32, device=device),
            torch.zeros(1, dtype=torch.int32, device=device))


def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor | None = None,
                  cu: torch.Tensor | None = None, slots: torch.Tensor | None = None):
    """x [T, C], weight [C, K], state [K - 1, C] (the inputs before x, zeros at the
    start) -> (silu(conv) [T, C], new state).  With ``cu`` [B + 1] and ``slots`` [B]
    (int32, on the device) x is a packed batch and ``state`` a pool [n, K - 1, C] that is
    updated in place (GPU only)."""
    T, C = x.shape
    K = weight.shape[1]
    if USE_KERNELS and x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and 2 <= K <= 8 \
            and x.stride(1) == 1:
        if state is None:
            state = torch.zeros(K - 1, C, dtype=x.dtype, device=x.device)
        elif cu is None:
            state = state.to(x.dtype).clone()     # callers keep the state they passed in
        assert state.is_contiguous() and state.dtype == x.dtype
        B = 1 if cu is None else slots.shape[0]
        if cu is None:
            cu, slots = _one_sequence(T, x.device)
        w = weight if weight.dtype in (torch.bfloat16, torch.float32) else weight.float()
        w = w.contiguous()
        y = torch.empty(T, C, dtype=x.dtype, device=x.device)
        N.call("us_causal_conv1d", N.ptr(x), x.stride(0), N.ptr(w), N.ptr(state), N.ptr(y), C,
               N.ptr(cu), N.ptr(slots), B, T, C, K, int(x.dtype == torch.bfloat16),
               int(w.dtype == torch.bfloat16), N.stream())
        return y, state
    assert cu is None, "packed batches run on the GPU kernels only"
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
    if USE_KERNELS and q.is_cuda and q.shape[-1] in _KERNEL_DK \
            and q.dtype in (torch.bfloat16, torch.float32) \
            and q.dtype == k.dtype == v.dtype:
        T, H, Dk = q.shape
        S = torch.zeros(H, Dk, v.shape[-1], dtype=torch.float32, device=q.device) \
            if state is None else state.float().clone()
        cu, slots = _one_sequence(T, q.device)
        out = gated_delta_rule_packed(q, k, v, S.unsqueeze(0), cu, slots, g=g.float().contiguous(),
                                      beta=beta.float().contiguous())
        return out, S
    if q.shape[0] > 16:
        return gated_delta_rule_chunked(q, k, v, g, beta, state, chunk)
    return gated_delta_rule_steps(q, k, v, g, beta, state)


def gated_delta_rule_packed(q, k, v, state, cu, slots, g=None, beta=None, raw=None,
                            eps: float = 1e-6):
    """The kernel form.  q, k [T, Hk, Dk] and v [T, Hv, Dv] may be strided views (last
    dimension dense) of one projection; Hk divides Hv (a key head serves Hv / Hk value
    heads).  ``state`` [n, Hv, Dk, Dv] FP32 is updated in place for the sequences
    ``slots`` [B] whose rows are ``cu`` [B + 1].  Gates: ``g`` and ``beta`` [T, Hv] FP32, or
    ``raw = (a, b, A, dt_bias)`` with a, b [T, Hv] views of the projection:
    g = A * softplus(a + dt_bias), beta = sigmoid(b), formed in the kernel."""
    T, Hk, Dk = q.shape
    Hv, Dv = v.shape[1], v.shape[2]
    assert q.stride(2) == k.stride(2) == v.stride(2) == 1 and state.dtype == torch.float32
    assert state.is_contiguous() and state.shape[1:] == (Hv, Dk, Dv)
    out = torch.empty(T, Hv, Dv, dtype=torch.float32, device=q.device)
    bf16 = int(q.dtype == torch.bfloat16)
    if raw is not None:
        a, b, A, dt_bias = raw
        assert a.dtype == q.dtype and a.stride(1) == 1 and a.stride(0) == b.stride(0)
        gates = (None, None, N.ptr(a), N.ptr(b), a.stride(0), N.ptr(A), N.ptr(dt_bias))
    else:
        assert g.dtype == torch.float32 and g.is_contiguous() and beta.is_contiguous()
        gates = (N.ptr(g), N.ptr(beta), None, None, Hv, None, None)
    N.call("us_gated_delta_rule", N.ptr(q), N.ptr(k), N.ptr(v), q.stride(0), k.stride(0),
           v.stride(0), q.stride(1), k.stride(1), v.stride(1), bf16, *gates, N.ptr(state),
           N.ptr(out), N.ptr(cu), N.ptr(slots), slots.shape[0], Hk, Hv, Dk, Dv, eps, N.stream())
    return out


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
    """Per-head RMSNorm of x (weight w) times silu(gate).  x [T, Hv, Dv]; on a GPU an FP32
    x (the rule's output) goes straight into the kernel and the result has gate's type."""
    if USE_KERNELS and x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 3 \
            and gate.dtype in (torch.bfloat16, torch.float32) and gate.stride(2) == 1:
        T, Hv, Dv = x.shape
        w = w.to(gate.dtype).contiguous()
        y = torch.empty(T, Hv, Dv, dtype=gate.dtype, device=x.device)
        N.call("us_rmsnorm_gated", N.ptr(x), N.ptr(w), N.ptr(gate), gate.stride(0), gate.stride(1),
               N.ptr(y), T * Hv, Hv, Dv, eps, int(gate.dtype == torch.bfloat16), N.stream())
        return y
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w
    return (y.float() * torch.nn.functional.silu(gate.float())).to(x.dtype)
