"""Multi-token-prediction head of the Qwen3.5-MoE family and the drafter built on it.

The head is one extra decoder layer that shares the target's embedding and output
matrices.  For position p it combines the target's hidden state with the embedding of
the token that *follows* it,

    x_p = fc([ norm_e(embed(t_{p+1})) ; norm_h(h_p) ])

runs the layer (attention over the head's own key / value stream, then the MoE or
dense feed-forward) and reads the prediction of t_{p+2} through the shared output
matrix.  Drafting k tokens applies it recurrently: its own output stands in for the
next hidden state and its own prediction for the next token.

``MtpDrafter`` plugs into ``LLMEngine.speculative_step``: the verification call hands it
the target's hidden states of the verified positions (``observe``), from which it
extends its stream and proposes the next drafts (``propose_for``).  The runner's prefill
hands it the prompt's hidden rows too (``tap``), so the head's key / value stream covers the
prompt as the reference's draft KV group does.  Whatever the head proposes, the output is
the target's own greedy choice.

Checkpoint names (``mtp.`` prefix): ``fc.weight`` [H, 2H], ``pre_fc_norm_embedding.weight``,
``pre_fc_norm_hidden.weight``, ``norm.weight``, ``layers.0.*`` as a decoder layer.

Reference behaviour: crates/models/src/qwen3/mtp.rs,
crates/engine/src/runner/causal_lm/speculation.rs (reference project paths).
"""
from __future__ import annotations

import math

import torch

from ..engine.speculation import Drafter
from ..ops import reference as R


class MtpHead:
    def __init__(self, target):
        """``target``: an unsharded ``Qwen3MoeModel`` whose embedding / output matrices,
        rotary table and config the head shares."""
        self.t, self.cfg = target, target.cfg
        self.device, self.dtype = target.device, target.dtype
        self.w: dict = {}

    # ------------------------------------------------------------- weights --
    def _shapes(self) -> dict:
        c = self.cfg
        H, D = c.hidden_size, c.head_dim
        s = {"fc.weight": (H, 2 * H), "pre_fc_norm_embedding.weight": (H,),
             "pre_fc_norm_hidden.weight": (H,), "norm.weight": (H,),
             "layers.0.input_layernorm.weight": (H,),
             "layers.0.post_attention_layernorm.weight": (H,),
             "layers.0.self_attn.q_proj.weight": (c.num_attention_heads * D, H),
             "layers.0.self_attn.k_proj.weight": (c.num_key_value_heads * D, H),
             "layers.0.self_attn.v_proj.weight": (c.num_key_value_heads * D, H),
             "layers.0.self_attn.o_proj.weight": (H, c.num_attention_heads * D),
             "layers.0.self_attn.q_norm.weight": (D,), "layers.0.self_attn.k_norm.weight": (D,)}
        if c.num_experts:
            I = c.moe_intermediate_size
            s["layers.0.mlp.gate.weight"] = (c.num_experts, H)
            s["layers.0.mlp.experts.w13"] = (c.num_experts, 2 * I, H)
            s["layers.0.mlp.experts.w2"] = (c.num_experts, H, I)
        else:
            I = c.intermediate_size
            s["layers.0.mlp.w13"] = (2 * I, H)
            s["layers.0.mlp.down_proj.weight"] = (H, I)
        return s

    def init_random(self, seed: int = 0, std: float = 0.02) -> "MtpHead":
        g = torch.Generator().manual_seed(seed)
        for name, shape in self._shapes().items():
            if len(shape) == 1:
                t = torch.ones(shape)
            else:
                t = torch.randn(*shape, generator=g) * std
            self.w[name] = t.to(device=self.device, dtype=self.dtype)
        return self

    def load_state(self, loader, prefix: str = "mtp.") -> "MtpHead":
        c = self.cfg

        def get(n):
            return loader.get(prefix + n).to(device=self.device, dtype=self.dtype)
        for name, shape in self._shapes().items():
            if name.endswith("experts.w13"):
                I = c.moe_intermediate_size
                w13 = torch.empty(shape, device=self.device, dtype=self.dtype)
                w2 = torch.empty(c.num_experts, c.hidden_size, I, device=self.device,
                                 dtype=self.dtype)
                for e in range(c.num_experts):
                    pe = f"layers.0.mlp.experts.{e}."
                    w13[e, :I], w13[e, I:] = get(pe + "up_proj.weight"), get(pe + "gate_proj.weight")
                    w2[e] = get(pe + "down_proj.weight")
                self.w[name], self.w["layers.0.mlp.experts.w2"] = w13, w2
            elif name.endswith("experts.w2"):
                continue
            elif name == "layers.0.mlp.w13":
                self.w[name] = torch.cat([get("layers.0.mlp.up_proj.weight"),
                                          get("layers.0.mlp.gate_proj.weight")], 0)
            else:
                self.w[name] = get(name)
        return self

    def export_state(self, prefix: str = "mtp.") -> dict:
        c, out = self.cfg, {}
        for name, t in self.w.items():
            if name.endswith("experts.w13"):
                I = c.moe_intermediate_size
                for e in range(c.num_experts):
                    pe = prefix + f"layers.0.mlp.experts.{e}."
                    out[pe + "up_proj.weight"], out[pe + "gate_proj.weight"] = t[e, :I], t[e, I:]
                    out[pe + "down_proj.weight"] = self.w["layers.0.mlp.experts.w2"][e]
            elif name.endswith("experts.w2"):
                continue
            elif name == "layers.0.mlp.w13":
                I = t.shape[0] // 2
                out[prefix + "layers.0.mlp.up_proj.weight"] = t[:I]
                out[prefix + "layers.0.mlp.gate_proj.weight"] = t[I:]
            else:
                out[prefix + name] = t
        return {k: v.detach().contiguous() for k, v in out.items()}

    # ------------------------------------------------------------- forward --
    def rows(self, hidden: torch.Tensor, next_tokens, position: int, kv: list):
        """T consecutive positions at once: ``hidden`` [T, H] of positions p .. p + T - 1, the
        token after each, the head's key / value stream ``kv`` = [K [n, Hkv, D], V] (extended in
        place; attention is causal inside the call and sees the whole earlier stream).
        Returns (head outputs [T, H], logits [T, V])."""
        c, w, t = self.cfg, self.w, self.t
        eps, D = c.rms_norm_eps, c.head_dim
        Hq, Hkv = c.num_attention_heads, c.num_key_value_heads
        toks = torch.as_tensor(next_tokens, device=self.device).long().reshape(-1)
        T = toks.shape[0]
        x = torch.cat([R.rmsnorm(t.embed[toks], w["pre_fc_norm_embedding.weight"], eps),
                       R.rmsnorm(hidden.reshape(T, -1).to(self.dtype),
                                 w["pre_fc_norm_hidden.weight"], eps)], -1)
        x = R.linear(x, w["fc.weight"])
        n = R.rmsnorm(x, w["layers.0.input_layernorm.weight"], eps)
        q = R.linear(n, w["layers.0.self_attn.q_proj.weight"]).view(T, Hq, D)
        k = R.linear(n, w["layers.0.self_attn.k_proj.weight"]).view(T, Hkv, D)
        v = R.linear(n, w["layers.0.self_attn.v_proj.weight"]).view(T, Hkv, D)
        pos = torch.arange(position, position + T, device=self.device)
        q, k = R.qk_norm_rope(q, k, w["layers.0.self_attn.q_norm.weight"],
                              w["layers.0.self_attn.k_norm.weight"], pos, t.inv_freq, D, False, eps)
        kv[0] = k if kv[0] is None else torch.cat([kv[0], k], 0)
        kv[1] = v if kv[1] is None else torch.cat([kv[1], v], 0)
        from ..ops.attention import cached_causal_attention
        att = cached_causal_attention(q, kv[0], kv[1], 1.0 / math.sqrt(D)) \
            .reshape(T, Hq * D).to(self.dtype)
        x = x + R.linear(att, w["layers.0.self_attn.o_proj.weight"])
        n = R.rmsnorm(x, w["layers.0.post_attention_layernorm.weight"], eps)
        if c.num_experts:
            logits = R.linear(n, w["layers.0.mlp.gate.weight"], out_dtype=torch.float32)
            ids, wts = R.topk_softmax(logits, c.num_experts_per_tok, c.norm_topk_prob)
            y = R.moe_experts(n, ids, wts, w["layers.0.mlp.experts.w13"],
                              w["layers.0.mlp.experts.w2"])
        else:
            y = R.linear(R.linear_gated(n, w["layers.0.mlp.w13"]),
                         w["layers.0.mlp.down_proj.weight"])
        x = x + y
        out = R.rmsnorm(x, w["norm.weight"], eps)
        return x, R.linear(out, t.lm_head, out_dtype=torch.float32)

    def step(self, hidden: torch.Tensor, next_token: int, position: int, kv: list):
        """One position: (head output [H], logits [V])."""
        x, logits = self.rows(hidden[None], [int(next_token)], position, kv)
        return x[0], logits[0]


class MtpDrafter(Drafter):
    """Drafts with an ``MtpHead``; needs the target's hidden states (``needs_hidden``):
    the engine passes them to ``observe`` after every verification."""
    needs_hidden = True

    def __init__(self, head: MtpHead, k: int = 2, window: int = 1024):
        self.head, self.k, self.window = head, k, window
        self.state: dict = {}           # request id -> {"kv": [K, V], "pos": int, "out", "tok"}

    def ready(self, request_id: str) -> bool:
        return "tok" in self.state.get(request_id, {})

    def forget(self, keep_ids) -> None:
        for rid in [r for r in self.state if r not in keep_ids]:
            del self.state[rid]

    def observe(self, request_id: str, first_position: int, hidden: torch.Tensor,
                next_tokens: list) -> None:
        """``hidden[i]`` is the target's state at position ``first_position + i`` and
        ``next_tokens[i]`` the token that follows it (accepted or the target's own)."""
        st = self.state.setdefault(request_id, {"kv": [None, None]})
        if not len(next_tokens):
            return
        outs, logits_all = self.head.rows(hidden[:len(next_tokens)], list(next_tokens),
                                          first_position, st["kv"])
        out, logits = outs[-1], logits_all[-1]
        if st["kv"][0].shape[0] > self.window:
            st["kv"] = [st["kv"][0][-self.window:], st["kv"][1][-self.window:]]
        st["pos"] = first_position + len(next_tokens) - 1
        st["out"], st["tok"] = out, int(logits.argmax())

    def tap(self, request, start: int, hidden: torch.Tensor) -> None:
        """Prefill hook of the runner: the target's hidden rows of prompt positions
        start .. start + T - 1.  Every position whose next token is already known extends the
        head's stream, so drafting starts with the prompt's context (the last position waits
        for its sampled token and arrives through ``observe``)."""
        ids = request.all_ids
        rid = request.request_id
        if start == 0:
            self.state.pop(rid, None)              # a fresh (or recomputed) prompt: new stream
        n = min(hidden.shape[0], len(ids) - 1 - start)
        if n > 0:
            self.observe(rid, start, hidden[:n], ids[start + 1:start + 1 + n])
        if n < hidden.shape[0]:                    # the last position: its token is being sampled
            self.state.setdefault(rid, {"kv": [None, None]})["pending"] = \
                (start + n, hidden[n:n + 1].detach().clone())

    def propose_for(self, request) -> list:
        st = self.state.get(request.request_id)
        if st is not None and st.get("pending") is not None:
            pos, row = st.pop("pending")
            ids = request.all_ids
            if pos + 1 < len(ids) and (st["kv"][0] is None or "pos" not in st or st["pos"] == pos - 1):
                self.observe(request.request_id, pos, row, [ids[pos + 1]])
        if st is None or "tok" not in st:
            return []
        drafts = [st["tok"]]
        # recurrent drafts run on a copy of the stream: only verified positions stay in it
        kv = [st["kv"][0].clone(), st["kv"][1].clone()]
        out, pos = st["out"], st["pos"]
        while len(drafts) < self.k:
            pos += 1
            out, logits = self.head.step(out, drafts[-1], pos, kv)
            drafts.append(int(logits.argmax()))
        return drafts

    def propose(self, token_ids) -> list:          # interface of drafters without state
        return []
