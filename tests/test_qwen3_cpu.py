"""Tiny Qwen3-MoE on CPU: the engine (paged cache, scheduler, fused-op CPU
formulas) must reproduce an independent FP32 reference decode."""
import os

import pytest
import torch

from uniserve_v1_b200.engine.engine import LLMEngine
from uniserve_v1_b200.engine.types import SamplingParams
from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
from uniserve_v1_b200.models.reference_cpu import ReferenceQwen3Moe


def _tiny():
    torch.manual_seed(0)
    return Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)


def test_greedy_decode_matches_reference():
    model = _tiny()
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, 1024, (32,), generator=g).tolist()
    ref = ReferenceQwen3Moe(model).greedy(torch.tensor(prompt), 16)
    eng = LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=256, use_graphs=False)
    out = eng.generate([prompt], SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True))
    assert out[0] == ref


def test_batched_requests_match_single():
    model = _tiny()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (5, 17, 32, 40)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    eng = LLMEngine(model, num_pages=128, max_num_seqs=8, max_model_len=256, use_graphs=False)
    batched = eng.generate(prompts, sp)
    for p, b in zip(prompts, batched):
        single = LLMEngine(model, num_pages=64, max_num_seqs=2, max_model_len=256,
                           use_graphs=False).generate([p], sp)[0]
        assert single == b


def test_chunked_prefill_and_prefix_cache():
    model = _tiny()
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, 1024, (70,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    whole = LLMEngine(model, num_pages=64, max_num_seqs=2, max_model_len=256,
                      use_graphs=False).generate([prompt], sp)[0]
    eng = LLMEngine(model, num_pages=64, max_num_seqs=2, max_model_len=256, use_graphs=False,
                    max_num_batched_tokens=24)
    assert eng.generate([prompt], sp)[0] == whole
    # second run of the same prompt is served from cached pages
    assert eng.generate([prompt], sp)[0] == whole
    assert eng.stats()["cached_tokens"] >= 64


def test_sampling_is_batch_invariant():
    model = _tiny()
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1024, (12,), generator=g).tolist() for _ in range(3)]
    sps = [SamplingParams(temperature=0.8, top_k=20, top_p=0.95, seed=100 + i, max_tokens=6,
                          ignore_eos=True) for i in range(3)]
    eng = LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=128, use_graphs=False)
    together = eng.generate(prompts, sps)
    for p, sp, t in zip(prompts, sps, together):
        alone = LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=128,
                          use_graphs=False).generate([p], sp)[0]
        assert alone == t


def test_host_kv_tier_brings_back_evicted_prefix_pages():
    """With a device pool too small to retain an old prompt's pages, the host tier keeps
    them: the prompt's second run is served from host copies (cached tokens reported,
    same tokens generated) instead of being recomputed."""
    import torch
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    g = torch.Generator().manual_seed(3)
    first = torch.randint(0, 1024, (70,), generator=g).tolist()
    others = [torch.randint(0, 1024, (70,), generator=g).tolist() for _ in range(3)]

    def run(host_pages):
        eng = LLMEngine(model, num_pages=12, page_size=16, max_num_seqs=2, max_model_len=128,
                        use_graphs=False, host_kv_pages=host_pages)
        a = eng.generate([first], sp)[0]
        for o in others:                       # push the first prompt's pages out of the pool
            eng.generate([o], sp)
        rid = eng.add_request(first, sp)
        req = eng.scheduler.requests[rid]
        while eng.has_work():
            eng.step()
        return a, req.output_ids, req.num_cached, eng.blocks.host_stats()
    a0, b0, cached0, st0 = run(0)
    a1, b1, cached1, st1 = run(32)
    assert a0 == a1 == b0 == b1
    assert cached0 == 0 and st0["host_slots"] == 0
    assert cached1 == 64 and st1["host_hits"] >= 4 and st1["host_offloads"] >= 4


def test_host_slot_with_pending_fetch_is_not_recycled_by_offloads_of_the_same_step():
    """A tiny host tier: a prefix match hands out host slots, and the device pages it then
    allocates evict cached pages whose offloads would recycle exactly those slots.  The
    matched slots stay pinned until the copies are handed over, so after the moves every
    fetched device page holds the content of its own key; offloads with no unpinned slot
    are dropped, and no slot appears twice in one offload batch."""
    import numpy as np
    from uniserve_v1_b200.engine.block_manager import BlockManager
    bm = BlockManager(num_pages=5, page_size=4)          # 4 usable device pages
    bm.enable_host_tier(2)
    key = lambda i: (1000 + i, 7)
    device = {}                                          # page -> content tag
    host = {}                                            # slot -> content tag

    def moves():
        off, fet = bm.take_moves()
        assert len({s for _, s in off}) == len(off)
        for page, slot in off:
            host[slot] = device[page]
        for slot, page in fet:
            device[page] = host[slot]

    # contents 0..3 committed on the device, released (cached, unreferenced)
    pages = bm.allocate(4)
    for i, pg in enumerate(pages):
        device[pg] = i
        assert bm.commit(pg, key(i)) == pg
    bm.release(pages)
    # two fresh pages push contents 0 and 1 to the two host slots
    a = bm.allocate(2)
    moves()
    for pg in a:
        device[pg] = "x"
    assert sorted(host.values()) == [0, 1]
    bm.release(a)                                        # unkeyed: plain free pages
    keys = np.array([key(0), key(1)], dtype=np.uint64)
    # take every free page so that the fetch below must evict cached pages 2 and 3,
    # whose offloads want host slots while both slots have a pending fetch
    hold = bm.allocate(2)
    got = bm.fetch_prefix(keys, 0, 2)
    assert len(got) == 2
    moves()
    assert [device[pg] for pg in got] == [0, 1]          # not the evicted pages' content
    assert bm.host_stats()["host_used"] == 2
    bm.release(hold + got)
    # the pins are gone: later evictions use the slots again
    more = bm.allocate(4)
    moves()
    assert sorted(host.values()) == [0, 1]               # contents 0, 1 offloaded again
    bm.release(more)


def test_speculative_steps_reproduce_plain_decoding():
    """Verification keeps the agreed prefix plus one model token: whatever the drafter
    proposes, the output equals step-by-step greedy decoding; an oracle drafter advances
    k + 1 tokens per step, a wrong one still advances one."""
    import torch
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.speculation import Drafter, NgramDrafter, accept
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    assert accept([5, 6, 7], [5, 6, 9, 1]) == [5, 6, 9]
    assert accept([], [4]) == [4] and accept([1], [2, 3]) == [2]
    assert NgramDrafter(n=2, k=3).propose([1, 2, 3, 4, 9, 2, 3]) == [4, 9, 2]
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (11, 30)]
    mk = lambda: LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=128,
                           use_graphs=False)
    ref = mk().generate(prompts, sp)

    class Oracle(Drafter):
        k = 3

        def propose(self, ids):
            for p, r in zip(prompts, ref):
                full = p + r
                if list(ids) == full[:len(ids)]:
                    return full[len(ids):len(ids) + self.k]
            return []

    class Wrong(Drafter):
        k = 3

        def propose(self, ids):
            return [(ids[-1] + 1) % 1024] * 3

    for drafter, min_rate in ((Oracle(), 0.99), (Wrong(), 0.0), (NgramDrafter(), 0.0)):
        eng = mk()
        rids = [eng.add_request(p, sp) for p in prompts]
        outs = {r: [] for r in rids}
        steps = 0
        while eng.has_work():
            for o in eng.speculative_step(drafter):
                outs[o.request_id].extend(o.new_token_ids)
            steps += 1
        assert [outs[r] for r in rids] == ref
        st = eng.spec_stats
        if st["proposed"]:
            assert st["accepted"] / st["proposed"] >= min_rate
        if isinstance(drafter, Oracle):
            assert steps <= 2 + 4 + 1          # prefill steps + ceil(11 / 4) verify steps


def test_mtp_drafter_keeps_outputs_and_round_trips_its_weights():
    """A multi-token-prediction head drafts from the target's hidden states: whatever it
    proposes the output stays the target's greedy decoding; its weights load back from
    their checkpoint names."""
    import torch
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.models.qwen3_mtp import MtpDrafter, MtpHead
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    head = MtpHead(model).init_random(seed=7)
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (9, 21)]
    mk = lambda: LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=128,
                           use_graphs=False)
    ref = mk().generate(prompts, sp)
    eng, drafter = mk(), MtpDrafter(head, k=2)
    rids = [eng.add_request(p, sp) for p in prompts]
    outs = {r: [] for r in rids}
    while eng.has_work():
        for o in eng.speculative_step(drafter):
            outs[o.request_id].extend(o.new_token_ids)
    assert [outs[r] for r in rids] == ref
    assert eng.spec_stats["proposed"] >= 2 * 4          # it did draft, two tokens at a time
    # the prompt's hidden rows reached the head at prefill: its stream covered the prompt
    # before the first draft, without a bootstrap verification
    eng2, d2 = mk(), MtpDrafter(head, k=2)
    rid = eng2.add_request(prompts[1], sp)
    eng2.speculative_step(d2)                           # prefill
    assert d2.state[rid]["kv"][0].shape[0] == len(prompts[1]) - 1 and "pending" in d2.state[rid]
    eng2.speculative_step(d2)                           # first verification, already with drafts
    assert eng2.spec_stats["proposed"] == 2
    assert d2.state[rid]["kv"][0].shape[0] >= len(prompts[1]) + 1
    # the stream holds verified positions only, and finished requests are forgotten
    drafter.forget(set())
    assert drafter.state == {}

    class Dict:
        def __init__(self, d): self.d = d
        def get(self, n): return self.d[n]
        def has(self, n): return n in self.d
    state = head.export_state()
    assert "mtp.fc.weight" in state and "mtp.layers.0.mlp.experts.3.gate_proj.weight" in state
    again = MtpHead(model).load_state(Dict(state))
    h = torch.randn(model.cfg.hidden_size, generator=g)
    a = head.step(h, 5, 12, [None, None])
    b = again.step(h, 5, 12, [None, None])
    torch.testing.assert_close(a[1], b[1], rtol=0, atol=0)


def test_dense_qwen3_family():
    """The dense Qwen3 family (no experts): same decoder, gated MLP in every layer; the
    Hugging Face config of `Qwen3ForCausalLM` maps onto it."""
    import torch
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.models.reference_cpu import ReferenceQwen3Moe
    hf = {"architectures": ["Qwen3ForCausalLM"], "vocab_size": 512, "hidden_size": 128,
          "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2,
          "head_dim": 32, "intermediate_size": 256, "rms_norm_eps": 1e-6, "rope_theta": 1e6,
          "max_position_embeddings": 512, "eos_token_id": 511}
    cfg = Qwen3MoeConfig.from_hf(hf)
    assert cfg.num_experts == 0 and not cfg.is_moe_layer(0)
    model = Qwen3MoeModel(cfg, "cpu", torch.float32).init_random(0)
    assert all(lw.dense for lw in model.layers)
    prompt = [1, 2, 3, 4, 5]
    out = LLMEngine(model, num_pages=32, max_num_seqs=2, max_model_len=128,
                    use_graphs=False).generate(
        [prompt], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))[0]
    seq = list(prompt)
    for t in out:                                  # every token is the oracle's argmax
        logits, _ = ReferenceQwen3Moe(model).forward(torch.tensor(seq))
        assert int(logits[-1].argmax()) == t
        seq.append(t)


def test_gated_delta_rule_chunked_equals_stepwise():
    """Chunks of 64 (and a ragged tail), carried state, strong and weak decay."""
    import torch
    from uniserve_v1_b200.ops import gated_delta as GD
    g_ = torch.Generator().manual_seed(0)
    T, H, Dk, Dv = 150, 3, 16, 24
    q, k = torch.randn(T, H, Dk, generator=g_), torch.randn(T, H, Dk, generator=g_)
    v = torch.randn(T, H, Dv, generator=g_)
    beta = torch.rand(T, H, generator=g_)
    for scale in (0.01, 2.0):
        g = -torch.rand(T, H, generator=g_) * scale
        s0 = torch.randn(H, Dk, Dv, generator=g_) * 0.3
        o1, s1 = GD.gated_delta_rule_steps(q, k, v, g, beta, s0)
        o2, s2 = GD.gated_delta_rule_chunked(q, k, v, g, beta, s0, chunk=64)
        torch.testing.assert_close(o2, o1, atol=2e-4, rtol=2e-4)
        torch.testing.assert_close(s2, s1, atol=2e-4, rtol=2e-4)
        # a prompt in two calls equals one call
        oa, sa = GD.gated_delta_rule(q[:70], k[:70], v[:70], g[:70], beta[:70], s0)
        ob, sb = GD.gated_delta_rule(q[70:], k[70:], v[70:], g[70:], beta[70:], sa)
        torch.testing.assert_close(torch.cat([oa, ob]), o1, atol=2e-4, rtol=2e-4)
    x = torch.randn(20, 6, generator=g_)
    w = torch.randn(6, 4, generator=g_)
    y_all, st_all = GD.causal_conv1d(x, w)
    y_a, st = GD.causal_conv1d(x[:7], w)
    y_b, st = GD.causal_conv1d(x[7:], w, st)
    torch.testing.assert_close(torch.cat([y_a, y_b]), y_all)
    torch.testing.assert_close(st, st_all)


def test_hybrid_decoder_batched_decode_equals_sequential():
    """Several sequences advancing in one batched step (shared projections and experts,
    vectorised delta rule and convolution, per-sequence attention) produce the logits of
    separate calls, and the dense-state engine takes that path."""
    import torch
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_5 import Qwen35MoeModel
    model = Qwen35MoeModel(Qwen35MoeModel.tiny_config(), "cpu", torch.float32).init_random(seed=0)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1000, (n,), generator=g) for n in (7, 19, 4)]
    states = [model.new_state() for _ in prompts]
    for p, st in zip(prompts, states):
        model.forward(p, st, 0)
    import copy
    seq_states = copy.deepcopy(states)
    toks = torch.tensor([11, 22, 33])
    pos = torch.tensor([len(p) for p in prompts])
    got = model.decode_batch(toks, states, pos[None].expand(3, -1))
    want = torch.cat([model.forward(toks[i:i + 1], seq_states[i], int(pos[i])) for i in range(3)])
    torch.testing.assert_close(got, want, atol=2e-5, rtol=2e-5)
    again = model.decode_batch(toks, states, (pos + 1)[None].expand(3, -1))      # states advanced
    want2 = torch.cat([model.forward(toks[i:i + 1], seq_states[i], int(pos[i]) + 1) for i in range(3)])
    torch.testing.assert_close(again, want2, atol=2e-5, rtol=2e-5)
    calls = {"n": 0}
    inner = model.decode_batch

    def counted(*a):
        calls["n"] += 1
        return inner(*a)
    model.decode_batch = counted
    eng = DenseStateEngine(model, max_num_seqs=4)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    outs = eng.generate([p.tolist() for p in prompts], sp)
    model.decode_batch = inner
    assert calls["n"] >= 4
    assert outs == [DenseStateEngine(model).generate([p.tolist()], sp)[0] for p in prompts]


def test_dense_state_engine_reuses_state_snapshots_of_a_shared_prefix():
    """Recurrent decoders cache whole-state snapshots at interval boundaries of a prompt: a
    later request with the same prefix (and the same isolation salt) starts from the longest
    one, reads only the rest, and answers the same."""
    import torch
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_5 import Qwen35MoeModel
    model = Qwen35MoeModel(Qwen35MoeModel.tiny_config(), "cpu", torch.float32).init_random(seed=0)
    g = torch.Generator().manual_seed(3)
    shared = torch.randint(0, 1000, (70,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    cold = DenseStateEngine(model, state_cache_entries=0)
    want_a = cold.generate([shared + [1, 2, 3]], sp)[0]
    want_b = cold.generate([shared + [9, 8]], sp)[0]
    assert cold.stats()["cached_tokens"] == 0
    eng = DenseStateEngine(model, state_interval=16, prefill_chunk=32)
    assert eng.generate([shared + [1, 2, 3]], sp)[0] == want_a
    first = eng.stats()["prefill_tokens"]
    assert eng.generate([shared + [9, 8]], sp)[0] == want_b
    st = eng.stats()
    assert st["cached_tokens"] == 64 and st["prefill_tokens"] - first == 72 - 64
    rid = eng.add_request(shared + [9, 8], sp, cache_salt="tenant-2")       # another tenant
    while eng.has_work():
        eng.step()
    assert eng.requests[rid].num_cached == 0 and eng.requests[rid].output_ids == want_b
    assert eng.blocks.flush() > 0 and not eng.state_cache


def test_dense_state_engine_speculation_rolls_recurrent_state_back():
    """Speculative steps on the hybrid decoder: accepted drafts advance several tokens per
    call, a refused draft restores the snapshot of the recurrent state and replays the accepted
    part; outputs equal plain decoding whatever the drafter proposes."""
    import torch
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.engine.speculation import Drafter, NgramDrafter
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_5 import Qwen35MoeModel
    model = Qwen35MoeModel(Qwen35MoeModel.tiny_config(), "cpu", torch.float32).init_random(seed=0)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (12, 25)]
    sp = SamplingParams(temperature=0.0, max_tokens=11, ignore_eos=True)
    ref = DenseStateEngine(model).generate(prompts, sp)

    class Oracle(Drafter):
        k = 3

        def propose(self, ids):
            for p, r in zip(prompts, ref):
                full = p + r
                if list(ids) == full[:len(ids)]:
                    return full[len(ids):len(ids) + self.k]
            return []

    class HalfWrong(Oracle):
        def propose(self, ids):
            d = super().propose(ids)
            return d[:1] + [(t + 1) % 1000 for t in d[1:]]
    for drafter, lo, hi in ((Oracle(), 0.99, 1.0), (HalfWrong(), 0.2, 0.6), (NgramDrafter(), 0.0, 1.0)):
        eng = DenseStateEngine(model)
        rids = [eng.add_request(p, sp) for p in prompts]
        outs = {r: [] for r in rids}
        steps = 0
        while eng.has_work():
            for o in eng.speculative_step(drafter):
                outs[o.request_id].extend(o.new_token_ids)
            steps += 1
        assert [outs[r] for r in rids] == ref
        st = eng.spec_stats
        if st["proposed"]:
            assert lo <= st["accepted"] / st["proposed"] <= hi
        if isinstance(drafter, Oracle) and not isinstance(drafter, HalfWrong):
            assert steps <= 1 + 4          # one prompt step, then ceil(10 / 4) + 1 verifications


def test_fp8_kv_pages_write_rule_and_engine_tokens():
    """The scaled page write on the CPU restatement: a page's scale is the largest magnitude
    it has seen / 448, rows written earlier are re-encoded when it grows, a row at offset 0
    starts the page afresh; then an engine with E4M3 pages gives (nearly) the tokens of the
    bf16-page engine and its hand-off carries floating-point pages."""
    from uniserve_v1_b200.ops import reference as R
    page, Hkv, D = 4, 2, 8
    kc = torch.zeros(3, page, Hkv, D, dtype=torch.uint8)
    vc = torch.zeros_like(kc)
    ks, vs = torch.zeros(3), torch.zeros(3)
    g = torch.Generator().manual_seed(0)
    k1 = torch.randn(2, Hkv, D, generator=g)
    R.kv_write_scaled(kc, vc, ks, vs, k1, k1 * 2, torch.tensor([4, 5]))          # page 1, rows 0-1
    assert float(ks[1]) == pytest.approx(float(k1.abs().max()) / 448.0)
    assert float(vs[1]) == pytest.approx(float(k1.abs().max()) * 2 / 448.0)
    big = torch.randn(1, Hkv, D, generator=g) * 10
    R.kv_write_scaled(kc, vc, ks, vs, big, big, torch.tensor([6]))               # grows the scale
    assert float(ks[1]) == pytest.approx(float(big.abs().max()) / 448.0)
    back = R.kv_dequant(kc, ks)[1]
    assert torch.allclose(back[2], big[0], rtol=0.07, atol=float(ks[1]))
    assert torch.allclose(back[:2], k1, rtol=0.07, atol=float(ks[1]) * 2)        # re-encoded rows
    small = torch.randn(1, Hkv, D, generator=g) * 0.01
    R.kv_write_scaled(kc, vc, ks, vs, small, small, torch.tensor([4]))           # offset 0: afresh
    assert float(ks[1]) == pytest.approx(float(small.abs().max()) / 448.0)
    assert float(ks[0]) == 0.0 and float(ks[2]) == 0.0

    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.handoff import export_request, import_request
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    cfg = Qwen3MoeConfig.tiny()
    prompts = [[(5 * i + j) % cfg.vocab_size for i in range(n)] for j, n in enumerate((21, 9, 40))]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    outs = {}
    for kv in (None, "fp8"):
        model = Qwen3MoeModel(cfg, "cpu", torch.float32).init_random(seed=0)
        eng = LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=128, use_graphs=False,
                        max_num_batched_tokens=16, kv_dtype=kv)            # chunked prefill too
        outs[kv] = eng.generate(prompts, sp)
        if kv == "fp8":
            assert eng.runner.kv_caches[0][0].dtype == torch.uint8
            rid = eng.add_request(prompts[0], SamplingParams(temperature=0.0, max_tokens=6,
                                                             ignore_eos=True))
            while eng.scheduler.requests[rid].num_computed < len(prompts[0]):
                eng.step()
            h = export_request(eng, rid)
            assert h.kv[0][0].dtype == torch.bfloat16
            model2 = Qwen3MoeModel(cfg, "cpu", torch.float32).init_random(seed=0)
            eng2 = LLMEngine(model2, num_pages=64, max_num_seqs=4, max_model_len=128,
                             use_graphs=False, kv_dtype="fp8")
            import_request(eng2, [h])
            done = []
            while eng2.has_work():
                done += [o for o in eng2.step() if o.finished]
            assert done and len(eng2.scheduler.requests) >= 0
    same = sum(a == b for x, y in zip(outs[None], outs["fp8"]) for a, b in zip(x, y))
    total = sum(len(x) for x in outs[None])
    assert same >= 0.7 * total, (outs[None], outs["fp8"])


def test_decode_steps_in_flight_give_the_same_tokens():
    """Two-turn decode (the next step is issued before the last one is read) against plain
    stepping: requests that stop at different lengths, one aborted while steps are in
    flight, one that arrives in the middle; every call returns one step's tokens."""
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    cfg = Qwen3MoeConfig.tiny()
    prompts = [[(7 * i + j) % cfg.vocab_size for i in range(n)] for j, n in enumerate((12, 30, 19, 8))]
    lens = (5, 40, 17, 26)

    def run(pipeline):
        model = Qwen3MoeModel(cfg, "cpu", torch.float32).init_random(seed=0)
        eng = LLMEngine(model, num_pages=128, max_num_seqs=8, max_model_len=128, use_graphs=False,
                        pipeline_decode=pipeline)
        eng.stream_steps = 7                      # several uploads of the step state per request
        ids = [eng.add_request(p, SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True))
               for p, n in zip(prompts[:3], lens[:3])]
        got, calls, late = {i: [] for i in ids}, 0, None
        while eng.has_work():
            outs = eng.step()
            calls += 1
            for o in outs:
                got.setdefault(o.request_id, []).extend(o.new_token_ids)
            per_call = {}
            for o in outs:
                per_call[o.request_id] = per_call.get(o.request_id, 0) + len(o.new_token_ids)
            assert all(v <= 1 for v in per_call.values())          # one step per call
            if calls == 9:
                eng.abort(ids[2])
            if calls == 12:
                late = eng.add_request(prompts[3], SamplingParams(temperature=0.0, max_tokens=lens[3],
                                                                  ignore_eos=True))
        return [got[i] for i in ids] + [got[late]], calls, eng
    plain, calls_plain, eng0 = run(False)
    piped, calls_piped, eng = run(True)
    assert plain[0] == piped[0] and plain[1] == piped[1] and plain[3] == piped[3]
    assert len(plain[0]) == 5 and len(plain[1]) == 40 and len(plain[3]) == 26
    n = min(len(plain[2]), len(piped[2]))
    assert n >= 5 and plain[2][:n] == piped[2][:n]                  # the aborted one, up to the abort
    assert eng._stream is None and eng.blocks.num_free == eng0.blocks.num_free   # no page leaked


@pytest.mark.parametrize("kv_dtype", ["auto", "fp8_e4m3"])
def test_prefix_cache_outlives_the_engine_through_a_file(tmp_path, kv_dtype):
    """An engine writes its content-keyed pages to a file, a second engine of the same model
    reads them: prompts the first one computed are cache hits on the second and produce the
    same tokens; a file of another page size or model is refused; pages beyond the reader's
    free pool are dropped oldest first."""
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.prefix_store import load_prefix_cache, save_prefix_cache
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    import dataclasses
    cfg = Qwen3MoeConfig.tiny()
    if kv_dtype != "auto":
        cfg = dataclasses.replace(cfg, head_dim=128)
    model = Qwen3MoeModel(cfg, "cpu", torch.float32).init_random(seed=0)
    extra = {} if kv_dtype == "auto" else {"kv_dtype": kv_dtype}

    def engine(pages=64, page_size=16):
        return LLMEngine(model, num_pages=pages, page_size=page_size, max_num_seqs=4,
                         max_model_len=256, use_graphs=False, **extra)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (70, 40)]
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    a = engine()
    first = a.generate(prompts, sp)
    want = a.generate(prompts, sp)       # through the cached pages (E4M3 pages round the keys)
    if kv_dtype == "auto":
        assert want == first
    path = str(tmp_path / "prefix.kv")
    saved = save_prefix_cache(a, path)
    assert saved["pages"] >= 6 and os.path.getsize(path) == saved["bytes"]

    b = engine()
    got = load_prefix_cache(b, path, remove=False)
    assert got["pages"] == saved["pages"] and got["dropped"] == 0
    hits0 = b.blocks.stats()["hits"]
    assert b.generate(prompts, sp) == want
    assert b.blocks.stats()["hits"] - hits0 >= 6          # the prompts' full pages were found
    assert b.scheduler.stats["prefill_tokens"] < sum(len(p) for p in prompts) // 2

    assert "page_size" in load_prefix_cache(engine(page_size=8), path, remove=False)["refused"]
    other = Qwen3MoeModel(cfg, "cpu", torch.float32).init_random(seed=1)
    if a.blocks.identity != LLMEngine(other, num_pages=16, use_graphs=False).blocks.identity:
        e2 = LLMEngine(other, num_pages=64, max_num_seqs=4, max_model_len=256, use_graphs=False,
                       **extra)
        assert "identity" in load_prefix_cache(e2, path, remove=False)["refused"]
    small = engine(pages=5)                                # room for three pages
    few = load_prefix_cache(small, path, remove=True)
    assert 0 < few["pages"] <= 4 and few["dropped"] == saved["pages"] - few["pages"]
    assert not os.path.exists(path)
    with open(path, "wb") as f:
        f.write(b"not a cache file")
    assert load_prefix_cache(engine(), path)["refused"] == "not a prefix-cache file"


def test_persistent_decode_partition_covers_every_tile_and_names_its_partials():
    """The work partition of the persistent decode-attention kernel, restated on the host and
    enumerated over random batches: every tile of every (sequence, kv head) pair is in exactly
    one segment, a range has at most two partial segments (its first and its last), and the
    slots a merging CTA derives from the partition alone are the slots the partial segments
    were written to, one arrival per range the pair spans."""
    import random
    from uniserve_v1_b200.ops import reference as R
    rng = random.Random(7)
    for _ in range(400):
        B, Hkv = rng.randint(1, 40), rng.choice([1, 2, 4, 8])
        lens = [rng.choice([0, 1, 100, 128, 129, 500, 1100, 4000, rng.randint(0, 3000)])
                for _ in range(B)]
        n = rng.choice([1, 2, 7, 148])
        ranges = R.persist_segments(lens, Hkv, n)
        tiles = [(l + 127) // 128 for l in lens]
        seen, partial = {}, {}
        for c, segs in enumerate(ranges):
            assert segs, "no range is empty"
            assert sum(1 for s in segs if not s[4]) <= 2
            for k, (b, hk, t0, count, whole, slot) in enumerate(segs):
                for t in range(t0, t0 + count):
                    assert (b, hk, t) not in seen
                    seen[(b, hk, t)] = c
                if not whole:
                    assert k in (0, len(segs) - 1) and slot == (0 if k == 0 else 1)
                    partial.setdefault((b, hk), []).append((c, slot))
        assert len(seen) == Hkv * sum(tiles)
        for (b, hk), written in partial.items():
            assert R.persist_merge_slots(lens, Hkv, n, b, hk) == sorted(written)
            assert len(written) >= 2


def test_expert_load_counts_every_live_route():
    """While the expert load is lent, every forward adds each token's routes to its layer's
    counters: prompt tokens and generated tokens, k routes each; nothing is counted before it
    is lent or after it is taken back, and the tokens are the same either way."""
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    cfg = Qwen3MoeConfig.tiny()
    model = Qwen3MoeModel(cfg, "cpu", torch.float32).init_random(seed=0)
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    prompts = [[1, 2, 3, 4, 5, 6, 7], [9, 8, 7]]

    def run():
        return LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=64,
                         use_graphs=False, enable_prefix_cache=False).generate(prompts, sp)
    want = run()
    assert model.expert_load_snapshot() == {}
    model.enable_expert_load()
    assert run() == want
    snap = model.expert_load_snapshot()
    forwards = sum(len(p) for p in prompts) + len(prompts) * (sp.max_tokens - 1)
    routed = [i for i, lw in enumerate(model.layers) if not lw.dense]
    assert sorted(snap) == routed and routed
    for row in snap.values():
        assert len(row) == cfg.num_experts and sum(row) == forwards * cfg.num_experts_per_tok
    model.enable_expert_load(False)
    assert run() == want and model.expert_load_snapshot() == {}
