"""Qwen4-exp building blocks against their own definitions."""
import torch

from uniserve_v1_b200.models.qwen4_exp import HyperConnection, NgramEmbedding, PleLayer, ngram_ids


def test_hyper_connection_reduces_to_a_plain_residual_and_defers_its_combine():
    g = torch.Generator().manual_seed(0)
    plain = HyperConnection(hidden=16, streams=1, rank=4)           # all-zero gates
    S = torch.randn(5, 16, generator=g)
    _, h, logits = plain.read(S)
    sn = S * torch.rsqrt(S.pow(2).mean(-1, keepdim=True) + 1e-6)
    torch.testing.assert_close(h, 0.5 * sn)                          # sigmoid(0) = 1 / 2
    y = torch.randn(5, 16, generator=g)
    torch.testing.assert_close(HyperConnection.fold(S, y, logits, 1), S + y)   # gain 2 * 1 / 2
    hc = HyperConnection(hidden=8, streams=3, rank=4).init_random(1, 0.3)
    S = torch.randn(6, 24, generator=g)
    y = torch.randn(6, 8, generator=g)
    S0, h0, r0 = hc.read(S)
    nxt = HyperConnection(hidden=8, streams=3, rank=4).init_random(2, 0.3)
    S1, h1, _ = nxt.read(S0, pending=(y, r0))                        # deferred combine
    want = S.view(6, 3, 8) + y[:, None, :] * (2 * torch.sigmoid(r0 / 3))[:, :, None]
    torch.testing.assert_close(S1, want.view(6, 24))
    torch.testing.assert_close(h1, nxt.read(want.view(6, 24))[1])
    tail = HyperConnection(hidden=8, streams=3, rank=4, injects=False).init_random(3)
    assert tail.read(S)[2] is None and tail.down.shape == (4, 24)


def test_ngram_ids_match_wrapping_integer_arithmetic():
    mult = torch.tensor([0x9E3779B97F4A7C15 - (1 << 64), 0x2545F4914F6CDD1D, 0x632BE59BD9B4E019],
                        dtype=torch.int64)
    parts = torch.tensor([1009, 2003, 3001, 4001], dtype=torch.int64)
    offs = torch.tensor([0, 1009, 3012, 6013], dtype=torch.int64)
    eos = 7
    toks = torch.tensor([5, 9, 7, 11, 13, 2], dtype=torch.int64)
    ids = ngram_ids(toks, eos, mult, parts, offs, heads_per_ngram=2)
    assert ids.shape == (6, 4)
    M = [(int(m) + (1 << 64)) % (1 << 64) for m in mult]

    def signed(x):
        x %= 1 << 64
        return x - (1 << 64) if x >= (1 << 63) else x
    for t in range(6):
        prev, stopped = [], False
        for k in (1, 2):
            p = int(toks[t - k]) if t - k >= 0 else eos
            stopped = stopped or p == eos
            prev.append(eos if stopped else p)
        mix = (int(toks[t]) * M[0]) % (1 << 64)
        for k in (1, 2):
            mix ^= (prev[k - 1] * M[k]) % (1 << 64)
            for h in range((k - 1) * 2, k * 2):
                assert int(ids[t, h]) == signed(mix) % int(parts[h]) + int(offs[h]), (t, h)
    assert bool(((ids >= offs) & (ids < offs + parts)).all())
    table = (torch.randn(10100, 8, generator=torch.Generator().manual_seed(1)) * 2).to(
        torch.float8_e4m3fn).view(torch.uint8)
    emb = NgramEmbedding(table, 0.5, eos, mult, parts, offs, 2)
    e = emb.forward(toks, torch.float32)
    assert e.shape == (6, 32)
    torch.testing.assert_close(e[3, :8], table.view(torch.float8_e4m3fn)[ids[3, 0]].float() * 0.5)


def test_ple_layer_is_causal_and_carries_its_convolution_state():
    g = torch.Generator().manual_seed(2)
    ple = PleLayer(hidden=8, streams=2, embed=12, kernel=3, dilation=2).init_random(0, 0.3)
    e, S = torch.randn(9, 12, generator=g), torch.randn(9, 16, generator=g)
    out, st = ple.forward(e, S)
    assert out.shape == (9, 16) and st.shape == (4, 16)
    e2, S2 = e.clone(), S.clone()
    e2[6:], S2[6:] = 0.0, 1.0                                        # later tokens change
    torch.testing.assert_close(ple.forward(e2, S2)[0][:6], out[:6])
    a, sa = ple.forward(e[:4], S[:4])
    b, sb = ple.forward(e[4:], S[4:], sa)
    torch.testing.assert_close(torch.cat([a, b]), out)
    torch.testing.assert_close(sb, st)


def _dense_gated(att, x, mask):
    """Causal gated attention of the same weights over the tokens ``mask`` [T, T] allows."""
    from uniserve_v1_b200.models.qwen4_exp import gemma_norm, partial_rope
    T, H, hd = x.shape[0], att.heads, att.hd
    pos = torch.arange(T)
    qg = (x @ att.q_proj.t()).view(T, H, 2, hd)
    q = partial_rope(gemma_norm(qg[:, :, 0], att.q_norm, att.eps), pos, att.rot, att.theta)
    k = partial_rope(gemma_norm((x @ att.k_proj.t()).view(T, att.kv, hd), att.k_norm, att.eps),
                     pos, att.rot, att.theta).repeat_interleave(H // att.kv, 1)
    v = (x @ att.v_proj.t()).view(T, att.kv, hd).repeat_interleave(H // att.kv, 1)
    sc = torch.einsum("thd,shd->hts", q, k) * hd ** -0.5
    sc = sc.masked_fill(~mask[None], float("-inf"))
    o = torch.einsum("hts,shd->thd", torch.softmax(sc, -1), v) * torch.sigmoid(qg[:, :, 1])
    return o.reshape(T, H * hd) @ att.o_proj.t()


def test_indexed_attention_selects_groups_and_matches_masked_attention():
    from uniserve_v1_b200.models.qwen4_exp import IndexedAttention
    g = torch.Generator().manual_seed(3)
    T = 23
    x = torch.randn(T, 32, generator=g)
    kw = dict(hidden=32, heads=4, kv_heads=2, head_dim=16, index_heads=2, index_dim=8, ratio=4,
              rotary_dim=8)
    wide = IndexedAttention(budget=24, **kw).init_random(0)          # every group fits
    out, cache, sel = wide.forward(x)
    assert sel.shape == (T, 24 + 3) and cache["k"].shape == (T, 2, 16)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    torch.testing.assert_close(out, _dense_gated(wide, x, causal), rtol=1e-4, atol=1e-5)
    for t in range(T):                                               # what a row names
        row = sel[t][sel[t] >= 0].tolist()
        assert sorted(row) == list(range(t + 1))
        assert row[len(row) - (t + 1) % 4:] == list(range((t + 1) // 4 * 4, t + 1))
    narrow = IndexedAttention(budget=8, **kw).init_random(0)         # two groups of the visible
    out2, _, sel2 = narrow.forward(x)
    mask = torch.zeros(T, T, dtype=torch.bool)
    for t in range(T):
        row = sel2[t][sel2[t] >= 0]
        assert len(set(row.tolist())) == len(row) and int(row.max()) <= t
        assert len(row) == min((t + 1) // 4, 2) * 4 + (t + 1) % 4
        mask[t, row] = True
    torch.testing.assert_close(out2, _dense_gated(narrow, x, mask), rtol=1e-4, atol=1e-5)
    assert not torch.allclose(out2[12:], out[12:], atol=1e-4)        # the budget binds
    keys = narrow.index_keys(cache["raw"])                           # rank order by score
    s = torch.relu(torch.einsum("hd,gd->hg", _q_idx(narrow, x)[T - 1], keys)).sum(0)[:(T) // 4]
    assert sel2[T - 1, :8:4].tolist() == (s.topk(2).indices * 4).tolist()
    a, c, sa = narrow.forward(x[:10])                                # a prompt in pieces
    b, c, sb = narrow.forward(x[10:], c)
    torch.testing.assert_close(torch.cat([a, b]), out2, rtol=1e-4, atol=1e-5)
    assert torch.equal(torch.cat([sa, sb]), sel2)


def _q_idx(att, x):
    from uniserve_v1_b200.models.qwen4_exp import gemma_norm, partial_rope
    iq = (x @ att.index_qk_proj.t()).view(x.shape[0], att.ih + 1, att.idim)
    return partial_rope(gemma_norm(iq[:, :att.ih], att.q_layernorm, att.eps),
                        torch.arange(x.shape[0]), att.irot, att.theta)


def test_qwen4_decoder_runs_a_prompt_in_pieces_and_is_causal():
    from uniserve_v1_b200.models.qwen3_5 import Qwen35MoeModel
    from uniserve_v1_b200.models.qwen4_exp import Qwen4ExpModel
    mult = torch.tensor([0x9E3779B97F4A7C15 - (1 << 64), 0x2545F4914F6CDD1D], dtype=torch.int64)
    parts, offs = torch.tensor([211, 307], dtype=torch.int64), torch.tensor([0, 211])
    table = torch.randn(518, 6, generator=torch.Generator().manual_seed(5)).to(
        torch.float8_e4m3fn).view(torch.uint8)
    cfg = Qwen35MoeModel.tiny_config()
    ngram = NgramEmbedding(table, 0.25, cfg.eos_token_id, mult, parts, offs, 2)
    model = Qwen4ExpModel(cfg, streams=2, ple_layers=(0, 3), ngram=ngram).init_random(0)
    assert [("self_attn" in L) for L in model.layers] == [False, False, False, True]
    ids = torch.randint(0, 1000, (21,), generator=torch.Generator().manual_seed(6))
    whole = model.forward(ids, model.new_state())
    assert whole.shape == (21, cfg.vocab_size) and bool(torch.isfinite(whole).all())
    st = model.new_state()
    pieces = torch.cat([model.forward(ids[:7], st), model.forward(ids[7:8], st),
                        model.forward(ids[8:], st)])
    torch.testing.assert_close(pieces, whole, rtol=2e-3, atol=2e-4)
    other = ids.clone()
    other[15:] = 3
    torch.testing.assert_close(model.forward(other, model.new_state())[:15], whole[:15],
                               rtol=2e-3, atol=2e-4)
    tri = torch.tensor([0x9E3779B97F4A7C15 - (1 << 64), 0x2545F4914F6CDD1D, 0x632BE59BD9B4E019],
                       dtype=torch.int64)                     # 3-grams: the window reaches two back
    ngram3 = NgramEmbedding(table, 0.25, cfg.eos_token_id, tri, torch.tensor([211, 307]),
                            torch.tensor([0, 211]), 1)
    m3 = Qwen4ExpModel(cfg, streams=2, ple_layers=(1,), ngram=ngram3).init_random(2)
    assert m3.layers[1]["ple"].dil == 3
    w3, st = m3.forward(ids, m3.new_state()), m3.new_state()
    p3 = torch.cat([m3.forward(ids[:1], st), m3.forward(ids[1:2], st), m3.forward(ids[2:9], st),
                    m3.forward(ids[9:], st)])
    torch.testing.assert_close(p3, w3, rtol=2e-3, atol=2e-4)
    out = model.generate(ids.tolist(), 5)
    assert out == model.generate(ids.tolist(), 5) and len(out) == 5
    assert out[0] == int(whole[-1].argmax())


def test_qwen4_decoder_serves_through_the_dense_state_engine():
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_5 import Qwen35MoeModel
    from uniserve_v1_b200.models.qwen4_exp import Qwen4ExpModel
    cfg = Qwen35MoeModel.tiny_config()
    mult = torch.tensor([0x9E3779B97F4A7C15 - (1 << 64), 0x2545F4914F6CDD1D], dtype=torch.int64)
    table = torch.randn(518, 6, generator=torch.Generator().manual_seed(5)).to(
        torch.float8_e4m3fn).view(torch.uint8)
    ngram = NgramEmbedding(table, 0.25, cfg.eos_token_id, mult,
                           torch.tensor([211, 307]), torch.tensor([0, 211]), 2)
    model = Qwen4ExpModel(cfg, ple_layers=(1,), ngram=ngram).init_random(1)
    g = torch.Generator().manual_seed(7)
    shared = torch.randint(0, 1000, (40,), generator=g).tolist()
    prompts = [shared + torch.randint(0, 1000, (n,), generator=g).tolist() for n in (5, 11, 3)]
    want = [model.generate(p, 6) for p in prompts]
    eng = DenseStateEngine(model, max_num_seqs=2, prefill_chunk=16, state_interval=8)
    p = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    ids = [eng.add_request(q, p) for q in prompts]
    got = {i: [] for i in ids}
    for _ in range(200):
        for o in eng.step():
            got[o.request_id] += o.new_token_ids
        if not eng.running and not eng.waiting:
            break
    for i, w in zip(ids, want):
        assert got[i][:len(w)] == w, (got[i], w)
    assert eng._stats["cached_tokens"] >= 32                         # the third began from a snapshot


def test_qwen4_decoder_answers_chat_requests():
    from fastapi.testclient import TestClient
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.models.qwen4_exp import Qwen4ExpModel
    from uniserve_v1_b200.server.app import create_app
    from uniserve_v1_b200.config.policy import Package
    from uniserve_v1_b200.server.tokenizer import ByteTokenizer
    model = Qwen4ExpModel.tiny()
    eng = DenseStateEngine(model, max_num_seqs=4, max_model_len=256)
    pkg = Package.parse('model = "random:qwen4_exp:tiny"\nserved_model_name = "q4"\n')
    app = create_app(package=pkg, engine=eng, tokenizer=ByteTokenizer(1024, 1023),
                     served_model_name="q4")
    with TestClient(app) as c:
        body = {"model": "q4", "messages": [{"role": "user", "content": "hello"}],
                "max_tokens": 5, "temperature": 0, "ignore_eos": True}
        a = c.post("/v1/chat/completions", json=body).json()
        b = c.post("/v1/chat/completions", json=body).json()
        assert a["choices"][0]["message"] == b["choices"][0]["message"]
        assert a["usage"]["completion_tokens"] == 5


def test_qwen4_speculative_steps_replay_every_kind_of_state():
    """A refused draft restores the delta-rule matrices, the convolution windows of the PLE
    layers, the attention's keys, values and raw index keys and the token history."""
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.engine.speculation import Drafter
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen4_exp import Qwen4ExpModel
    model = Qwen4ExpModel.tiny(3)
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (9, 14)]
    want = [model.generate(p, 9) for p in prompts]

    class Oracle(Drafter):
        k = 3

        def propose(self, ids):
            for p, w in zip(prompts, want):
                if ids[:len(p)] == p:
                    done = len(ids) - len(p)
                    return w[done:done + 3]
            return []

    class HalfRight(Oracle):
        def propose(self, ids):
            d = super().propose(ids)
            return d[:1] + [(t + 1) % 1000 for t in d[1:]]

    sp = SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True)
    for drafter in (Oracle(), HalfRight()):
        eng = DenseStateEngine(model, max_num_seqs=4, state_cache_entries=0)
        ids = [eng.add_request(p, sp) for p in prompts]
        got = {i: [] for i in ids}
        for _ in range(100):
            for o in eng.speculative_step(drafter):
                got[o.request_id] += o.new_token_ids
            if not eng.running and not eng.waiting:
                break
        assert [got[i] for i in ids] == [w[:9] for w in want]
        st = eng.spec_stats
        assert st["proposed"] > 0
        if isinstance(drafter, HalfRight):
            assert 0 < st["accepted"] < st["proposed"]
        else:
            assert st["accepted"] == st["proposed"]


def test_qwen4_mtp_entries_in_pieces_and_chained_drafts_leave_the_cache_as_it_was():
    from uniserve_v1_b200.models.qwen4_exp import Qwen4ExpModel, Qwen4Mtp
    model = Qwen4ExpModel.tiny(1)
    mtp = Qwen4Mtp(model).init_random(4)
    ids = torch.randint(0, 1000, (18,), generator=torch.Generator().manual_seed(2))
    logits, S = model.forward(ids, model.new_state(), return_streams=True)
    assert S.shape == (18, model.C * model.cfg.hidden_size)
    nxt = torch.cat([ids[1:], logits[-1].argmax()[None]])            # the token after each position
    st = mtp.new_state()
    S1, d = mtp.observe(S, nxt, st)
    assert d.shape == (18, model.cfg.vocab_size) and bool(torch.isfinite(d).all())
    st2 = mtp.new_state()
    a = mtp.observe(S[:7], nxt[:7], st2)
    b = mtp.observe(S[7:], nxt[7:], st2)
    torch.testing.assert_close(torch.cat([a[1], b[1]]), d, rtol=2e-3, atol=2e-4)
    torch.testing.assert_close(torch.cat([a[0], b[0]]), S1, rtol=2e-3, atol=2e-4)
    other = nxt.clone()
    other[12:] = 5                                                    # causal in its entries
    torch.testing.assert_close(mtp.observe(S, other, mtp.new_state())[1][:12], d[:12],
                               rtol=2e-3, atol=2e-4)
    before = {n: t.clone() for n, t in st["attn"].items()}
    drafts = mtp.draft(S1[-1:], d[-1], 3, st)
    assert len(drafts) == 3 and drafts[0] == int(d[-1].argmax())
    assert all(torch.equal(st["attn"][n], before[n]) for n in before)
    assert mtp.draft(S1[-1:], d[-1], 3, st) == drafts
    # the second draft is the entry chained on the drafter's own streams
    S2, d2 = mtp.forward(S1[-1:], torch.tensor(drafts[:1]), {"attn": {n: t.clone() for n, t in
                                                                   before.items()}})
    assert drafts[1] == int(d2[-1].argmax())


def test_qwen4_mtp_drafter_in_the_engine_matches_plain_decoding():
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen4_exp import Qwen4ExpModel, Qwen4Mtp, Qwen4MtpDrafter
    model = Qwen4ExpModel.tiny(5)
    g = torch.Generator().manual_seed(13)
    shared = torch.randint(0, 1000, (24,), generator=g).tolist()
    prompts = [shared + torch.randint(0, 1000, (n,), generator=g).tolist() for n in (6, 3)]
    want = [model.generate(p, 8) for p in prompts]
    drafter = Qwen4MtpDrafter(Qwen4Mtp(model).init_random(6), k=3)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    eng = DenseStateEngine(model, max_num_seqs=1, prefill_chunk=16, state_interval=8)
    ids = [eng.add_request(p, sp) for p in prompts]     # the second starts from a snapshot
    got = {i: [] for i in ids}
    for _ in range(200):
        for o in eng.speculative_step(drafter):
            got[o.request_id] += o.new_token_ids
        if not eng.running and not eng.waiting:
            break
    assert [got[i][:len(w)] for i, w in zip(ids, want)] == want
    assert eng.spec_stats["proposed"] >= 3 * 4 and eng._stats["cached_tokens"] >= 16
    # the cache the drafter keeps in a request's state holds the committed positions only
    st = model.new_state()
    model.forward(torch.tensor(prompts[0]), st)
    assert st["mtp"]["attn"]["k"].shape[0] == len(prompts[0]) - 1
    d1 = drafter.propose_from_state(prompts[0] + [7], st)
    assert len(d1) == 3 and st["mtp"]["attn"]["k"].shape[0] == len(prompts[0]) - 1
    assert drafter.propose_from_state(prompts[0] + [7], st) == d1
    model.tap = None


def test_qwen4_checkpoint_round_trip(tmp_path):
    import json
    from uniserve_v1_b200.checkpoint.safetensors_io import (CheckpointLoader, resolve_family,
                                                            save_file)
    from uniserve_v1_b200.models.qwen4_exp import Qwen4ExpModel
    model = Qwen4ExpModel.tiny(7)
    tensors = model.export_state()
    assert "model.language_model.layers.0.attn_hyper_connection.block_inject_weight.weight" in tensors
    assert "model.language_model.layers.3.self_attn.indexer.index_qk_proj.weight" in tensors
    assert tensors["model.language_model.layers.0.ple.ple_embedding.ngram_embedding.shard_0.weight"
                   ].dtype == torch.float8_e4m3fn
    assert "model.language_model.hyper_connection_mixer.block_inject_weight.weight" not in tensors
    names = sorted(tensors)
    save_file({n: tensors[n] for n in names[::2]}, tmp_path / "model-00001-of-00002.safetensors")
    save_file({n: tensors[n] for n in names[1::2]}, tmp_path / "model-00002-of-00002.safetensors")
    (tmp_path / "config.json").write_text(json.dumps(model.hf_config()))
    assert resolve_family(tmp_path) == "qwen4_exp"
    again = Qwen4ExpModel.from_checkpoint(CheckpointLoader(tmp_path))
    assert again.C == model.C and again.ple_layers == model.ple_layers
    assert [("self_attn" in L, "ple" in L) for L in again.layers] == \
        [("self_attn" in L, "ple" in L) for L in model.layers]
    ids = torch.randint(0, 1000, (19,), generator=torch.Generator().manual_seed(3))
    torch.testing.assert_close(again.forward(ids, again.new_state()),
                               model.forward(ids, model.new_state()), rtol=1e-4, atol=1e-5)
    assert again.generate(ids.tolist(), 4) == model.generate(ids.tolist(), 4)
    # the checkpoint's own drafter
    from uniserve_v1_b200.models.qwen4_exp import Qwen4Mtp
    mtp = Qwen4Mtp(model).init_random(8)
    save_file(mtp.export_state(), tmp_path / "model-mtp.safetensors")
    ld = CheckpointLoader(tmp_path)
    assert ld.has("mtp.fc_hidden.weight") and ld.has("mtp.layers.0.self_attn.indexer.index_qk_proj.weight")
    mtp2 = Qwen4Mtp(again).load_state(ld)
    _, S = model.forward(ids, model.new_state(), return_streams=True)
    nxt = torch.roll(ids, -1)
    torch.testing.assert_close(mtp2.observe(S, nxt, mtp2.new_state())[1],
                               mtp.observe(S, nxt, mtp.new_state())[1], rtol=1e-4, atol=1e-5)


def test_hybrid_family_mtp_drafter_in_the_engine(tmp_path):
    """The hybrid (gated delta net) family drafts with its own MTP layer: same answers as plain
    decoding, the module's stream covers exactly the committed positions, batched decode steps
    keep it in step, and a checkpoint's mtp.* tensors load."""
    from uniserve_v1_b200.checkpoint.safetensors_io import CheckpointLoader, save_file
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_5 import HybridMtp, HybridMtpDrafter, Qwen35MoeModel
    model = Qwen35MoeModel(Qwen35MoeModel.tiny_config(), "cpu", torch.float32).init_random(0)
    g = torch.Generator().manual_seed(17)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (13, 7)]
    want = [model.generate(p, 8) for p in prompts]
    mtp = HybridMtp(model).init_random(3)
    drafter = HybridMtpDrafter(mtp, k=2)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    eng = DenseStateEngine(model, max_num_seqs=2, state_cache_entries=0)
    ids = [eng.add_request(p, sp) for p in prompts]
    got = {i: [] for i in ids}
    for n in range(200):
        step = eng.step if n == 2 else (lambda: eng.speculative_step(drafter))   # one batched step
        for o in step():
            got[o.request_id] += o.new_token_ids
        if not eng.running and not eng.waiting:
            break
    assert [got[i][:len(w)] for i, w in zip(ids, want)] == want
    assert eng.spec_stats["proposed"] >= 8
    st = model.new_state()
    model.forward(torch.tensor(prompts[0]), st)
    assert st.mtp["pos"] == len(prompts[0]) - 1 == st.mtp["kv"].k.shape[0]
    d = drafter.propose_from_state(prompts[0] + [5], st)
    assert len(d) == 2 and st.mtp["kv"].k.shape[0] == len(prompts[0]) - 1
    assert drafter.propose_from_state(prompts[0] + [5, 6], st) == []      # the stream is behind
    import copy
    assert copy.deepcopy(st).mtp["pos"] == st.mtp["pos"]
    # mtp.* names of a checkpoint
    L, I, S = mtp.w["layer"], model.cfg.moe_intermediate_size, model.cfg.shared_expert_intermediate_size
    t = {"mtp.fc.weight": mtp.w["fc"], "mtp.norm.weight": mtp.w["norm"] - 1,
         "mtp.pre_fc_norm_embedding.weight": mtp.w["norm_e"] - 1,
         "mtp.pre_fc_norm_hidden.weight": mtp.w["norm_h"] - 1,
         "mtp.layers.0.input_layernorm.weight": L["in_norm"] - 1,
         "mtp.layers.0.post_attention_layernorm.weight": L["post_norm"] - 1,
         "mtp.layers.0.self_attn.q_norm.weight": L["q_norm"] - 1,
         "mtp.layers.0.self_attn.k_norm.weight": L["k_norm"] - 1,
         "mtp.layers.0.mlp.gate.weight": L["router"],
         "mtp.layers.0.mlp.experts.gate_up_proj": torch.cat([L["w13"][:, I:], L["w13"][:, :I]], 1),
         "mtp.layers.0.mlp.experts.down_proj": L["w2"],
         "mtp.layers.0.mlp.shared_expert.up_proj.weight": L["s13"][:S],
         "mtp.layers.0.mlp.shared_expert.gate_proj.weight": L["s13"][S:],
         "mtp.layers.0.mlp.shared_expert.down_proj.weight": L["s2"],
         "mtp.layers.0.mlp.shared_expert_gate.weight": L["sgate"]}
    for n in "qkvo":
        t[f"mtp.layers.0.self_attn.{n}_proj.weight"] = L[n]
    save_file({k: v.contiguous() for k, v in t.items()}, tmp_path / "model.safetensors")
    (tmp_path / "config.json").write_text("{}")
    loaded = HybridMtp(model).load_state(CheckpointLoader(tmp_path))
    h = torch.randn(5, model.cfg.hidden_size, generator=g)
    from uniserve_v1_b200.models.qwen3_5 import LayerState
    a = mtp.rows(h, torch.tensor([1, 2, 3, 4, 5]), 0, LayerState())[1]
    b = loaded.rows(h, torch.tensor([1, 2, 3, 4, 5]), 0, LayerState())[1]
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    model.tap = None
