"""Golden parity with Hugging Face transformers: a tiny Qwen3-MoE (and dense Qwen3)
checkpoint written by transformers is loaded through the safetensors reader and must
reproduce transformers' own logits and greedy continuation on CPU."""
import json

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _save(model, cfg, path):
    from uniserve_v1_b200.checkpoint.safetensors_io import save_file
    path.mkdir(parents=True, exist_ok=True)
    state = {k: v.detach().clone().contiguous() for k, v in model.state_dict().items()}
    save_file(state, path / "model.safetensors")
    d = cfg.to_dict()
    d["architectures"] = [type(model).__name__]
    (path / "config.json").write_text(json.dumps(d))


def _compare(path, hf, prompt):
    from uniserve_v1_b200.checkpoint.safetensors_io import CheckpointLoader, resolve_family
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.models.reference_cpu import ReferenceQwen3Moe
    assert resolve_family(path) == "qwen3_moe"
    ld = CheckpointLoader(path)
    cfg = Qwen3MoeConfig.from_hf(ld.config)
    model = Qwen3MoeModel(cfg, "cpu", torch.float32).load_state(ld)
    ids = torch.tensor([prompt])
    with torch.no_grad():
        want = hf(ids).logits[0]
        gen = hf.generate(ids, max_new_tokens=6, do_sample=False)[0, len(prompt):].tolist()
    got, _ = ReferenceQwen3Moe(model).forward(torch.tensor(prompt))
    torch.testing.assert_close(got, want, atol=2e-4, rtol=2e-4)
    out = LLMEngine(model, num_pages=32, max_num_seqs=2, max_model_len=128,
                    use_graphs=False).generate(
        [prompt], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))[0]
    assert out == gen


def test_qwen3_moe_matches_transformers(tmp_path):
    from transformers import Qwen3MoeConfig as HfCfg, Qwen3MoeForCausalLM
    torch.manual_seed(0)
    cfg = HfCfg(vocab_size=512, hidden_size=128, intermediate_size=256, moe_intermediate_size=64,
                num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                num_experts=8, num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1,
                mlp_only_layers=[], max_position_embeddings=256, rope_theta=1e6,
                rms_norm_eps=1e-6, tie_word_embeddings=False, eos_token_id=511, pad_token_id=0,
                torch_dtype="float32", attention_dropout=0.0, router_aux_loss_coef=0.0)
    hf = Qwen3MoeForCausalLM(cfg).eval()
    _save(hf, cfg, tmp_path / "moe")
    _compare(tmp_path / "moe", hf, [3, 17, 250, 4, 99, 100, 7, 7, 12])


def test_qwen3_dense_matches_transformers(tmp_path):
    from transformers import Qwen3Config as HfCfg, Qwen3ForCausalLM
    torch.manual_seed(1)
    cfg = HfCfg(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                max_position_embeddings=256, rope_theta=1e6, rms_norm_eps=1e-6,
                tie_word_embeddings=True, eos_token_id=511, pad_token_id=0, torch_dtype="float32",
                attention_dropout=0.0)
    hf = Qwen3ForCausalLM(cfg).eval()
    _save(hf, cfg, tmp_path / "dense")
    _compare(tmp_path / "dense", hf, [5, 9, 2, 44, 300, 12])


def test_qwen3_5_moe_hybrid_decoder_matches_transformers(tmp_path):
    """Gated-delta-net layers, gated attention with partial rotary embedding, experts plus
    a gated shared expert: logits of a tiny random `Qwen3_5MoeForCausalLM` checkpoint, for the
    whole prompt at once and for the same prompt run in chunks and then token by token."""
    import json
    import pytest
    import torch
    tr = pytest.importorskip("transformers")
    from transformers.models.qwen3_5_moe.configuration_qwen3_5_moe import Qwen3_5MoeTextConfig
    from transformers.models.qwen3_5_moe.modeling_qwen3_5_moe import Qwen3_5MoeForCausalLM
    from uniserve_v1_b200.checkpoint.safetensors_io import CheckpointLoader, save_file
    from uniserve_v1_b200.models.qwen3_5 import Qwen35Config, Qwen35MoeModel
    hf_cfg = Qwen3_5MoeTextConfig(
        vocab_size=300, hidden_size=64, num_hidden_layers=4, num_attention_heads=4,
        num_key_value_heads=2, head_dim=32, linear_num_key_heads=2, linear_num_value_heads=4,
        linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4,
        num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32,
        shared_expert_intermediate_size=48, max_position_embeddings=256,
        layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"])
    torch.manual_seed(0)
    hf = Qwen3_5MoeForCausalLM(hf_cfg).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():                   # norms and gates away from their init
            if p.dim() == 1 or "experts" in n:
                p.copy_(torch.randn_like(p) * 0.3)
    state = {k: v.detach().clone().contiguous() for k, v in hf.state_dict().items()}
    save_file(state, tmp_path / "model.safetensors")
    (tmp_path / "config.json").write_text(json.dumps(hf_cfg.to_dict()))
    ld = CheckpointLoader(tmp_path)
    cfg = Qwen35Config.from_hf(ld.config)
    assert cfg.layer_types[3] == "full_attention" and cfg.partial_rotary_factor == 0.25
    model = Qwen35MoeModel(cfg, "cpu", torch.float32).load_state(ld)
    ids = torch.randint(0, 300, (19,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(ids[None]).logits[0]
    got = model.forward(ids, model.new_state())
    torch.testing.assert_close(got, want, atol=2e-4, rtol=2e-3)
    st = model.new_state()
    parts = [model.forward(ids[:7], st, 0), model.forward(ids[7:15], st, 7)]
    parts += [model.forward(ids[i:i + 1], st, i) for i in range(15, 19)]
    torch.testing.assert_close(torch.cat(parts), want, atol=2e-4, rtol=2e-3)
    with torch.no_grad():
        ref_gen = hf.generate(ids[None], max_new_tokens=6, do_sample=False)[0, 19:].tolist()
    assert model.generate(ids.tolist(), 6, chunk=8)[:len(ref_gen)] == ref_gen


def test_qwen3_vl_vision_tower_matches_transformers(tmp_path):
    """Patch embedding, interpolated position grid, 2-D rotary attention per frame, merger
    and deep-stack mergers of a tiny random `Qwen3VLVisionModel`, for an image and a
    two-frame video of different sizes in one call; and the splice into text rows."""
    import pytest
    import torch
    pytest.importorskip("transformers")
    from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLVisionConfig
    from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLVisionModel
    from uniserve_v1_b200.checkpoint.safetensors_io import CheckpointLoader, save_file
    from uniserve_v1_b200.models.qwen3_vl_vision import Qwen3VLVisionTower, VisionConfig, splice
    hf_cfg = Qwen3VLVisionConfig(depth=3, hidden_size=64, intermediate_size=96, num_heads=2,
                                 in_channels=3, patch_size=4, temporal_patch_size=2,
                                 spatial_merge_size=2, out_hidden_size=48,
                                 num_position_embeddings=36, deepstack_visual_indexes=[0, 2])
    torch.manual_seed(0)
    hf = Qwen3VLVisionModel(hf_cfg).float().eval()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() == 1:
                p.copy_(torch.randn_like(p) * 0.2 + (1.0 if p.abs().mean() > 0.5 else 0.0))
    save_file({"model.visual." + k: v.detach().clone().contiguous()
               for k, v in hf.state_dict().items()}, tmp_path / "model.safetensors")
    (tmp_path / "config.json").write_text("{}")
    cfg = VisionConfig.from_hf(hf_cfg.to_dict())
    tower = Qwen3VLVisionTower(cfg, "cpu", torch.float32).load_state(CheckpointLoader(tmp_path))
    grids = [(1, 4, 6), (2, 6, 4)]
    n = sum(t * h * w for t, h, w in grids)
    pixels = torch.randn(n, 3 * 2 * 4 * 4, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf(pixels, grid_thw=torch.tensor(grids))
    rows, deep = tower.forward(pixels, grids)
    torch.testing.assert_close(rows, ref.pooler_output, atol=2e-4, rtol=2e-3)
    assert len(deep) == 2
    for a, b in zip(deep, ref.deepstack_features):
        torch.testing.assert_close(a, b, atol=2e-4, rtol=2e-3)
    assert rows.shape == (n // 4, 48)
    ids = torch.tensor([1, 9, 9, 2] + [9] * (n // 4 - 2) + [3])
    emb = torch.zeros(ids.numel(), 48)
    out = splice(emb, ids, 9, rows)
    assert torch.equal(out[1], rows[0]) and torch.equal(out[-2], rows[-1]) and out[0].abs().sum() == 0
    with pytest.raises(ValueError):
        splice(emb, ids[:-3], 9, rows)


def test_dense_state_engine_serves_the_hybrid_decoder(tmp_path):
    """Continuous batching over per-sequence states: requests that arrive at different
    steps and read their prompts in chunks produce what each produces alone."""
    import json
    import pytest
    import torch
    pytest.importorskip("transformers")
    from transformers.models.qwen3_5_moe.configuration_qwen3_5_moe import Qwen3_5MoeTextConfig
    from transformers.models.qwen3_5_moe.modeling_qwen3_5_moe import Qwen3_5MoeForCausalLM
    from uniserve_v1_b200.checkpoint.safetensors_io import CheckpointLoader, save_file
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_5 import Qwen35Config, Qwen35MoeModel
    hf_cfg = Qwen3_5MoeTextConfig(
        vocab_size=200, hidden_size=32, num_hidden_layers=2, num_attention_heads=2,
        num_key_value_heads=1, head_dim=16, linear_num_key_heads=1, linear_num_value_heads=2,
        linear_key_head_dim=8, linear_value_head_dim=8, num_experts=4, num_experts_per_tok=2,
        moe_intermediate_size=16, shared_expert_intermediate_size=16, max_position_embeddings=128,
        layer_types=["linear_attention", "full_attention"], eos_token_id=199)
    torch.manual_seed(3)
    hf = Qwen3_5MoeForCausalLM(hf_cfg).float().eval()
    save_file({k: v.detach().clone().contiguous() for k, v in hf.state_dict().items()},
              tmp_path / "model.safetensors")
    (tmp_path / "config.json").write_text(json.dumps(hf_cfg.to_dict()))
    ld = CheckpointLoader(tmp_path)
    model = Qwen35MoeModel(Qwen35Config.from_hf(ld.config), "cpu", torch.float32).load_state(ld)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 199, (n,), generator=g).tolist() for n in (5, 23, 11)]
    params = [SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True),
              SamplingParams(temperature=0.9, top_p=0.8, seed=7, max_tokens=8, ignore_eos=True),
              SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)]
    alone = [DenseStateEngine(model).generate([p], sp)[0] for p, sp in zip(prompts, params)]
    assert alone[0] == model.generate(prompts[0], 6)
    eng = DenseStateEngine(model, max_num_seqs=2, prefill_chunk=8)
    rids = [eng.add_request(prompts[0], params[0])]
    outs = {rids[0]: []}
    step = 0
    while eng.has_work() or step < 3:
        if step == 1:
            rids.append(eng.add_request(prompts[1], params[1]))
            rids.append(eng.add_request(prompts[2], params[2]))    # waits for a free state
            outs.update({rids[1]: [], rids[2]: []})
        for o in eng.step():
            outs[o.request_id].extend(o.new_token_ids)
        step += 1
    assert [outs[r] for r in rids] == alone
    assert eng.stats()["finished"] == 3 and not eng.states
    rid = eng.add_request(prompts[1], params[1])
    eng.step()
    assert eng.abort(rid) and not eng.has_work()


def test_fixture_generator_round_trip(tmp_path):
    """Fixtures written by the generator are reproduced by the package's own loaders and
    decoders (paged engine for the Qwen3 families, dense-state engine for the hybrid one)."""
    from uniserve_v1_b200.checkpoint.safetensors_io import CheckpointLoader, resolve_family
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_5 import Qwen35Config, Qwen35MoeModel
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.testing import model_fixtures as MF
    assert MF.main([str(tmp_path), "qwen3", "qwen3_5_moe"]) == 0
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    for fam in ("qwen3", "qwen3_5_moe"):
        ref = json.loads((tmp_path / fam / "reference.json").read_text())
        ld = CheckpointLoader(tmp_path / fam)
        if resolve_family(tmp_path / fam) == "qwen3_5_moe":
            model = Qwen35MoeModel(Qwen35Config.from_hf(ld.config), "cpu", torch.float32).load_state(ld)
            out = DenseStateEngine(model).generate([ref["prompt"]], sp)[0]
        else:
            model = Qwen3MoeModel(Qwen3MoeConfig.from_hf(ld.config), "cpu", torch.float32).load_state(ld)
            out = LLMEngine(model, num_pages=32, max_num_seqs=2, max_model_len=128,
                            use_graphs=False).generate([ref["prompt"]], sp)[0]
        assert out == ref["greedy"], fam


def test_decoder_as_text_encoder_matches_transformers_hidden_states(tmp_path):
    """The cache-free causal pass returns the residual stream after n blocks
    (`hidden_states[n]` of transformers); the video service's model-backed text encoder
    serves and caches those rows."""
    from transformers import Qwen3Config as HfCfg, Qwen3ForCausalLM
    from uniserve_v1_b200.checkpoint.safetensors_io import CheckpointLoader
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.server.tokenizer import ByteTokenizer
    from uniserve_v1_b200.server.video_service import ModelTextEncoder
    torch.manual_seed(2)
    cfg = HfCfg(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=3,
                num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                max_position_embeddings=256, rope_theta=1e6, rms_norm_eps=1e-6,
                tie_word_embeddings=False, eos_token_id=511, pad_token_id=0)
    hf = Qwen3ForCausalLM(cfg).float().eval()
    _save(hf, cfg, tmp_path / "enc")
    ld = CheckpointLoader(tmp_path / "enc")
    model = Qwen3MoeModel(Qwen3MoeConfig.from_hf(ld.config), "cpu", torch.float32).load_state(ld)
    ids = [5, 300, 17, 17, 450, 2, 99]
    with torch.no_grad():
        hs = hf(torch.tensor([ids]), output_hidden_states=True).hidden_states
    for n in (0, 1, 2):
        torch.testing.assert_close(model.encode(ids, n), hs[n][0], atol=2e-4, rtol=2e-4)
    # transformers reports the last entry after the final norm
    from uniserve_v1_b200.ops import reference as R
    torch.testing.assert_close(R.rmsnorm(model.encode(ids), model.final_norm, 1e-6), hs[3][0],
                               atol=2e-4, rtol=2e-4)
    enc = ModelTextEncoder(model, ByteTokenizer(512, 511), num_layers=2)
    a = enc.encode("a sunset over water", "cpu")
    assert a.shape == (len(ByteTokenizer(512, 511).encode("a sunset over water")), 64)
    assert enc.encode("a sunset over water", "cpu") is not None and len(enc.cache) == 1
    torch.testing.assert_close(a, model.encode(ByteTokenizer(512, 511).encode("a sunset over water"), 2))


def test_qwen3_5_multimodal_prompt_matches_transformers(tmp_path):
    """Image rows from the vision tower spliced at the placeholder tokens, three-axis
    interleaved rotary positions, then greedy decoding: a tiny random
    `Qwen3_5MoeForConditionalGeneration`."""
    import pytest
    pytest.importorskip("transformers")
    from transformers.models.qwen3_5_moe.configuration_qwen3_5_moe import (
        Qwen3_5MoeConfig, Qwen3_5MoeTextConfig, Qwen3_5MoeVisionConfig)
    from transformers.models.qwen3_5_moe.modeling_qwen3_5_moe import \
        Qwen3_5MoeForConditionalGeneration
    from uniserve_v1_b200.checkpoint.safetensors_io import CheckpointLoader, save_file
    from uniserve_v1_b200.models.qwen3_5 import (Qwen35Config, Qwen35MoeModel, Qwen35Multimodal,
                                                 mrope_positions)
    from uniserve_v1_b200.models.qwen3_vl_vision import Qwen3VLVisionTower, VisionConfig
    tc = Qwen3_5MoeTextConfig(
        vocab_size=300, hidden_size=64, num_hidden_layers=4, num_attention_heads=4,
        num_key_value_heads=2, head_dim=32, linear_num_key_heads=2, linear_num_value_heads=4,
        linear_key_head_dim=16, linear_value_head_dim=16, num_experts=8, num_experts_per_tok=2,
        moe_intermediate_size=32, shared_expert_intermediate_size=48, max_position_embeddings=256,
        layer_types=["linear_attention", "full_attention", "linear_attention", "full_attention"],
        rope_parameters={"rope_type": "default", "rope_theta": 10000.0,
                         "partial_rotary_factor": 0.25, "mrope_section": [2, 1, 1],
                         "mrope_interleaved": True})
    vc = Qwen3_5MoeVisionConfig(depth=2, hidden_size=32, intermediate_size=48, num_heads=2,
                                patch_size=4, temporal_patch_size=2, spatial_merge_size=2,
                                out_hidden_size=64, num_position_embeddings=16)
    cfg = Qwen3_5MoeConfig(text_config=tc.to_dict(), vision_config=vc.to_dict(),
                           image_token_id=290, video_token_id=291, vision_start_token_id=292,
                           vision_end_token_id=293)
    torch.manual_seed(0)
    hf = Qwen3_5MoeForConditionalGeneration(cfg).float().eval()
    save_file({k: v.detach().clone().contiguous() for k, v in hf.state_dict().items()},
              tmp_path / "model.safetensors")
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    ld = CheckpointLoader(tmp_path)
    tcfg = Qwen35Config.from_hf(ld.config)
    assert tcfg.mrope_section == (2, 1, 1) and tcfg.image_token_id == 290
    text = Qwen35MoeModel(tcfg, "cpu", torch.float32).load_state(ld)
    tower = Qwen3VLVisionTower(VisionConfig.from_hf({**ld.config["vision_config"],
                                                      "deepstack_visual_indexes": []}),
                               "cpu", torch.float32).load_state(ld)
    grid = (1, 4, 6)                                   # 24 patches -> 6 merged rows
    prompt = [5, 17, 292] + [290] * 6 + [293, 40, 41, 7]
    pixels = torch.randn(24, 3 * 2 * 4 * 4, generator=torch.Generator().manual_seed(1))
    types = torch.tensor([[1 if t == 290 else 0 for t in prompt]])
    pos3, nxt = mrope_positions(prompt, 290, [grid], 2)
    assert pos3[:, 3].tolist() == [3, 3, 3] and pos3[:, 8].tolist() == [3, 4, 5] and nxt == 10
    with torch.no_grad():
        out = hf(input_ids=torch.tensor([prompt]), pixel_values=pixels,
                 image_grid_thw=torch.tensor([grid]), mm_token_type_ids=types)
        gen = hf.generate(input_ids=torch.tensor([prompt]), pixel_values=pixels,
                          image_grid_thw=torch.tensor([grid]), mm_token_type_ids=types,
                          max_new_tokens=5, do_sample=False)[0, len(prompt):].tolist()
    mm = Qwen35Multimodal(text, tower)
    logits, _ = mm.prefill(prompt, pixels, [grid], text.new_state())
    torch.testing.assert_close(logits, out.logits[0], atol=3e-4, rtol=2e-3)
    assert mm.generate(prompt, pixels, [grid], 5) == gen


def test_image_preprocessing_matches_the_transformers_processor():
    """Patch rows and grids of the Qwen-VL image processor for an image that needs no
    resize (exact) and one that does (same grid, close values: resampling filters differ)."""
    import io
    import base64
    import numpy as np
    import pytest
    from PIL import Image
    from transformers.models.qwen2_vl.image_processing_qwen2_vl import Qwen2VLImageProcessor
    from uniserve_v1_b200.server import images as IM
    proc = Qwen2VLImageProcessor(patch_size=16, temporal_patch_size=2, merge_size=2,
                                 min_pixels=64 * 64, max_pixels=1280 * 28 * 28,
                                 image_mean=[0.5, 0.5, 0.5], image_std=[0.5, 0.5, 0.5])
    rng = np.random.RandomState(0)
    exact = rng.randint(0, 256, (96, 160, 3), dtype=np.uint8)
    want = proc(images=[Image.fromarray(exact)], return_tensors="pt")
    rows, grid = IM.preprocess(exact)
    assert list(grid) == want["image_grid_thw"][0].tolist() == [1, 6, 10]
    torch.testing.assert_close(rows, want["pixel_values"], atol=1e-6, rtol=0)
    odd = rng.randint(0, 256, (75, 131, 3), dtype=np.uint8)
    want = proc(images=[Image.fromarray(odd)], return_tensors="pt")
    rows, grid = IM.preprocess(odd)
    assert list(grid) == want["image_grid_thw"][0].tolist()
    assert float((rows - want["pixel_values"]).abs().mean()) < 0.05
    buf = io.BytesIO()
    Image.fromarray(exact).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    assert np.array_equal(IM.load_image(url), exact)
    with pytest.raises(ValueError):
        IM.load_image("https://example.com/cat.png")
    assert IM.expand_placeholders([1, 9, 2], 9, [(1, 6, 10)], 2) == [1] + [9] * 15 + [2]
    assert IM.collect([{"role": "user", "content": [{"type": "text", "text": "hi"},
                                                    {"type": "image_url", "image_url": {"url": url}}]}]) == [url]


def test_qwen3_vl_with_deepstack_matches_transformers(tmp_path):
    """Dense Qwen3-VL: three-axis rotary positions over the whole head, vision rows at the
    placeholders, deep-stack rows added after the first layers; logits and greedy decoding of a
    tiny random `Qwen3VLForConditionalGeneration`, and the dense-state engine on the same
    request with its prompt read in chunks."""
    import pytest
    pytest.importorskip("transformers")
    from transformers.models.qwen3_vl.configuration_qwen3_vl import (Qwen3VLConfig,
                                                                     Qwen3VLTextConfig as HfText,
                                                                     Qwen3VLVisionConfig)
    from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLForConditionalGeneration
    from uniserve_v1_b200.checkpoint.safetensors_io import CheckpointLoader, save_file
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_5 import Qwen35Multimodal
    from uniserve_v1_b200.models.qwen3_vl import Qwen3VLDenseModel, Qwen3VLTextConfig
    from uniserve_v1_b200.models.qwen3_vl_vision import Qwen3VLVisionTower, VisionConfig
    tc = HfText(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=3,
                num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                max_position_embeddings=256, eos_token_id=299,
                rope_parameters={"rope_type": "default", "rope_theta": 10000.0,
                                 "mrope_section": [4, 2, 2], "mrope_interleaved": True})
    vc = Qwen3VLVisionConfig(depth=3, hidden_size=32, intermediate_size=48, num_heads=2,
                             patch_size=4, temporal_patch_size=2, spatial_merge_size=2,
                             out_hidden_size=64, num_position_embeddings=16,
                             deepstack_visual_indexes=[0, 2])
    cfg = Qwen3VLConfig(text_config=tc.to_dict(), vision_config=vc.to_dict(), image_token_id=290,
                        video_token_id=291, vision_start_token_id=292, vision_end_token_id=293)
    torch.manual_seed(0)
    hf = Qwen3VLForConditionalGeneration(cfg).float().eval()
    save_file({k: v.detach().clone().contiguous() for k, v in hf.state_dict().items()},
              tmp_path / "model.safetensors")
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    ld = CheckpointLoader(tmp_path)
    tcfg = Qwen3VLTextConfig.from_hf(ld.config)
    assert tcfg.mrope_section == (4, 2, 2) and tcfg.image_token_id == 290
    text = Qwen3VLDenseModel(tcfg, "cpu", torch.float32).load_state(ld)
    tower = Qwen3VLVisionTower(VisionConfig.from_hf(ld.config), "cpu", torch.float32).load_state(ld)
    grid = (1, 4, 6)
    prompt = [5, 17, 292] + [290] * 6 + [293, 40, 41, 7]
    pixels = torch.randn(24, 3 * 2 * 4 * 4, generator=torch.Generator().manual_seed(1))
    types = torch.tensor([[1 if t == 290 else 0 for t in prompt]])
    kw = dict(input_ids=torch.tensor([prompt]), pixel_values=pixels,
              image_grid_thw=torch.tensor([grid]), mm_token_type_ids=types)
    with torch.no_grad():
        want = hf(**kw).logits[0]
        gen = hf.generate(**kw, max_new_tokens=5, do_sample=False)[0, len(prompt):].tolist()
    mm = Qwen35Multimodal(text, tower)
    logits, _ = mm.prefill(prompt, pixels, [grid], text.new_state())
    torch.testing.assert_close(logits, want, atol=3e-4, rtol=2e-3)
    assert mm.generate(prompt, pixels, [grid], 5) == gen
    eng = DenseStateEngine(text, prefill_chunk=5, tower=tower)
    rid = eng.add_request(prompt, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True),
                          media=(pixels, [grid]))
    while eng.has_work():
        eng.step()
    assert eng.requests[rid].output_ids == gen


def test_qwen3_vl_moe_matches_transformers(tmp_path):
    """The expert variant of Qwen3-VL (stacked expert tensors, routed MLP in every layer) with
    an image in the prompt."""
    import pytest
    pytest.importorskip("transformers")
    from transformers.models.qwen3_vl_moe.configuration_qwen3_vl_moe import (
        Qwen3VLMoeConfig, Qwen3VLMoeTextConfig, Qwen3VLMoeVisionConfig)
    from transformers.models.qwen3_vl_moe.modeling_qwen3_vl_moe import \
        Qwen3VLMoeForConditionalGeneration
    from uniserve_v1_b200.checkpoint.safetensors_io import (CheckpointLoader, resolve_family,
                                                            save_file)
    from uniserve_v1_b200.models.qwen3_5 import Qwen35Multimodal
    from uniserve_v1_b200.models.qwen3_vl import Qwen3VLDenseModel, Qwen3VLTextConfig
    from uniserve_v1_b200.models.qwen3_vl_vision import Qwen3VLVisionTower, VisionConfig
    tc = Qwen3VLMoeTextConfig(vocab_size=300, hidden_size=64, intermediate_size=96,
                              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                              head_dim=16, num_experts=4, num_experts_per_tok=2,
                              moe_intermediate_size=32, max_position_embeddings=256,
                              eos_token_id=299,
                              rope_parameters={"rope_type": "default", "rope_theta": 10000.0,
                                               "mrope_section": [4, 2, 2],
                                               "mrope_interleaved": True})
    vc = Qwen3VLMoeVisionConfig(depth=2, hidden_size=32, intermediate_size=48, num_heads=2,
                                patch_size=4, temporal_patch_size=2, spatial_merge_size=2,
                                out_hidden_size=64, num_position_embeddings=16,
                                deepstack_visual_indexes=[1])
    cfg = Qwen3VLMoeConfig(text_config=tc.to_dict(), vision_config=vc.to_dict(),
                           image_token_id=290, video_token_id=291, vision_start_token_id=292,
                           vision_end_token_id=293)
    torch.manual_seed(0)
    hf = Qwen3VLMoeForConditionalGeneration(cfg).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "experts" in n:
                p.copy_(torch.randn_like(p) * 0.1)
    save_file({k: v.detach().clone().contiguous() for k, v in hf.state_dict().items()},
              tmp_path / "model.safetensors")
    d = cfg.to_dict()
    d["architectures"] = ["Qwen3VLMoeForConditionalGeneration"]
    (tmp_path / "config.json").write_text(json.dumps(d))
    assert resolve_family(tmp_path) == "qwen3_vl"
    ld = CheckpointLoader(tmp_path)
    tcfg = Qwen3VLTextConfig.from_hf(ld.config)
    assert tcfg.num_experts == 4 and tcfg.is_moe_layer(0)
    text = Qwen3VLDenseModel(tcfg, "cpu", torch.float32).load_state(ld)
    tower = Qwen3VLVisionTower(VisionConfig.from_hf(ld.config), "cpu", torch.float32).load_state(ld)
    grid = (1, 4, 4)
    prompt = [5, 292] + [290] * 4 + [293, 40, 7]
    pixels = torch.randn(16, 3 * 2 * 4 * 4, generator=torch.Generator().manual_seed(1))
    types = torch.tensor([[1 if t == 290 else 0 for t in prompt]])
    kw = dict(input_ids=torch.tensor([prompt]), pixel_values=pixels,
              image_grid_thw=torch.tensor([grid]), mm_token_type_ids=types)
    with torch.no_grad():
        want = hf(**kw).logits[0]
        gen = hf.generate(**kw, max_new_tokens=4, do_sample=False)[0, len(prompt):].tolist()
    mm = Qwen35Multimodal(text, tower)
    logits, _ = mm.prefill(prompt, pixels, [grid], text.new_state())
    torch.testing.assert_close(logits, want, atol=3e-4, rtol=2e-3)
    assert mm.generate(prompt, pixels, [grid], 4) == gen


def test_qwen3_5_dense_variant_matches_transformers(tmp_path):
    """`Qwen3_5ForCausalLM`: the hybrid decoder with one gated MLP per layer instead of experts."""
    import pytest
    pytest.importorskip("transformers")
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5TextConfig
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5ForCausalLM
    from uniserve_v1_b200.checkpoint.safetensors_io import CheckpointLoader, save_file
    from uniserve_v1_b200.models.qwen3_5 import Qwen35Config, Qwen35MoeModel
    hf_cfg = Qwen3_5TextConfig(
        vocab_size=200, hidden_size=64, intermediate_size=96, num_hidden_layers=4,
        num_attention_heads=4, num_key_value_heads=2, head_dim=32, linear_num_key_heads=2,
        linear_num_value_heads=4, linear_key_head_dim=16, linear_value_head_dim=16,
        max_position_embeddings=128,
        layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"])
    torch.manual_seed(4)
    hf = Qwen3_5ForCausalLM(hf_cfg).float().eval()
    save_file({k: v.detach().clone().contiguous() for k, v in hf.state_dict().items()},
              tmp_path / "model.safetensors")
    (tmp_path / "config.json").write_text(json.dumps(hf_cfg.to_dict()))
    ld = CheckpointLoader(tmp_path)
    cfg = Qwen35Config.from_hf(ld.config)
    assert cfg.num_experts == 0 and cfg.intermediate_size == 96
    model = Qwen35MoeModel(cfg, "cpu", torch.float32).load_state(ld)
    ids = torch.randint(0, 200, (23,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(ids[None]).logits[0]
        gen = hf.generate(ids[None], max_new_tokens=5, do_sample=False)[0, 23:].tolist()
    st = model.new_state()
    got = torch.cat([model.forward(ids[:20], st, 0), model.forward(ids[20:], st, 20)])
    torch.testing.assert_close(got, want, atol=2e-4, rtol=2e-3)
    assert model.generate(ids.tolist(), 5)[:len(gen)] == gen


def test_qwen3_next_packed_projections_match_transformers(tmp_path):
    """`Qwen3NextForCausalLM` stores the linear layers' projections packed per key head; the
    loader unpacks them into the hybrid decoder's layout."""
    import pytest
    pytest.importorskip("transformers")
    from transformers.models.qwen3_next.configuration_qwen3_next import Qwen3NextConfig
    from transformers.models.qwen3_next.modeling_qwen3_next import Qwen3NextForCausalLM
    from uniserve_v1_b200.checkpoint.safetensors_io import CheckpointLoader, save_file
    from uniserve_v1_b200.models.qwen3_5 import Qwen35Config, Qwen35MoeModel
    hf_cfg = Qwen3NextConfig(
        vocab_size=200, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=2, head_dim=32, linear_num_key_heads=2,
        linear_num_value_heads=4, linear_key_head_dim=16, linear_value_head_dim=16,
        num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
        shared_expert_intermediate_size=32, max_position_embeddings=128, norm_topk_prob=True,
        layer_types=["linear_attention", "full_attention"])
    torch.manual_seed(6)
    hf = Qwen3NextForCausalLM(hf_cfg).float().eval()
    save_file({k: v.detach().clone().contiguous() for k, v in hf.state_dict().items()},
              tmp_path / "model.safetensors")
    (tmp_path / "config.json").write_text(json.dumps(hf_cfg.to_dict()))
    ld = CheckpointLoader(tmp_path)
    model = Qwen35MoeModel(Qwen35Config.from_hf(ld.config), "cpu", torch.float32).load_state(ld)
    ids = torch.randint(0, 200, (17,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(ids[None]).logits[0]
    torch.testing.assert_close(model.forward(ids, model.new_state()), want, atol=2e-4, rtol=2e-3)
