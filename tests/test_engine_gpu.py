"""The engine on a GPU: graphs replay what eager computes, and the bf16 model
stays close to the FP32 CPU reference."""
import pytest
import torch

from uniserve_v1_b200.engine.engine import LLMEngine
from uniserve_v1_b200.engine.types import SamplingParams
from uniserve_v1_b200.models.qwen3_moe import AttnMeta, Qwen3MoeConfig, Qwen3MoeModel
from uniserve_v1_b200.models.reference_cpu import ReferenceQwen3Moe
from uniserve_v1_b200.ops import native as N

pytestmark = pytest.mark.gpu


def _cfg():
    return Qwen3MoeConfig(vocab_size=2048, hidden_size=512, num_hidden_layers=2,
                          num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                          num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256,
                          eos_token_id=2047, max_position_embeddings=1024)


def test_prefill_logits_close_to_fp32_reference():
    model = Qwen3MoeModel(_cfg(), "cuda", torch.bfloat16).init_random(seed=0)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, 2048, (48,), generator=g)
    ref_logits, _ = ReferenceQwen3Moe(model).forward(prompt)
    caches = model.new_kv_caches(16, 16)
    ids = prompt.to("cuda", torch.int32)
    pos = torch.arange(48, device="cuda", dtype=torch.int32)
    slots = torch.arange(16, 16 + 48, device="cuda", dtype=torch.int32)
    cu = torch.tensor([0, 48], device="cuda", dtype=torch.int32)
    meta = AttnMeta("prefill", slots, cu_q=cu, cu_k=cu, max_q=48, max_k=48, context_lens=[0])
    hidden = model.forward(ids, pos, meta, caches)
    logits = model.logits(hidden).float().cpu()
    torch.cuda.synchronize()
    N.raise_on_device_error()
    err = (logits - ref_logits).abs().max().item()
    scale = ref_logits.abs().max().item()
    assert err < 0.05 * scale + 0.05, (err, scale)


def test_graph_replay_equals_eager_and_cpu_ops():
    model = Qwen3MoeModel(_cfg(), "cuda", torch.bfloat16).init_random(seed=0)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (9, 33, 20)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    eager = LLMEngine(model, num_pages=128, max_num_seqs=4, max_model_len=256,
                      use_graphs=False).generate(prompts, sp)
    graphs = LLMEngine(model, num_pages=128, max_num_seqs=4, max_model_len=256,
                       use_graphs=True).generate(prompts, sp)
    N.raise_on_device_error()
    assert eager == graphs


def test_sampled_requests_are_reproducible():
    model = Qwen3MoeModel(_cfg(), "cuda", torch.bfloat16).init_random(seed=0)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 2048, (16,), generator=g).tolist() for _ in range(3)]
    sps = [SamplingParams(temperature=0.9, top_k=40, top_p=0.9, seed=5 + i, max_tokens=8,
                          ignore_eos=True) for i in range(3)]
    a = LLMEngine(model, num_pages=128, max_num_seqs=4, max_model_len=256).generate(prompts, sps)
    b = LLMEngine(model, num_pages=128, max_num_seqs=4, max_model_len=256).generate(prompts, sps)
    assert a == b
    pen = SamplingParams(temperature=0.7, repetition_penalty=1.2, presence_penalty=0.5,
                         logit_bias={7: 4.0}, logprobs=True, top_logprobs=3, seed=3, max_tokens=6,
                         ignore_eos=True)
    eng = LLMEngine(model, num_pages=128, max_num_seqs=4, max_model_len=256)
    out = eng.generate(prompts[:1], pen)
    req = list(eng.scheduler.requests.values())[0]
    assert len(out[0]) == 6 and len(req.logprobs) == 6 and len(req.logprobs[0][2]) == 3


def test_multi_step_decode_matches_single_steps():
    model = Qwen3MoeModel(_cfg(), "cuda", torch.bfloat16).init_random(seed=0)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 2048, (20,), generator=g).tolist() for _ in range(2)]
    sp = SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True)
    ref = LLMEngine(model, num_pages=128, max_num_seqs=4, max_model_len=256).generate(prompts, sp)
    eng = LLMEngine(model, num_pages=128, max_num_seqs=4, max_model_len=256)
    ids = [eng.add_request(p, sp) for p in prompts]
    eng.step()                                    # prefill + first token
    reqs = [eng.scheduler.requests[i] for i in ids]
    for r in reqs:                                # pages for 8 more tokens
        need = eng.scheduler._pages_needed(r, r.num_tokens + 8)
        r.pages.extend(eng.blocks.allocate(need))
    toks, _ = eng.runner.decode(reqs, steps=8)
    for i, r in enumerate(reqs):
        assert r.output_ids + toks[:, i].tolist() == ref[i]


def test_fp8_block_experts_stay_close_to_bf16_and_run_under_graphs():
    """Block-scaled FP8 expert weights: prefill logits near the bf16 model's, and the
    decode graphs replay what eager computes."""
    torch.manual_seed(0)
    bf = Qwen3MoeModel(_cfg(), "cuda", torch.bfloat16).init_random(seed=0)
    q8 = Qwen3MoeModel(_cfg(), "cuda", torch.bfloat16, expert_quant="fp8_block").init_random(seed=0)
    assert q8.layers[0].fp8 is not None and q8.layers[0].w13 is None
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, 2048, (48,), generator=g)
    outs = []
    for model in (bf, q8):
        caches = model.new_kv_caches(16, 16)
        ids = prompt.to("cuda", torch.int32)
        pos = torch.arange(48, device="cuda", dtype=torch.int32)
        slots = torch.arange(16, 16 + 48, device="cuda", dtype=torch.int32)
        cu = torch.tensor([0, 48], device="cuda", dtype=torch.int32)
        meta = AttnMeta("prefill", slots, cu_q=cu, cu_k=cu, max_q=48, max_k=48, context_lens=[0])
        outs.append(model.logits(model.forward(ids, pos, meta, caches)).float().cpu())
    torch.cuda.synchronize()
    N.raise_on_device_error()
    err = (outs[0] - outs[1]).abs().max().item()
    scale = outs[0].abs().max().item()
    assert err < 0.15 * scale + 0.05, (err, scale)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    prompts = [prompt.tolist()[:20], prompt.tolist()[5:40]]
    eager = LLMEngine(q8, num_pages=64, max_num_seqs=4, max_model_len=128,
                      use_graphs=False).generate(prompts, sp)
    graphs = LLMEngine(q8, num_pages=64, max_num_seqs=4, max_model_len=128,
                       use_graphs=True).generate(prompts, sp)
    assert eager == graphs


def test_host_kv_tier_on_gpu_restores_evicted_prefix():
    model = Qwen3MoeModel(_cfg(), "cuda", torch.bfloat16).init_random(seed=0)
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    g = torch.Generator().manual_seed(3)
    first = torch.randint(0, 2048, (70,), generator=g).tolist()
    others = [torch.randint(0, 2048, (70,), generator=g).tolist() for _ in range(3)]

    def run(host_pages):
        eng = LLMEngine(model, num_pages=12, page_size=16, max_num_seqs=2, max_model_len=128,
                        use_graphs=False, host_kv_pages=host_pages)
        a = eng.generate([first], sp)[0]
        for o in others:
            eng.generate([o], sp)
        rid = eng.add_request(first, sp)
        req = eng.scheduler.requests[rid]
        while eng.has_work():
            eng.step()
        return a, req.output_ids, req.num_cached
    a0, b0, c0 = run(0)
    a1, b1, c1 = run(32)
    torch.cuda.synchronize()
    N.raise_on_device_error()
    assert a0 == a1 == b0 == b1 and c0 == 0 and c1 == 64


@pytest.mark.parametrize("kv_dtype", ["auto", "fp8_e4m3"])
def test_prefix_cache_file_between_two_gpu_engines(tmp_path, kv_dtype):
    """The cached pages of one engine, written to a file and read by another engine on the
    GPU (bf16 pages, and E4M3 pages with their scales): the prompt is found cached and the
    tokens are those of the first engine's own cached run."""
    from uniserve_v1_b200.engine.prefix_store import load_prefix_cache, save_prefix_cache
    model = Qwen3MoeModel(_cfg(), "cuda", torch.bfloat16).init_random(seed=0)
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, 2048, (100,), generator=g).tolist()
    extra = {} if kv_dtype == "auto" else {"kv_dtype": kv_dtype}

    def engine():
        return LLMEngine(model, num_pages=32, page_size=16, max_num_seqs=2, max_model_len=256,
                         use_graphs=False, **extra)
    a = engine()
    a.generate([prompt], sp)
    want = a.generate([prompt], sp)[0]                    # through its cached pages
    path = str(tmp_path / "gpu.kv")
    saved = save_prefix_cache(a, path)
    assert saved["pages"] >= 6
    b = engine()
    assert load_prefix_cache(b, path)["pages"] == saved["pages"]
    rid = b.add_request(prompt, sp)
    req = b.scheduler.requests[rid]
    while b.has_work():
        b.step()
    torch.cuda.synchronize()
    N.raise_on_device_error()
    assert req.num_cached >= 96 and req.output_ids == want
