"""Policy package parsing (the reference's example deployments parse verbatim),
effects, revisions; safetensors round trip and loading a tiny HF checkpoint."""
import json

import pytest
import torch

from uniserve_v1_b200.checkpoint.safetensors_io import (CheckpointLoader, parse_model_id,
                                                        resolve_family, save_file)
from uniserve_v1_b200.config.policy import (ConfigError, Package, RevisionStore, parse_bytes,
                                            parse_duration, strongest_effect)

TP4 = '''
model = "Qwen/Qwen3-30B-A3B"
[moe_config]
expert_parallel = true
[[worker_groups]]
id = "model"
ranks = ["cuda:0-3"]
queue_depth = 2
[worker_groups.blocks.model]
tensor_parallel_size = 4
[programs.chunk]
source = "uniserve:chunk"
period = "10s"
args = { tpot = "50ms", ttft = "1s", low = 512, high = 8192 }
[programs.expert-order]
source = "uniserve:expert-order"
period = "10m"
args = { ranks = 4 }
'''

AFD = '''
model = "Qwen/Qwen3-30B-A3B"
hosts = ["rank-1", "rank-2"]
[moe_config]
expert_parallel = true
[[worker_groups]]
id = "attention"
ranks = ["rank-1/cuda:0-1"]
queue_depth = 2
[worker_groups.blocks.model]
tensor_parallel_size = 2
[[worker_groups]]
id = "experts"
role = "experts"
ranks = ["rank-2/cuda:0-1"]
queue_depth = 2
'''

ULYSSES8 = '''
model = "FastVideo/FastVideo-FastH3-8-Step-V2"
served_model_name = "FastH3"
[[worker_groups]]
id = "model"
ranks = ["cuda:0-7"]
queue_depth = 6
[worker_groups.blocks.transformer]
sequence_parallel = { kind = "ulysses", ulysses_degree = 8, projection = "exchange" }
[worker_groups.blocks.text_encoder]
tensor_parallel_size = 8
[worker_groups.blocks.video_decoder]
distribution = "temporal_units"
[worker_groups.blocks.muxer]
ranks = [0]
'''

DP8 = '''
model = "FastVideo/FastVideo-FastH3-8-Step-V2"
[[worker_groups]]
id = "text"
ranks = ["cuda:0-7"]
queue_depth = 24
mem_fraction_static = 0.18
[worker_groups.blocks.text_encoder]
tensor_parallel_size = 8
[[worker_groups]]
id = "flow"
copies = 8
ranks = ["cuda:0-7"]
queue_depth = 6
mem_fraction_static = 0.81
[worker_groups.blocks.transformer]
'''


def test_literals():
    assert parse_duration("250ms") == 0.25 and parse_duration("10m") == 600 and parse_duration(3) == 3
    assert parse_bytes("64MiB") == 64 << 20 and parse_bytes("1GB") == 10**9
    with pytest.raises(ConfigError):
        parse_duration("soon", "x.y")


def test_reference_deployments_parse():
    p = Package.parse(TP4)
    assert p.model == "Qwen/Qwen3-30B-A3B" and p.moe_config.expert_parallel
    g = p.worker_groups[0]
    assert [str(r) for r in g.ranks] == ["cuda:0", "cuda:1", "cuda:2", "cuda:3"]
    assert g.blocks["model"].tensor_parallel_size == 4
    assert p.programs["chunk"].period == 10.0 and p.programs["expert-order"].args == {"ranks": 4}
    a = Package.parse(AFD)
    assert a.worker_groups[1].role == "experts" and a.worker_groups[1].ranks[0].host == "rank-2"
    u = Package.parse(ULYSSES8)
    sp = u.worker_groups[0].blocks["transformer"].sequence_parallel
    assert sp.kind == "ulysses" and sp.ulysses_degree == 8 and sp.projection == "exchange"
    assert u.worker_groups[0].blocks["video_decoder"].distribution == "temporal_units"
    d = Package.parse(DP8)
    assert d.worker_groups[1].copies == 8 and d.worker_groups[0].mem_fraction_static == 0.18
    assert d.layout()["groups"][1]["copies"] == 8


def test_strict_errors_name_the_path():
    with pytest.raises(ConfigError) as e:
        Package.parse('model = "a/b"\n[kv_cache_config]\nblok_size = 16\n')
    assert "kv_cache_config.blok_size" in str(e.value)
    with pytest.raises(ConfigError) as e:
        Package.parse('model = "a/b"\n[[worker_groups]]\nid="g"\nranks=["cpu:0"]\n')
    assert "CUDA devices only" in str(e.value)
    with pytest.raises(ConfigError) as e:
        Package.parse('model = "a/b"\nquantization_config = {}\n')
    assert "quantization" in str(e.value)
    with pytest.raises(ConfigError):
        Package.parse('model = "a/b"\n[[worker_groups]]\nid="e"\nrole="experts"\nranks=["cuda:0"]\n')


def test_effects_and_diff(tmp_path):
    a = Package.parse('model = "a/b"\n')
    b = Package.parse('model = "a/b"\nserved_model_name = "x"\n[kv_cache_config]\nprefix_caching = false\n')
    ch = a.diff(b)
    assert {c[0] for c in ch} == {"served_model_name", "kv_cache_config.prefix_caching"}
    assert strongest_effect(ch) == "step"
    c = Package.parse('model = "a/b"\ntensor_parallel_size = 2\n')
    assert strongest_effect(a.diff(c)) == "epoch"
    assert Package.effect_of("speculative_config.num_draft_tokens") == "generation"
    rs = RevisionStore("dep", str(tmp_path))
    assert rs.commit('model = "a/b"\n') == 1 and rs.commit('model = "a/b"\npaused = true\n') == 2
    assert rs.current().paused is True and rs.revisions() == [1, 2]


def test_safetensors_roundtrip_and_model_load(tmp_path):
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    cfg = Qwen3MoeConfig.tiny()
    ref = Qwen3MoeModel(cfg, "cpu", torch.float32).init_random(seed=3)
    D, Hq, Hkv, I = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.moe_intermediate_size
    tensors = {"model.embed_tokens.weight": ref.embed, "model.norm.weight": ref.final_norm,
               "lm_head.weight": ref.lm_head}
    for i, lw in enumerate(ref.layers):
        p = f"model.layers.{i}."
        tensors[p + "input_layernorm.weight"] = lw.input_norm
        tensors[p + "post_attention_layernorm.weight"] = lw.post_norm
        tensors[p + "self_attn.q_proj.weight"] = lw.qkv[:Hq * D]
        tensors[p + "self_attn.k_proj.weight"] = lw.qkv[Hq * D:(Hq + Hkv) * D]
        tensors[p + "self_attn.v_proj.weight"] = lw.qkv[(Hq + Hkv) * D:]
        tensors[p + "self_attn.o_proj.weight"] = lw.o_proj
        tensors[p + "self_attn.q_norm.weight"] = lw.q_norm
        tensors[p + "self_attn.k_norm.weight"] = lw.k_norm
        tensors[p + "mlp.gate.weight"] = lw.router
        for e in range(cfg.num_experts):
            tensors[p + f"mlp.experts.{e}.up_proj.weight"] = lw.w13[e, :I]
            tensors[p + f"mlp.experts.{e}.gate_proj.weight"] = lw.w13[e, I:]
            tensors[p + f"mlp.experts.{e}.down_proj.weight"] = lw.w2[e]
    names = sorted(tensors)
    half = len(names) // 2
    save_file({n: tensors[n] for n in names[:half]}, tmp_path / "model-00001-of-00002.safetensors")
    save_file({n: tensors[n] for n in names[half:]}, tmp_path / "model-00002-of-00002.safetensors")
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {
        n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
        for i, n in enumerate(names)}}))
    hf = {"architectures": ["Qwen3MoeForCausalLM"], "vocab_size": cfg.vocab_size,
          "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_hidden_layers,
          "num_attention_heads": Hq, "num_key_value_heads": Hkv, "head_dim": D,
          "num_experts": cfg.num_experts, "num_experts_per_tok": cfg.num_experts_per_tok,
          "moe_intermediate_size": I, "rope_theta": cfg.rope_theta, "eos_token_id": cfg.eos_token_id,
          "max_position_embeddings": cfg.max_position_embeddings, "rms_norm_eps": cfg.rms_norm_eps,
          "norm_topk_prob": True}
    (tmp_path / "config.json").write_text(json.dumps(hf))
    assert resolve_family(tmp_path) == "qwen3_moe"
    ld = CheckpointLoader(tmp_path)
    assert ld.has("lm_head.weight") and len(ld.identity()) == 2
    loaded = Qwen3MoeModel(Qwen3MoeConfig.from_hf(ld.config), "cpu", torch.float32).load_state(ld)
    assert torch.equal(loaded.layers[1].w13, ref.layers[1].w13)
    assert torch.equal(loaded.layers[0].qkv, ref.layers[0].qkv)
    assert parse_model_id("Qwen/Qwen3-30B-A3B@abc/sub/dir") == ("Qwen/Qwen3-30B-A3B", "abc", "sub/dir")


def test_fp8_block_weight_roundtrip_and_cpu_linear():
    import torch
    from uniserve_v1_b200.ops import fp8 as Q
    g = torch.Generator().manual_seed(0)
    w = torch.randn(2, 256, 384, generator=g) * 0.1
    q, s = Q.quantize_weight_block128(w)
    assert q.dtype == torch.uint8 and s.shape == (2, 2, 3)
    back = Q.dequantize_weight_block128(q, s)
    assert (back - w).abs().max() <= 0.07 * w.abs().max()
    x = torch.randn(5, 384, generator=g).to(torch.bfloat16)
    y = Q.linear_fp8_block(x, q[0], s[0])
    ref = x.float() @ w[0].t()
    assert ((y.float() - ref).norm() / ref.norm()) < 0.08


def test_adapter_fusion(tmp_path):
    """Low-rank pairs, full-rank deltas, bias deltas and assigned tensors fuse into the
    checkpoint's values at the loading boundary; untouched tensors read through."""
    import torch
    from uniserve_v1_b200.checkpoint.adapter import AdaptedLoader, Adapter
    from uniserve_v1_b200.checkpoint.safetensors_io import CheckpointLoader, save_file
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g)
    base = {"blocks.0.attn.to_q.weight": r(16, 8).to(torch.bfloat16),
            "blocks.0.attn.to_q.bias": r(16).to(torch.bfloat16),
            "blocks.0.ff.weight": r(8, 8).to(torch.bfloat16),
            "norm.weight": r(8).to(torch.bfloat16)}
    (tmp_path / "ckpt").mkdir()
    save_file(base, tmp_path / "ckpt" / "model.safetensors")
    edits = {"blocks.0.attn.to_q.lora_A": r(2, 8), "blocks.0.attn.to_q.lora_B": r(16, 2),
             "blocks.0.attn.to_q.diff_b": r(16), "blocks.0.ff.diff": r(8, 8),
             "blocks.0.attn.to_gate_compress.set_weight": r(16, 8).to(torch.bfloat16)}
    (tmp_path / "ad").mkdir()
    save_file(edits, tmp_path / "ad" / "adapter_model.safetensors")
    ad = Adapter(tmp_path / "ad")
    assert ad.contents() == {"low_rank": 2, "diff": 2, "assign": 1}
    ld = AdaptedLoader(CheckpointLoader(tmp_path / "ckpt"), ad)
    w = ld.get("blocks.0.attn.to_q.weight")
    want = (edits["blocks.0.attn.to_q.lora_B"] @ edits["blocks.0.attn.to_q.lora_A"] +
            base["blocks.0.attn.to_q.weight"].float()).to(torch.bfloat16)
    assert w.dtype == torch.bfloat16 and torch.equal(w, want)
    assert torch.equal(ld.get("blocks.0.attn.to_q.bias"),
                       (edits["blocks.0.attn.to_q.diff_b"] + base["blocks.0.attn.to_q.bias"].float())
                       .to(torch.bfloat16))
    assert torch.equal(ld.get("blocks.0.ff.weight"),
                       (edits["blocks.0.ff.diff"] + base["blocks.0.ff.weight"].float())
                       .to(torch.bfloat16))
    assert torch.equal(ld.get("norm.weight"), base["norm.weight"])
    assert ld.has("blocks.0.attn.to_gate_compress.weight")
    assert torch.equal(ld.get("blocks.0.attn.to_gate_compress.weight"),
                       edits["blocks.0.attn.to_gate_compress.set_weight"])
    bad = dict(edits)
    del bad["blocks.0.attn.to_q.lora_B"]
    (tmp_path / "bad").mkdir()
    save_file(bad, tmp_path / "bad" / "adapter_model.safetensors")
    import pytest
    with pytest.raises(ValueError):
        Adapter(tmp_path / "bad")


def test_reference_deployment_examples_resolve_to_axes():
    """Every deployment example of the reference tree parses verbatim and resolves to the
    parallel axes the serve command builds."""
    import glob
    import os
    from uniserve_v1_b200.config.policy import Package
    from uniserve_v1_b200.server.multirank import package_parallelism
    from pathlib import Path
    root = os.environ.get("UNISERVE_REFERENCE_CONFIGS",
                          str(Path(__file__).resolve().parents[2] / "reference" / "configs"))
    if not os.path.isdir(root):
        import pytest
        pytest.skip("reference tree not present")
    seen = {}
    for f in sorted(glob.glob(root + "/**/config.toml", recursive=True)):
        seen[f[len(root) + 1:-len("/config.toml")]] = package_parallelism(
            Package.parse(open(f).read()))
    assert seen["qwen3_moe/tp4"] == {"world": 4, "axes": {"tensor": 4}}
    assert seen["minimax_h3/ulysses8"] == {"world": 8, "axes": {"ulysses": 8}}
    assert seen["minimax_h3/gather8"] == {"world": 8, "axes": {"gather": 8}}
    assert seen["minimax_h3/fasth3-ulysses4x2"] == {"world": 4, "axes": {"ulysses": 4}}
    assert len(seen) >= 10


def test_reference_afd_package_resolves_to_an_expert_union():
    """The reference's disaggregated deployment (a TP2 attention group and two expert
    ranks) resolves to a union of two attention members and two experts-only ranks; its
    tensor-parallel deployment does not."""
    import os
    import pytest
    from uniserve_v1_b200.config.policy import Package
    from uniserve_v1_b200.server import multirank as MR
    from pathlib import Path
    root = os.environ.get("UNISERVE_REFERENCE_CONFIGS",
                          str(Path(__file__).resolve().parents[2] / "reference" / "configs"))
    if not os.path.isdir(root):
        pytest.skip("reference configs not present")
    afd = Package.load(os.path.join(root, "afd/qwen3_moe"))
    assert MR.package_union(afd) == {"sources": 2, "experts": 2, "shared": False}
    assert MR.package_world(afd) == 4
    tp4 = Package.load(os.path.join(root, "qwen3_moe/tp4"))
    assert MR.package_union(tp4) is None and MR.package_world(tp4) == 4
