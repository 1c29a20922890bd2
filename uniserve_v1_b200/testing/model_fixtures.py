"""Tiny Hugging Face checkpoints with reference outputs, for golden tests.

``python -m uniserve_v1_b200.testing.model_fixtures OUT_DIR [family ...]`` writes, per
family, a directory with ``model.safetensors`` + ``config.json`` produced by
``transformers`` from a fixed seed, and ``reference.json`` with the prompt, the logits'
checksum rows and the greedy continuation that ``transformers`` itself computes - what a
checkpoint loader and a decoder of this package must reproduce.

Families: ``qwen3_moe``, ``qwen3``, ``qwen3_5_moe`` (hybrid gated-delta-net decoder).

Reference behaviour: crates/models/python/src/model_fixtures (reference project path).
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

PROMPT = [3, 17, 250, 4, 99, 100, 7, 7, 12]


def _configs():
    from transformers import Qwen3Config, Qwen3MoeConfig
    from transformers.models.qwen3_5_moe.configuration_qwen3_5_moe import Qwen3_5MoeTextConfig
    common = dict(vocab_size=512, hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=32, max_position_embeddings=256,
                  rms_norm_eps=1e-6, tie_word_embeddings=False, eos_token_id=511)
    return {
        "qwen3_moe": ("Qwen3MoeForCausalLM", Qwen3MoeConfig(
            intermediate_size=256, moe_intermediate_size=64, num_experts=8, num_experts_per_tok=2,
            norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[], rope_theta=1e6,
            pad_token_id=0, **common)),
        "qwen3": ("Qwen3ForCausalLM", Qwen3Config(intermediate_size=256, rope_theta=1e6,
                                                  pad_token_id=0, **common)),
        "qwen3_5_moe": ("Qwen3_5MoeForCausalLM", Qwen3_5MoeTextConfig(
            linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=16,
            linear_value_head_dim=16, num_experts=8, num_experts_per_tok=2,
            moe_intermediate_size=32, shared_expert_intermediate_size=48,
            layer_types=["linear_attention", "full_attention"], **common)),
    }


def make(family: str, out_dir, seed: int = 0, new_tokens: int = 6) -> dict:
    """Writes the fixture of ``family`` into ``out_dir``; returns its reference record."""
    import transformers
    from ..checkpoint.safetensors_io import save_file
    cls_name, cfg = _configs()[family]
    torch.manual_seed(seed)
    hf = getattr(transformers, cls_name)(cfg).float().eval()
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    save_file({k: v.detach().clone().contiguous() for k, v in hf.state_dict().items()},
              out / "model.safetensors")
    d = cfg.to_dict()
    d["architectures"] = [cls_name]
    (out / "config.json").write_text(json.dumps(d))
    ids = torch.tensor([PROMPT])
    with torch.no_grad():
        logits = hf(ids).logits[0]
        gen = hf.generate(ids, max_new_tokens=new_tokens, do_sample=False)[0, len(PROMPT):].tolist()
    ref = {"family": family, "architecture": cls_name, "seed": seed, "prompt": PROMPT,
           "greedy": gen, "argmax": logits.argmax(-1).tolist(),
           "logit_rows": {str(i): logits[i, :8].tolist() for i in (0, len(PROMPT) - 1)}}
    (out / "reference.json").write_text(json.dumps(ref, indent=1))
    return ref


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        print(__doc__)
        return 2
    out, fams = Path(argv[0]), argv[1:] or list(_configs())
    for f in fams:
        ref = make(f, out / f)
        print(f"{f}: {out / f} greedy {ref['greedy']}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
