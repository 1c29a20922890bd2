"""The dense-state families on a GPU: the hybrid Qwen3.5 decoder, dense Qwen3-VL and the vision
tower in bf16 through the package's GEMM / MoE / attention kernels, against their own CPU run
(which the CPU tests tie to transformers)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(gpu, cpu, tol):
    err = (gpu.float().cpu() - cpu).norm() / cpu.norm()
    assert float(err) < tol, float(err)


def test_hybrid_decoder_bf16_on_gpu_tracks_fp32():
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_5 import Qwen35Config, Qwen35MoeModel
    from uniserve_v1_b200.ops import native as N
    cfg = Qwen35Config(vocab_size=2048, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, linear_num_key_heads=2,
                       linear_num_value_heads=4, linear_key_head_dim=64, linear_value_head_dim=64,
                       num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                       shared_expert_intermediate_size=128, eos_token_id=2047,
                       mrope_section=(6, 1, 1))
    # the CPU run uses the same bf16 weights and rounds where the kernels round, so that the
    # discrete expert choices agree and the comparison measures the kernels, not bf16 itself
    ref = Qwen35MoeModel(cfg, "cpu", torch.bfloat16).init_random(seed=0)
    gpu = Qwen35MoeModel(cfg, "cuda", torch.bfloat16)
    for k, v in ref.w.items():
        gpu.w[k] = {n: (t.to("cuda") if torch.is_tensor(t) else t) for n, t in v.items()} \
            if isinstance(v, dict) else v.to("cuda")
    ids = torch.randint(0, 2047, (37,), generator=torch.Generator().manual_seed(1))
    want = ref.forward(ids, ref.new_state()).float()
    st = gpu.new_state()
    got = torch.cat([gpu.forward(ids[:20].cuda(), st, 0), gpu.forward(ids[20:].cuda(), st, 20)])
    torch.cuda.synchronize()
    N.raise_on_device_error()
    _close(got, want, 0.06)
    eng = DenseStateEngine(gpu, max_num_seqs=4)
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    outs = eng.generate([ids[:9].tolist(), ids[9:30].tolist(), ids[30:].tolist()], sp)
    assert all(len(o) == 5 for o in outs)
    torch.cuda.synchronize()
    N.raise_on_device_error()


def test_vision_tower_bf16_on_gpu_tracks_fp32():
    from uniserve_v1_b200.models.qwen3_vl_vision import Qwen3VLVisionTower, VisionConfig
    from uniserve_v1_b200.ops import native as N
    vc = VisionConfig(depth=2, hidden_size=128, intermediate_size=256, num_heads=2, patch_size=8,
                      temporal_patch_size=2, spatial_merge_size=2, out_hidden_size=256,
                      num_position_embeddings=64, deepstack_visual_indexes=[0])
    g = torch.Generator().manual_seed(2)

    def rnd(*s):
        return torch.randn(*s, generator=g) * 0.05
    H, I, wide = 128, 256, 512
    w = {"patch_w": rnd(H, 3 * 2 * 64), "patch_b": rnd(H), "pos": rnd(64, H)}
    for i in range(2):
        w[i] = {"norm1.weight": torch.ones(H), "norm1.bias": torch.zeros(H),
                "norm2.weight": torch.ones(H), "norm2.bias": torch.zeros(H),
                "attn.qkv.weight": rnd(3 * H, H), "attn.qkv.bias": rnd(3 * H),
                "attn.proj.weight": rnd(H, H), "attn.proj.bias": rnd(H),
                "mlp.linear_fc1.weight": rnd(I, H), "mlp.linear_fc1.bias": rnd(I),
                "mlp.linear_fc2.weight": rnd(H, I), "mlp.linear_fc2.bias": rnd(H)}
    mk = lambda post: {"norm.weight": torch.ones(wide if post else H),
                       "norm.bias": torch.zeros(wide if post else H),
                       "linear_fc1.weight": rnd(wide, wide), "linear_fc1.bias": rnd(wide),
                       "linear_fc2.weight": rnd(256, wide), "linear_fc2.bias": rnd(256)}
    w["merger"], w["deepstack"] = mk(False), [mk(True)]
    ref = Qwen3VLVisionTower(vc, "cpu", torch.float32)
    ref.w = w
    gpu = Qwen3VLVisionTower(vc, "cuda", torch.bfloat16)
    conv = lambda t: t.to("cuda", torch.bfloat16)
    gpu.w = {k: ({n: conv(t) for n, t in v.items()} if isinstance(v, dict) else
                 [{n: conv(t) for n, t in d.items()} for d in v] if isinstance(v, list) else conv(v))
             for k, v in w.items()}
    grids = [(1, 8, 12), (2, 4, 4)]
    n = sum(t * h * ww for t, h, ww in grids)
    pixels = torch.randn(n, 3 * 2 * 64, generator=g)
    want, wdeep = ref.forward(pixels, grids)
    got, gdeep = gpu.forward(pixels, grids)
    torch.cuda.synchronize()
    N.raise_on_device_error()
    _close(got, want, 0.05)
    _close(gdeep[0], wdeep[0], 0.05)
