"""NVFP4 / FP8 exports: value tables, round trips, and loading a model through the
expanding loader."""
import json

import torch

from uniserve_v1_b200.checkpoint.quantized import DequantizingLoader, open_checkpoint
from uniserve_v1_b200.checkpoint.safetensors_io import CheckpointLoader, save_file
from uniserve_v1_b200.ops import nvfp4


def test_nvfp4_codes_and_packing():
    codes = torch.arange(16, dtype=torch.uint8).repeat(2)[None]          # [1, 32]
    packed = nvfp4.pack(codes)
    assert packed.shape == (1, 16) and int(packed[0, 0]) == 0x10 and int(packed[0, 7]) == 0xFE
    assert torch.equal(nvfp4.unpack(packed), codes)
    one = torch.ones(1, 2).to(torch.float8_e4m3fn)                          # block scale 1.0
    vals = nvfp4.dequantize(packed, one, 1.0, torch.float32)
    want = torch.tensor(nvfp4.E2M1_VALUES + tuple(-v for v in nvfp4.E2M1_VALUES)).repeat(2)
    assert torch.equal(vals[0], want)


def test_nvfp4_round_trip_is_exact_on_representable_values_and_close_otherwise():
    g = torch.Generator().manual_seed(0)
    table = torch.tensor(nvfp4.E2M1_VALUES + tuple(-v for v in nvfp4.E2M1_VALUES))
    exact = table[torch.randint(0, 16, (8, 64), generator=g)] * 0.25
    exact[:, 0] = 1.5                                   # every block reaches the top code
    exact = exact.reshape(8, 4, 16)
    exact[..., 0] = 6 * 0.25
    exact = exact.reshape(8, 64)
    p, s, gs = nvfp4.quantize(exact)
    assert p.shape == (8, 32) and s.shape == (8, 4) and s.dtype == torch.float8_e4m3fn
    torch.testing.assert_close(nvfp4.dequantize(p, s, gs, torch.float32), exact, rtol=0, atol=0)
    w = torch.randn(32, 128, generator=g) * 0.05
    p, s, gs = nvfp4.quantize(w)
    back = nvfp4.dequantize(p, s, gs, torch.float32)
    # half a step of the coarsest interval (4 .. 6) relative to the block's amax, plus the
    # E4M3 rounding of the block scale
    bmax = w.reshape(32, 8, 16).abs().amax(-1, keepdim=True).expand(32, 8, 16).reshape(32, 128)
    assert float(((back - w).abs() / bmax).max()) <= 1.0 / 6.0 + 0.07
    assert float((back - w).abs().mean() / w.abs().mean()) < 0.12


def _write(tmp_path, tensors, config):
    save_file(tensors, tmp_path / "model.safetensors")
    (tmp_path / "config.json").write_text(json.dumps(config))


def test_expanding_loader_reads_three_layouts(tmp_path):
    g = torch.Generator().manual_seed(1)
    w4, w8, wb = (torch.randn(256, 128, generator=g) * 0.03 for _ in range(3))
    p, s, gs = nvfp4.quantize(w4)
    s8 = w8.abs().max() / 448
    q8 = (w8 / s8).to(torch.float8_e4m3fn)
    sb = wb.reshape(2, 128, 1, 128).abs().amax((1, 3)) / 448
    qb = (wb.reshape(2, 128, 1, 128) / sb[:, None, :, None]).reshape(256, 128).to(torch.float8_e4m3fn)
    _write(tmp_path, {
        "a.weight": p, "a.weight_scale": s, "a.weight_scale_2": gs.reshape(1),
        "a.input_scale": torch.tensor([0.5]),
        "b.weight": q8, "b.weight_scale": s8.reshape(1),
        "c.weight": qb, "c.weight_scale_inv": sb,
        "d.weight": w4.to(torch.bfloat16),
    }, {"quantization_config": {"quant_algo": "MIXED"}})
    L = open_checkpoint(tmp_path, torch.float32)
    assert isinstance(L, DequantizingLoader)
    assert L.names() == {"a.weight", "a.input_scale", "b.weight", "c.weight", "d.weight"}
    torch.testing.assert_close(L.get("a.weight"), nvfp4.dequantize(p, s, gs, torch.float32))
    torch.testing.assert_close(L.get("b.weight"), q8.float() * s8)
    torch.testing.assert_close(L.get("c.weight"), wb, atol=float(sb.max()) * 16, rtol=0)
    assert L.get("d.weight").dtype == torch.bfloat16 and float(L.get("a.input_scale")) == 0.5
    assert L.expanded == {"nvfp4": 1, "fp8_tensor": 1, "fp8_block": 1}
    assert isinstance(open_checkpoint(tmp_path).loader, CheckpointLoader)


def test_qwen3_moe_loads_from_an_nvfp4_export(tmp_path):
    """Every 2-D projection exported as NVFP4: the model built through the expanding
    loader equals the model built from the expanded tensors."""
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    cfg = Qwen3MoeConfig.tiny()
    ref = Qwen3MoeModel(cfg, "cpu", torch.float32).init_random(seed=3)
    state = ref.export_state()
    quant, plain = {}, {}
    for name, t in state.items():
        if name.endswith("_proj.weight") and t.dim() == 2 and t.shape[1] % 16 == 0:
            p, s, gs = nvfp4.quantize(t)
            quant[name], quant[name + "_scale"], quant[name + "_scale_2"] = p, s, gs.reshape(1)
            plain[name] = nvfp4.dequantize(p, s, gs, torch.float32)
        else:
            quant[name] = t
            plain[name] = t
    save_file(quant, tmp_path / "model.safetensors")
    (tmp_path / "config.json").write_text(json.dumps({"quantization_config": {"quant_algo": "NVFP4"}}))
    L = open_checkpoint(tmp_path, torch.float32)

    class Plain:
        def has(self, n): return n in plain
        def get(self, n): return plain[n]
        def names(self): return plain.keys()
    a = Qwen3MoeModel(cfg, "cpu", torch.float32).load_state(L)
    b = Qwen3MoeModel(cfg, "cpu", torch.float32).load_state(Plain())
    for la, lb in zip(a.layers, b.layers):
        for f in ("qkv", "o_proj", "w13", "w2", "router", "input_norm"):
            torch.testing.assert_close(getattr(la, f), getattr(lb, f), rtol=0, atol=0)
    assert not torch.equal(a.layers[0].w2, ref.layers[0].w2)        # it really was 4-bit
    assert L.expanded["nvfp4"] > 0
