"""The video transformer on a GPU (bf16, CUDA kernels) against the same model in
FP32 on the CPU formulas."""
import pytest
import torch

from uniserve_v1_b200.models.minimax_h3 import Denoiser, H3Config, H3Transformer, dmd_ladder
from uniserve_v1_b200.ops import native as N

pytestmark = pytest.mark.gpu


def _run(model):
    cfg = model.cfg
    den = Denoiser(model, dmd_ladder((999, 500), 10.0), dmd_ladder((999, 500), 3.0))
    g = torch.Generator().manual_seed(5)
    text = torch.randn(9, cfg.text_dim, generator=g)
    st = den.prepare(seed=42, latent_frames=3, lat_h=8, lat_w=16, n_audio=20, text_features=text)
    den.run(st)
    return st.video.float().cpu(), st.audio.float().cpu()


def test_denoiser_gpu_close_to_cpu_fp32():
    gpu = H3Transformer(H3Config.tiny(), "cuda", torch.bfloat16).init_random(seed=0)
    vg, ag = _run(gpu)
    torch.cuda.synchronize()
    N.raise_on_device_error()
    vc, ac = _run(gpu.clone_to("cpu", torch.float32))
    # the noise is bit-identical on both devices; the two evaluations add a small
    # bf16 velocity error
    assert (vg - vc).abs().max() < 0.05, (vg - vc).abs().max()
    assert (ag - ac).abs().max() < 0.05, (ag - ac).abs().max()
