"""Media, diffusion and audio-convolution kernels against their PyTorch restatements."""
import pytest
import torch
import torch.nn.functional as TF

from uniserve_v1_b200.ops import diffusion as Dm
from uniserve_v1_b200.ops import media as M
from uniserve_v1_b200.ops import native as N

pytestmark = pytest.mark.gpu
DEV = "cuda"


def teardown_function(_):
    torch.cuda.synchronize()
    N.raise_on_device_error()


def test_noise_and_patch_and_euler():
    a = Dm.philox_normal((3, 1001), 7, 2, 1.0, DEV).cpu()
    b = Dm.philox_normal((3, 1001), 7, 2, 1.0, "cpu")
    torch.testing.assert_close(a, b, atol=2e-6, rtol=1e-5)
    x = torch.randn(24, 3, 8, 12, device=DEV)
    rows = Dm.patchify(x)
    torch.testing.assert_close(rows.cpu(), Dm.patchify(x.cpu()))
    assert torch.equal(Dm.unpatchify(rows, 24, 3, 8, 12), x)
    y, v = torch.randn(1000, device=DEV), torch.randn(1000, device=DEV)
    ref = y + v * -0.37
    torch.testing.assert_close(Dm.scaled_add_(y, v, -0.37), ref)


def test_colour_and_pcm():
    fr = torch.rand(3, 3, 32, 48, device=DEV) * 2.4 - 1.2
    y, u, v = M.rgb_to_yuv420(fr)
    yr, ur, vr = M.rgb_to_yuv420(fr.cpu())
    for g, r in ((y, yr), (u, ur), (v, vr)):
        assert (g.cpu().int() - r.int()).abs().max() <= 1
    assert (M.rgb_bytes(fr).cpu().int() - M.rgb_bytes(fr.cpu()).int()).abs().max() <= 1
    au = torch.rand(2, 999, device=DEV) * 2.4 - 1.2
    assert (M.pcm_interleave(au).cpu().int() - M.pcm_interleave(au.cpu()).int()).abs().max() <= 1


def test_tile_stitch_and_cross_fade():
    H, W, th, tw, ov = 40, 56, 24, 32, 8
    full = torch.randn(2, 3, H, W, device=DEV)
    canvas = torch.zeros_like(full)
    weight = torch.zeros(H, W, device=DEV)
    c2, w2 = torch.zeros(2, 3, H, W), torch.zeros(H, W)
    for y0 in (0, 16):
        for x0 in (0, 24):
            tile = full[:, :, y0:y0 + th, x0:x0 + tw].contiguous()
            M.tile_stitch_(canvas, weight, tile, y0, x0, ov)
            M.tile_stitch_(c2, w2, tile.cpu(), y0, x0, ov)
    M.tile_normalise_(canvas, weight)
    M.tile_normalise_(c2, w2)
    torch.testing.assert_close(canvas.cpu(), c2, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(canvas, full, atol=1e-5, rtol=1e-5)   # consistent tiles blend back
    a, b = torch.randn(5, 3, 8, 8, device=DEV), torch.randn(5, 3, 8, 8, device=DEV)
    torch.testing.assert_close(M.cross_fade(a, b).cpu(), M.cross_fade(a.cpu(), b.cpu()))


@pytest.mark.parametrize("Cin,Cout,K,stride,dil", [(32, 64, 7, 1, 1), (48, 40, 3, 1, 5),
                                                    (8, 16, 11, 1, 3), (16, 16, 4, 2, 1)])
def test_conv1d(Cin, Cout, K, stride, dil):
    x = torch.randn(2, Cin, 333, device=DEV)
    w, b = torch.randn(Cout, Cin, K, device=DEV) * 0.1, torch.randn(Cout, device=DEV)
    pad = dil * (K - 1) // 2
    torch.backends.cudnn.allow_tf32 = False
    ref = TF.conv1d(x.cpu(), w.cpu(), b.cpu(), stride, pad, dil)
    torch.testing.assert_close(M.conv1d(x, w, b, stride, pad, dil).cpu(), ref, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("r,k", [(5, 9), (2, 4)])
def test_conv_transpose1d_snake_activation(r, k):
    x = torch.randn(2, 24, 77, device=DEV)
    w, b = torch.randn(24, 12, k, device=DEV) * 0.1, torch.randn(12, device=DEV)
    ref = TF.conv_transpose1d(x.cpu(), w.cpu(), b.cpu(), r, (k - r) // 2)
    torch.testing.assert_close(M.conv_transpose1d(x, w, b, r, (k - r) // 2).cpu(), ref,
                               atol=1e-4, rtol=1e-4)
    la, lb = torch.randn(24, device=DEV) * 0.3, torch.randn(24, device=DEV) * 0.3
    taps = M.kaiser_sinc_taps(12).to(DEV)
    got = M.activation1d(x, taps, la, lb).cpu()
    want = M.activation1d_ref(x.cpu(), taps.cpu(), la.cpu(), lb.cpu())
    torch.testing.assert_close(got, want, atol=1e-4, rtol=1e-4)


def test_vae_decoders_gpu_close_to_cpu():
    from uniserve_v1_b200.models.h3_vae import (AudioVaeConfig, AudioVaeDecoder, VideoVaeConfig,
                                                VideoVaeDecoder)
    vg = VideoVaeDecoder(VideoVaeConfig.tiny(), DEV, torch.bfloat16).init_random(1)
    vc = VideoVaeDecoder(VideoVaeConfig.tiny(), "cpu", torch.float32)
    for name in ("post_quant", "proj_in", "registers", "norm_w", "norm_b", "proj_out"):
        setattr(vc, name, getattr(vg, name).float().cpu())
    vc.blocks = [{k: t.float().cpu() for k, t in b.items()} for b in vg.blocks]
    lat = torch.randn(4, 5, 6, 8)
    fg = vg.decode_unit(lat.to(DEV)).float().cpu()
    fc = vc.decode_unit(lat)
    assert fg.shape == (17, 3, 24, 32)
    assert (fg - fc).abs().max() < 0.05 * fc.abs().max() + 0.02
    ag = AudioVaeDecoder(AudioVaeConfig.tiny(), DEV).init_random(2)
    ac = AudioVaeDecoder(AudioVaeConfig.tiny(), "cpu")
    ac.conv_pre = tuple(t.cpu() for t in ag.conv_pre)
    ac.conv_post = tuple(t.cpu() for t in ag.conv_post)
    ac.act_post = tuple(t.cpu() for t in ag.act_post)
    mv = lambda o: (tuple(t.cpu() for t in o) if isinstance(o, tuple) else o)
    ac.stages = [dict(up=mv(s["up"]), rate=s["rate"], k=s["k"],
                      res=[[{k: mv(v) for k, v in cv.items()} for cv in convs] for convs in s["res"]])
                 for s in ag.stages]
    z = torch.randn(2, 8, 30)
    torch.testing.assert_close(ag.decode(z.to(DEV)).cpu(), ac.decode(z), atol=1e-4, rtol=1e-3)


def test_video_request_on_the_gpu_returns_a_decodable_clip(tmp_path):
    """A whole `VideoService.generate` request on the GPU (tiny transformer and decoders):
    the planes reach pinned host memory on a copy stream while the audio decoder runs, the MP4
    is built in memory, and a second request (buffers reused) gives the same bytes."""
    cv2 = pytest.importorskip("cv2")
    from uniserve_v1_b200.models.h3_vae import (AudioVaeConfig, AudioVaeDecoder, VideoVaeConfig,
                                                VideoVaeDecoder)
    from uniserve_v1_b200.models.minimax_h3 import H3Config, H3Transformer
    from uniserve_v1_b200.server.video_rules import VideoPlan
    from uniserve_v1_b200.server.video_service import VideoJob, VideoService
    cfg = H3Config.tiny()
    cfg.vae_spatial = 64
    tr = H3Transformer(cfg, "cuda", torch.bfloat16).init_random(0)
    vc = VideoVaeConfig.tiny()
    vc.latent_channels, vc.spatial = cfg.latent_channels, 64
    vv = VideoVaeDecoder(vc, "cuda", torch.bfloat16).init_random(1)
    av = AudioVaeDecoder(AudioVaeConfig(latent_channels=cfg.audio_channels, decoder_dim=128,
                                        rates=(5, 5, 2, 2, 2, 2, 2), kernels=(9, 9, 4, 4, 4, 4, 4),
                                        res_kernels=(3,), res_dilations=(1,)), "cuda").init_random(2)
    svc = VideoService(tr, vv, av, sizes=["256x256"], max_seconds=5)
    plan = VideoPlan("t2va", 256, 256, 39, 24, 1000, 8)
    one = svc.generate(VideoJob("a stream in a forest", plan))
    two = svc.generate(VideoJob("a stream in a forest", plan))
    assert one[4:8] == b"ftyp" and one == two
    path = tmp_path / "clip.mp4"
    path.write_bytes(one)
    cap = cv2.VideoCapture(str(path))
    n = 0
    while cap.read()[0]:
        n += 1
    assert n == 39
    assert svc.d2h_bytes >= 2 * 39 * 256 * 256 * 3 // 2
