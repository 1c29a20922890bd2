"""The host resamplers against the libraries whose arithmetic they restate."""
import numpy as np
import pytest
import torch

from uniserve_v1_b200.server import resample as RS

SHAPES = [(97, 133, 48, 64), (64, 64, 200, 150), (300, 200, 37, 300), (50, 80, 50, 33)]


@pytest.mark.parametrize("H,W,h,w", SHAPES)
def test_lanczos_is_pillows_to_the_bit(H, W, h, w):
    Image = pytest.importorskip("PIL.Image")
    img = np.random.default_rng(H).integers(0, 256, (H, W, 3), dtype=np.uint8)
    ref = np.asarray(Image.fromarray(img).resize((w, h), Image.Resampling.LANCZOS))
    assert np.array_equal(RS.lanczos_resize(img, h, w), ref)


@pytest.mark.parametrize("orig,new,n", [(44100, 16000, 5000), (16000, 44100, 3000),
                                        (48000, 32000, 4801), (8000, 8000, 100)])
def test_sinc_resample_is_torchaudios(orig, new, n):
    ta = pytest.importorskip("torchaudio")
    a = np.random.default_rng(n).standard_normal((2, n)).astype(np.float32)
    ref = ta.functional.resample(torch.from_numpy(a), orig, new).numpy()
    got = RS.sinc_resample(a, orig, new)
    assert got.shape == ref.shape
    # the same float32 kernels; the sums of ~100 products run in another order
    assert float(np.abs(got - ref).max()) <= 2.0 ** -14 * max(1.0, float(np.abs(ref).max()))


@pytest.mark.parametrize("H,W,h,w", SHAPES[:3])
def test_bicubic_antialias_is_torchs(H, W, h, w):
    rng = np.random.default_rng(W)
    x = rng.standard_normal((3, H, W)).astype(np.float32)
    kw = dict(size=(h, w), mode="bicubic", align_corners=False, antialias=True)
    ref = torch.nn.functional.interpolate(torch.from_numpy(x)[None], **kw)[0].numpy()
    assert float(np.abs(RS.bicubic_antialias(x, h, w) - ref).max()) <= 2.0 ** -14
    u = rng.integers(0, 256, (3, H, W), dtype=np.uint8)
    ref = torch.nn.functional.interpolate(torch.from_numpy(u)[None], **kw)[0].numpy()
    assert np.array_equal(RS.bicubic_antialias(u, h, w), ref)


def test_bad_arguments_are_refused():
    with pytest.raises(ValueError):
        RS.lanczos_resize(np.zeros((4, 4), np.uint8), 2, 2)
    with pytest.raises(ValueError):
        RS.sinc_resample(np.zeros((1, 8), np.float32), 0, 8000)
    with pytest.raises(ValueError):
        RS.bicubic_antialias(np.zeros((3, 4, 4), np.float32), 0, 2)
