"""Keyframe conditions of the video pipeline: the VAE encoder, condition rows in the denoiser,
first / last frame requests over HTTP."""
import base64
import io

import numpy as np
import pytest
import torch

from uniserve_v1_b200.models.h3_vae_encoder import (VideoEncoderConfig, VideoVaeEncoder,
                                                    normalize_pixels)


def test_encoder_is_causal_in_time_and_follows_the_frame_rule():
    cfg = VideoEncoderConfig.tiny(latent_channels=4, spatial=4)
    assert (cfg.spatial, cfg.temporal) == (4, 4)
    enc = VideoVaeEncoder(cfg).init_random(0)
    x = torch.randn(1, 3, 17, 32, 48, generator=torch.Generator().manual_seed(0))
    m = enc.forward(x)
    assert m.shape == (1, 8, 5, 8, 12)                       # 17 frames -> 5 latent frames
    later = x.clone()
    later[:, :, 9:] = 0.0                                     # frames 9.. change
    m2 = enc.forward(later)
    torch.testing.assert_close(m2[:, :, :3], m[:, :, :3])     # latent frame k reads frames <= 4k
    assert float((m2[:, :, 3:] - m[:, :, 3:]).abs().max()) > 1e-3
    still = enc.forward(x[:, :, :1])                          # a still is the clip's first frame
    torch.testing.assert_close(still[:, :, 0], m[:, :, 0])
    z = enc.encode_condition(x[0, :, :1], seed=3)
    assert z.shape == (4, 1, 8, 12)
    torch.testing.assert_close(z, enc.encode_condition(x[0, :, :1], seed=3))
    assert not torch.equal(z, enc.encode_condition(x[0, :, :1], seed=4))
    torch.testing.assert_close(z, z.half().float())           # rounded through FP16
    with pytest.raises(ValueError):
        enc.encode_condition(x[0, :, :1, :30], seed=3)
    with pytest.raises(ValueError):
        VideoVaeEncoder(VideoEncoderConfig(spatial_downsample_factors=(2, 2, 3, 2, 1)))
    px = normalize_pixels(torch.full((1, 2, 2, 3), 255, dtype=torch.uint8))
    torch.testing.assert_close(px[:, 0, 0, 0], (1 - torch.tensor([0.485, 0.456, 0.406])) /
                               torch.tensor([0.229, 0.224, 0.225]))


def test_tiled_encode_cross_fades_the_moments():
    from uniserve_v1_b200.models.h3_vae_encoder import blend_tiles
    a, b = torch.full((2, 4, 6), 1.0), torch.full((2, 4, 6), 3.0)
    out = blend_tiles([(0, 0, a), (0, 4, b)], 4, 10, 2)              # columns 4 and 5 shared
    assert out.shape == (2, 4, 10)
    torch.testing.assert_close(out[0, 0], torch.tensor([1, 1, 1, 1, 1 + 2 / 3, 1 + 4 / 3, 3, 3,
                                                        3, 3.0]))
    same = blend_tiles([(0, 0, a), (0, 4, a), (2, 0, a[:, :2]), (2, 4, a[:, :2])], 4, 10, 2)
    torch.testing.assert_close(same, torch.ones(2, 4, 10))             # weights sum to one
    cfg = VideoEncoderConfig.tiny(latent_channels=4, spatial=4)
    enc = VideoVaeEncoder(cfg).init_random(0)
    x = torch.randn(3, 1, 32, 48, generator=torch.Generator().manual_seed(1))
    whole = enc.moments(x)
    cfg.tile, cfg.tile_overlap = 64, 8
    torch.testing.assert_close(enc.moments(x), whole)                  # one tile holds the raster
    cfg.tile, cfg.tile_overlap = 32, 8
    tiled = enc.moments(x)
    assert tiled.shape == whole.shape and bool(torch.isfinite(tiled).all())
    left = enc._conv("quant_conv", enc.forward(x[None, :, :, :, :32]))[0]
    torch.testing.assert_close(tiled[..., :6], left[..., :6])          # outside the overlap
    assert enc.encode_condition(x, 2).shape == (4, 1, 8, 12)
    cfg.tile_overlap = 6
    with pytest.raises(ValueError):
        enc.moments(x)


def test_audio_encoder_keeps_channels_apart_and_projects_causally():
    from uniserve_v1_b200.models.h3_audio_encoder import (AudioEncoderConfig, AudioVaeEncoder,
                                                          padded_samples)
    cfg = AudioEncoderConfig.tiny(latent_channels=8)
    assert cfg.hop == 8 and AudioEncoderConfig().hop == 800           # 40 latent frames / s
    enc = AudioVaeEncoder(cfg).init_random(0)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 1, cfg.hop * 10, generator=g) * 0.3
    z = enc.encode(x)
    assert z.shape == (20, 8) and bool(torch.isfinite(z).all())
    muted = x.clone()
    muted[1] = 0.0                                                     # the other channel
    z2 = enc.encode(muted).view(10, 2, 8)
    torch.testing.assert_close(z2[:, 0], z.view(10, 2, 8)[:, 0])
    assert not torch.allclose(z2[:, 1], z.view(10, 2, 8)[:, 1])
    rows = torch.randn(10, cfg.latent_dim, generator=g)
    later = rows.clone()
    later[6:] = 0.0
    torch.testing.assert_close(enc.project(later)[:6], enc.project(rows)[:6])
    assert padded_samples(17, 8) == 24 and padded_samples(16, 8) == 16
    for bad in (x[:1], x[:, :, :-1], x.double()):
        with pytest.raises(ValueError):
            enc.encode(bad)
    with pytest.raises(ValueError):
        padded_samples(0, 8)
    with pytest.raises(ValueError):
        AudioVaeEncoder(AudioEncoderConfig(latent_dim=30, latent_channels=8))


def _wav(seed: int, rate: int = 320, seconds: float = 0.5, channels: int = 1) -> str:
    import wave
    pcm = (np.random.default_rng(seed).standard_normal((int(rate * seconds), channels)) * 8000
           ).astype(np.int16)
    buf = io.BytesIO()
    with wave.open(buf, "wb") as wv:
        wv.setnchannels(channels)
        wv.setsampwidth(2)
        wv.setframerate(rate)
        wv.writeframes(pcm.tobytes())
    return "data:audio/wav;base64," + base64.b64encode(buf.getvalue()).decode()


def test_wav_tracks_load_as_the_stereo_pair():
    from uniserve_v1_b200.models.h3_audio_encoder import load_wav
    mono = load_wav(_wav(0, 320, 0.5, 1), 320)
    assert mono.shape == (2, 1, 160) and torch.equal(mono[0], mono[1])
    stereo = load_wav(_wav(1, 640, 0.5, 2), 320)                       # resampled
    assert stereo.shape == (2, 1, 160) and not torch.equal(stereo[0], stereo[1])
    for bad in ("http://x/y.wav", "data:audio/wav;base64,AAAA", "data:audio/wav,xx"):
        with pytest.raises(ValueError):
            load_wav(bad, 320)


def _tiny_pipeline():
    from uniserve_v1_b200.models.h3_vae import (AudioVaeConfig, AudioVaeDecoder, VideoVaeConfig,
                                                VideoVaeDecoder)
    from uniserve_v1_b200.models.minimax_h3 import H3Config, H3Transformer
    cfg = H3Config.tiny()
    cfg.vae_spatial = 64
    tr = H3Transformer(cfg, "cpu", torch.float32).init_random(0)
    vc = VideoVaeConfig.tiny()
    vc.latent_channels, vc.spatial = cfg.latent_channels, 64
    vv = VideoVaeDecoder(vc, "cpu", torch.float32).init_random(1)
    av = AudioVaeDecoder(AudioVaeConfig(latent_channels=cfg.audio_channels, decoder_dim=128,
                                        rates=(5, 5, 2, 2, 2, 2, 2), kernels=(9, 9, 4, 4, 4, 4, 4),
                                        res_kernels=(3,), res_dilations=(1,)), "cpu").init_random(2)
    enc = VideoVaeEncoder(VideoEncoderConfig.tiny(cfg.latent_channels, 64)).init_random(3)
    return cfg, tr, vv, av, enc


def test_denoiser_takes_keyframe_rows_at_the_pinned_frames():
    from uniserve_v1_b200.models.minimax_h3 import GROUP_VCOND, Denoiser
    cfg, tr, _, _, enc = _tiny_pipeline()
    den = Denoiser(tr)
    g = torch.Generator().manual_seed(1)
    feats = torch.randn(6, cfg.text_dim, generator=g)
    lf, lh, lw = 3, 4, 4
    first = enc.encode_condition(torch.randn(3, 1, 256, 256, generator=g), 1)
    last = enc.encode_condition(torch.randn(3, 1, 256, 256, generator=g), 1)
    st = den.prepare(5, lf, lh, lw, 8, feats, [(0, first), (-1, last)])
    lay, per = st.layout, 4
    assert lay.n_cond == 2 * per and st.cond_rows.shape == (2 * per, cfg.hidden_size)
    c0 = lay.n_video + lay.n_audio + lay.n_text
    torch.testing.assert_close(lay.coords[:, c0:c0 + per], lay.coords[:, :per])
    torch.testing.assert_close(lay.coords[:, c0 + per:c0 + 2 * per],
                               lay.coords[:, 2 * per:3 * per])
    assert bool((lay.mod_index[c0:c0 + 2 * per] == 3 * GROUP_VCOND).all())
    a = den.run(st).video.clone()
    plain = den.run(den.prepare(5, lf, lh, lw, 8, feats)).video
    other = den.run(den.prepare(5, lf, lh, lw, 8, feats, [(0, last), (-1, first)])).video
    again = den.run(den.prepare(5, lf, lh, lw, 8, feats, [(0, first), (-1, last)])).video
    assert torch.isfinite(a).all() and torch.equal(a, again)
    assert not torch.allclose(a, plain) and not torch.allclose(a, other)
    with pytest.raises(ValueError):
        den.prepare(5, lf, lh, lw, 8, feats, [(0, first[:, :, :2])])
    # reference images: the clip's spatial grid, one time unit apart, before the clip
    st = den.prepare(5, lf, lh, lw, 8, feats, [(None, first), (0, last), (None, last)])
    lay = st.layout
    c0 = lay.n_video + lay.n_audio + lay.n_text
    assert lay.coords[0, c0:c0 + per].tolist() == [-2.0] * per
    assert lay.coords[0, c0 + 2 * per:c0 + 3 * per].tolist() == [-1.0] * per
    torch.testing.assert_close(lay.coords[1:, c0:c0 + per], lay.coords[1:, :per])
    torch.testing.assert_close(lay.coords[:, c0 + per:c0 + 2 * per], lay.coords[:, :per])
    b = den.run(st).video
    assert torch.isfinite(b).all() and not torch.allclose(b, a)
    # a reference track: clean audio-condition rows spread over its time unit
    from uniserve_v1_b200.models.minimax_h3 import GROUP_ACOND, TAG_AUDIO
    track = torch.randn(6, cfg.audio_channels, generator=g)
    st = den.prepare(5, lf, lh, lw, 8, feats, [(None, track), (None, first)])
    lay = st.layout
    c0 = lay.n_video + lay.n_audio + lay.n_text
    assert lay.n_cond == 6 + per and st.cond_rows.shape[0] == 6 + per
    assert bool((lay.mod_index[c0:c0 + 6] == 3 * GROUP_ACOND + TAG_AUDIO).all())
    assert bool((lay.mod_index[c0 + 6:c0 + 6 + per] == 3 * GROUP_VCOND).all())
    t = lay.coords[0, c0:c0 + 6]
    assert float(t[0]) == -2.0 and bool((t[1:] > t[:-1]).all()) and float(t[-1]) < -1.0
    assert lay.coords[0, c0 + 6:c0 + 6 + per].tolist() == [-1.0] * per
    c = den.run(st)
    assert torch.isfinite(c.video).all() and torch.isfinite(c.audio).all()
    with pytest.raises(ValueError):
        den.prepare(5, lf, lh, lw, 8, feats, [(0, track)])
    # a reference clip: several latent frames within one time unit
    clip = torch.cat([first, last, first], 1)
    st = den.prepare(5, lf, lh, lw, 8, feats, [(None, clip)])
    lay = st.layout
    c0 = lay.n_video + lay.n_audio + lay.n_text
    assert lay.n_cond == 3 * per
    torch.testing.assert_close(lay.coords[0, c0:c0 + 3 * per],
                               torch.tensor([-1.0, -2 / 3, -1 / 3]).repeat_interleave(per))
    torch.testing.assert_close(lay.coords[1:, c0 + per:c0 + 2 * per], lay.coords[1:, :per])
    assert torch.isfinite(den.run(st).video).all()
    with pytest.raises(ValueError):
        den.prepare(5, lf, lh, lw, 8, feats, [(0, clip)])


def _png(seed: int) -> str:
    from PIL import Image
    rgb = np.random.default_rng(seed).integers(0, 255, (90, 120, 3), dtype=np.uint8)
    buf = io.BytesIO()
    Image.fromarray(rgb).save(buf, format="PNG")
    return "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()


def _clip(tmp_path, frames: int) -> str:
    import cv2
    path = str(tmp_path / f"clip{frames}.mp4")
    out = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*"mp4v"), 24.0, (96, 64))
    rng = np.random.default_rng(frames)
    for _ in range(frames):
        out.write(rng.integers(0, 255, (64, 96, 3), dtype=np.uint8))
    out.release()
    from uniserve_v1_b200.server import images as IM
    IM.set_media_directory(tmp_path)
    return "file://" + path


def test_first_and_last_frame_requests_over_http(tmp_path):
    from fastapi.testclient import TestClient
    from uniserve_v1_b200.config.policy import Package
    from uniserve_v1_b200.server.app import create_app
    from uniserve_v1_b200.server.video_service import VideoService
    cfg, tr, vv, av, enc = _tiny_pipeline()
    pkg = Package.parse('model = "random:h3:tiny"\nserved_model_name = "FastH3"\n')
    body = {"model": "FastH3", "prompt": "a kite", "size": "256x256", "seconds": 4, "seed": 9,
            "input_references": [{"type": "image", "url": _png(0), "frame_index": 0},
                                 {"type": "image", "url": _png(1), "frame_index": -1}]}
    bare = VideoService(tr, vv, av, sizes=["256x256"], max_seconds=5)
    with TestClient(create_app(package=pkg, video_service=bare, served_model_name="FastH3")) as c:
        assert c.get("/v1/capabilities").json()["tasks"] == ["t2va"]
        r = c.post("/v1/videos/sync", json=body)
        assert r.status_code == 400 and r.json()["error"]["param"] == "input_references"
        plain = c.post("/v1/videos/sync", json={k: v for k, v in body.items()
                                                if k != "input_references"})
        assert plain.status_code == 200
        # multipart: text parts only, one per field
        form = {"model": "FastH3", "prompt": "a kite", "size": "256x256", "seconds": "4",
                "seed": "9"}
        same = c.post("/v1/videos/sync", data=form, files={"x": (None, "")})
        assert same.status_code == 400                               # a field outside the schema
        multi = c.post("/v1/videos/sync", files=[(k, (None, v)) for k, v in form.items()])
        assert multi.status_code == 200 and multi.content == plain.content
        up = c.post("/v1/videos/sync", data=form,
                    files={"input_reference": ("image.png", b"\x89PNG", "image/png")})
        assert up.status_code == 400 and up.json()["error"]["param"] == "input_reference"
        twice = c.post("/v1/videos/sync", files=[(k, (None, v)) for k, v in form.items()] +
                       [("seed", (None, "3"))])
        assert twice.status_code == 400 and twice.json()["error"]["param"] == "seed"
        assert c.post("/v1/videos/sync", content=b"x", headers={"content-type": "text/plain"}
                      ).status_code == 415
    svc = VideoService(tr, vv, av, sizes=["256x256"], max_seconds=5, video_encoder=enc)
    with TestClient(create_app(package=pkg, video_service=svc, served_model_name="FastH3")) as c:
        assert c.get("/v1/capabilities").json()["tasks"] == ["t2va", "fl2va", "ref2va"]
        r = c.post("/v1/videos/sync", json=body)
        assert r.status_code == 200, r.text
        assert r.content[4:8] == b"ftyp" and r.content != plain.content
        again = c.post("/v1/videos/sync", json=body)
        assert again.content == r.content
        refs = dict(body, input_references=[{"type": "image", "url": _png(2)}])
        with_ref = c.post("/v1/videos/sync", json=refs)
        assert with_ref.status_code == 200 and with_ref.content not in (r.content, plain.content)
        refs["input_references"] = [{"type": "audio", "url": _wav(3)}]
        no = c.post("/v1/videos/sync", json=refs)
        assert no.status_code == 400 and "audio" in no.json()["error"]["message"]
        from uniserve_v1_b200.models.h3_audio_encoder import AudioEncoderConfig, AudioVaeEncoder
        svc.audio_encoder = AudioVaeEncoder(AudioEncoderConfig.tiny(cfg.audio_channels)
                                            ).init_random(4)
        track = c.post("/v1/videos/sync", json=refs)
        assert track.status_code == 200, track.text
        assert track.content not in (with_ref.content, plain.content)
        refs["input_references"] = [{"type": "video", "url": "file:///nowhere.mp4"}]
        assert c.post("/v1/videos/sync", json=refs).status_code == 400
        refs["input_references"] = [{"type": "video", "url": _clip(tmp_path, 30)}]
        clip = c.post("/v1/videos/sync", json=refs)
        assert clip.status_code == 200, clip.text
        assert clip.content not in (track.content, with_ref.content, plain.content)
        refs["input_references"] = [{"type": "video", "url": _clip(tmp_path, 30),
                                     "start_time_seconds": 0.25}]      # 24 frames are left
        later = c.post("/v1/videos/sync", json=refs)
        assert later.status_code == 200 and later.content != clip.content
        refs["input_references"][0]["start_time_seconds"] = 1.0        # 6 frames are left
        assert c.post("/v1/videos/sync", json=refs).status_code == 400
        refs["input_references"] = [{"type": "audio", "url": _wav(3), "start_time_seconds": 2.0}]
        gone = c.post("/v1/videos/sync", json=refs)
        assert gone.status_code == 400 and "ends before" in gone.json()["error"]["message"]
        refs["input_references"] = [{"type": "video", "url": _clip(tmp_path, 9)}]
        short = c.post("/v1/videos/sync", json=refs)
        assert short.status_code == 400 and "17 frames" in short.json()["error"]["message"]
        body["input_references"][0]["url"] = "data:image/png;base64,AAAA"
        bad = c.post("/v1/videos/sync", json=body)
        assert bad.status_code == 400 and bad.json()["error"]["param"] == "input_references"


def test_finished_jobs_leave_the_store_by_age_and_by_size():
    """The job store keeps finished videos for `media_config.job_retention` and within
    `media_config.job_store_bytes`: older ones go first; jobs that still run stay."""
    import time
    import types
    from uniserve_v1_b200.server.video_service import VideoJob, VideoService
    cfg, tr, vv, av, enc = _tiny_pipeline()
    svc = VideoService(tr, vv, av, sizes=["256x256"], max_seconds=5, retention_s=100.0,
                       store_bytes=2500)
    plan = types.SimpleNamespace(width=256, height=256, num_frames=8, fps=24, seconds=1.0, seed=0,
                                 task="t2va")
    now = time.time()

    def job(age, nbytes, done=True):
        j = VideoJob("p", plan)
        if done:
            j.state, j.completed_at, j.content = "completed", now - age, b"x" * nbytes
        svc._jobs[j.id] = j
        return j
    old = job(500, 10)                    # past the retention
    a, b, c = job(50, 1000), job(40, 1000), job(30, 1000)
    running = job(0, 0, done=False)
    assert svc.get(old.id) is None
    assert svc.get(a.id) is None          # 3000 bytes > 2500: the oldest content goes
    assert svc.get(b.id) is b and svc.get(c.id) is c and svc.get(running.id) is running
    assert [j.id for j in svc.jobs()] == [b.id, c.id, running.id]
