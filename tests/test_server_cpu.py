"""HTTP API on CPU with the tiny model: chat (stream / non-stream), validation,
auth, admin policy, metrics query, and the video routes end to end (MP4 out)."""
import json

import pytest
import torch
from fastapi.testclient import TestClient

from uniserve_v1_b200.config.policy import Package
from uniserve_v1_b200.engine.engine import LLMEngine
from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
from uniserve_v1_b200.server.app import create_app
from uniserve_v1_b200.server.tokenizer import ByteTokenizer


@pytest.fixture(scope="module")
def chat_client():
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    eng = LLMEngine(model, num_pages=256, max_num_seqs=8, max_model_len=512, use_graphs=False)
    pkg = Package.parse('model = "random:tiny"\nserved_model_name = "tiny"\n')
    app = create_app(package=pkg, engine=eng, tokenizer=ByteTokenizer(1024, 1023),
                     served_model_name="tiny")
    with TestClient(app) as c:
        yield c


def test_basics_and_404(chat_client):
    assert chat_client.get("/health").json()["status"] == "ok"
    assert chat_client.get("/v1/models").json()["data"][0]["id"] == "tiny"
    r = chat_client.get("/nope")
    assert r.status_code == 404 and r.json() == {"detail": "Not Found"}
    assert chat_client.get("/v1/capabilities").status_code == 404      # text deployment


def test_chat_non_stream_and_determinism(chat_client):
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hello"}],
            "max_tokens": 8, "temperature": 0, "ignore_eos": True, "logprobs": True, "top_logprobs": 2}
    a = chat_client.post("/v1/chat/completions", json=body).json()
    b = chat_client.post("/v1/chat/completions", json=body).json()
    assert a["choices"][0]["message"] == b["choices"][0]["message"]
    assert a["usage"]["completion_tokens"] == 8 and a["choices"][0]["finish_reason"] == "length"
    assert len(a["choices"][0]["logprobs"]["content"]) == 8
    assert len(a["choices"][0]["logprobs"]["content"][0]["top_logprobs"]) == 2
    # second run reuses the cached prompt pages
    assert b["usage"]["prompt_tokens_details"]["cached_tokens"] > 0
    body["seed"], body["temperature"], body["top_p"] = 7, 0.9, 0.9
    c = chat_client.post("/v1/chat/completions", json=body).json()
    d = chat_client.post("/v1/chat/completions", json=body).json()
    assert c["choices"][0]["message"] == d["choices"][0]["message"]


def test_chat_stream(chat_client):
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 5,
            "temperature": 0, "stream": True, "ignore_eos": True,
            "stream_options": {"include_usage": True}}
    with chat_client.stream("POST", "/v1/chat/completions", json=body) as r:
        lines = [l for l in r.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    assert chunks[-1]["usage"]["completion_tokens"] == 5
    assert any(c["choices"] and c["choices"][0]["finish_reason"] == "length" for c in chunks)


def test_chat_validation(chat_client):
    r = chat_client.post("/v1/chat/completions", json={"model": "tiny", "messages": [], "x": 1})
    assert r.status_code == 400
    r = chat_client.post("/v1/chat/completions",
                         json={"model": "tiny", "messages": [{"role": "user", "content": "a"}],
                               "unknown_field": 1})
    assert r.status_code == 400 and "unknown_field" in r.json()["error"]["message"]
    r = chat_client.post("/v1/chat/completions",
                         json={"model": "other", "messages": [{"role": "user", "content": "a"}]})
    assert r.status_code == 404 and r.json()["error"]["code"] == "model_not_found"


def test_admin_policy_and_query(chat_client):
    assert chat_client.get("/admin/policy").json()["config"]["served_model_name"] == "tiny"
    r = chat_client.put("/admin/policy", content='model = "random:tiny"\nserved_model_name = "tiny"\n'
                                                 '[kv_cache_config]\nprefix_caching = false\n')
    assert r.status_code == 200 and r.json()["effect"] == "step"
    r = chat_client.put("/admin/policy", content='model = "random:tiny"\ntensor_parallel_size = 2\n')
    assert r.status_code == 409
    r = chat_client.put("/admin/policy", content='modle = "x"\n')
    assert r.status_code == 400
    q = chat_client.get("/admin/query", params={"q": "select kind, count(*) from events group by kind"})
    assert q.status_code == 200 and any(row[0] == "request" for row in q.json()["rows"])
    assert "uniserve_requests_total" in chat_client.get("/metrics").text
    assert chat_client.get("/admin/query", params={"q": "drop table events"}).status_code == 400


def test_api_key():
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    eng = LLMEngine(model, num_pages=64, max_num_seqs=2, max_model_len=128, use_graphs=False)
    pkg = Package.parse('model = "random:tiny"\n[server_config]\napi_key = "sekret"\n')
    app = create_app(package=pkg, engine=eng, tokenizer=ByteTokenizer(1024, 1023),
                     served_model_name="tiny")
    with TestClient(app) as c:
        assert c.get("/health").status_code == 200
        assert c.get("/v1/models").status_code == 401
        assert c.get("/v1/models", headers={"Authorization": "Bearer sekret"}).status_code == 200


def test_video_routes_produce_mp4():
    import cv2
    from uniserve_v1_b200.models.h3_vae import (AudioVaeConfig, AudioVaeDecoder, VideoVaeConfig,
                                                VideoVaeDecoder)
    from uniserve_v1_b200.models.minimax_h3 import H3Config, H3Transformer
    from uniserve_v1_b200.server.video_service import VideoService
    cfg = H3Config.tiny()
    cfg.vae_spatial = 64          # keep the CPU test small: 256x256 -> 4x4 latent
    tr = H3Transformer(cfg, "cpu", torch.float32).init_random(0)
    vc = VideoVaeConfig.tiny()
    vc.latent_channels, vc.spatial = cfg.latent_channels, 64
    vv = VideoVaeDecoder(vc, "cpu", torch.float32).init_random(1)
    av = AudioVaeDecoder(AudioVaeConfig(latent_channels=cfg.audio_channels, decoder_dim=128,
                                        rates=(5, 5, 2, 2, 2, 2, 2), kernels=(9, 9, 4, 4, 4, 4, 4),
                                        res_kernels=(3,), res_dilations=(1,)), "cpu").init_random(2)
    svc = VideoService(tr, vv, av, sizes=["256x256"], max_seconds=5)
    pkg = Package.parse('model = "random:h3:tiny"\nserved_model_name = "FastH3"\n')
    app = create_app(package=pkg, video_service=svc, served_model_name="FastH3")
    with TestClient(app) as c:
        caps = c.get("/v1/capabilities").json()
        assert caps["frame_rule"] == "17n + 5" and caps["sizes"] == ["256x256"]
        bad = c.post("/v1/videos/sync", json={"model": "FastH3", "prompt": "x", "seconds": 2})
        assert bad.status_code == 400 and bad.json()["error"]["param"] == "seconds"
        bad = c.post("/v1/videos/sync", json={"model": "FastH3", "prompt": "x", "guidance_scale": 2})
        assert bad.status_code == 400
        r = c.post("/v1/videos/sync", json={"model": "FastH3", "prompt": "a stream in a forest",
                                            "size": "256x256", "seconds": 4, "seed": 1000})
        assert r.status_code == 200, r.text
        assert r.headers["x-video-size"] == "256x256" and r.headers["x-video-num-frames"] == "107"
        assert r.headers["x-video-fps"] == "24" and r.content[4:8] == b"ftyp"
        open("/tmp/_us_test.mp4", "wb").write(r.content)
        cap = cv2.VideoCapture("/tmp/_us_test.mp4")
        assert cap.isOpened() and int(cap.get(cv2.CAP_PROP_FRAME_COUNT)) == 107
        ok, frame = cap.read()
        assert ok and frame.shape == (256, 256, 3)
        job = c.post("/v1/videos", json={"model": "FastH3", "prompt": "x", "num_frames": 107,
                                         "size": "256x256", "seed": 5}).json()
        assert job["status"] in ("queued", "in_progress", "completed") and job["num_frames"] == 107
        import time
        for _ in range(600):
            st = c.get(f"/v1/videos/{job['id']}").json()
            if st["status"] in ("completed", "failed"):
                break
            time.sleep(0.1)
        assert st["status"] == "completed", st
        assert c.get(f"/v1/videos/{job['id']}/content").content[4:8] == b"ftyp"
        assert c.delete(f"/v1/videos/{job['id']}").json()["deleted"] is True
        assert c.get(f"/v1/videos/{job['id']}").status_code == 404


def test_chat_on_the_dense_state_engine():
    """The hybrid (gated delta net) family behind the same chat routes."""
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.models.qwen3_5 import Qwen35MoeModel
    model = Qwen35MoeModel(Qwen35MoeModel.tiny_config(), "cpu", torch.float32).init_random(seed=0)
    eng = DenseStateEngine(model, max_num_seqs=4, max_model_len=256)
    pkg = Package.parse('model = "random:tiny"\nserved_model_name = "hybrid"\n')
    app = create_app(package=pkg, engine=eng, tokenizer=ByteTokenizer(1024, 1023),
                     served_model_name="hybrid")
    with TestClient(app) as c:
        body = {"model": "hybrid", "messages": [{"role": "user", "content": "hello"}],
                "max_tokens": 6, "temperature": 0, "ignore_eos": True}
        a = c.post("/v1/chat/completions", json=body).json()
        b = c.post("/v1/chat/completions", json=body).json()
        assert a["choices"][0]["message"] == b["choices"][0]["message"]
        assert a["usage"]["completion_tokens"] == 6
        body.update(stream=True, temperature=0.8, seed=3)
        with c.stream("POST", "/v1/chat/completions", json=body) as r:
            lines = [l for l in r.iter_lines() if l.startswith("data: ")]
        assert lines[-1] == "data: [DONE]" and len(lines) >= 4


def test_chat_with_speculative_decoding_gives_the_same_answers():
    """`speculative_config.num_draft_tokens` turns on prompt-lookup drafting in the engine
    loop; greedy answers are unchanged and sampled requests fall back to ordinary steps."""
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    answers = []
    for toml in ('model = "random:tiny"\nserved_model_name = "tiny"\n',
                 'model = "random:tiny"\nserved_model_name = "tiny"\n'
                 '[speculative_config]\nnum_draft_tokens = 3\n'):
        eng = LLMEngine(model, num_pages=256, max_num_seqs=8, max_model_len=512, use_graphs=False)
        app = create_app(package=Package.parse(toml), engine=eng, tokenizer=ByteTokenizer(1024, 1023),
                         served_model_name="tiny")
        with TestClient(app) as c:
            out = []
            for extra in ({"temperature": 0}, {"temperature": 0.8, "seed": 3}):
                body = dict({"model": "tiny", "max_tokens": 24, "ignore_eos": True,
                             "messages": [{"role": "user", "content": "abcabcabcabc abcabc"}]}, **extra)
                out.append(c.post("/v1/chat/completions", json=body).json()["choices"][0]["message"])
            answers.append(out)
            spec = eng.spec_stats
    assert answers[0] == answers[1]
    assert spec["steps"] > 0 and spec["proposed"] > 0


def test_video_job_resumes_from_its_last_step_boundary():
    """A denoising step that fails once: the job continues from the trajectory saved at the
    previous step boundary and produces the bytes of an undisturbed run."""
    from uniserve_v1_b200.models.h3_vae import (AudioVaeConfig, AudioVaeDecoder, VideoVaeConfig,
                                                VideoVaeDecoder)
    from uniserve_v1_b200.models.minimax_h3 import H3Config, H3Transformer
    from uniserve_v1_b200.server.video_rules import plan_request
    from uniserve_v1_b200.server.protocol import VideoGenerationRequest
    from uniserve_v1_b200.server.video_service import VideoService
    cfg = H3Config.tiny()
    cfg.vae_spatial = 64
    tr = H3Transformer(cfg, "cpu", torch.float32).init_random(0)
    vc = VideoVaeConfig.tiny()
    vc.latent_channels, vc.spatial = cfg.latent_channels, 64
    vv = VideoVaeDecoder(vc, "cpu", torch.float32).init_random(1)
    av = AudioVaeDecoder(AudioVaeConfig(latent_channels=cfg.audio_channels, decoder_dim=128,
                                        rates=(5, 5, 2, 2, 2, 2, 2), kernels=(9, 9, 4, 4, 4, 4, 4),
                                        res_kernels=(3,), res_dilations=(1,)), "cpu").init_random(2)

    def service():
        return VideoService(tr, vv, av, sizes=["256x256"], max_seconds=5)
    req = VideoGenerationRequest(model="FastH3", prompt="a stream", size="256x256", seconds=4,
                                 seed=7)
    svc = service()
    plan = plan_request(req, svc.sizes, svc.max_seconds, svc.steps)
    want = svc.submit("a stream", plan)
    want._done.wait(300)
    assert want.state == "completed" and want.resumed_from is None and not svc.latent_pool
    svc2 = service()
    inner, calls = svc2.denoiser.step, {"n": 0}

    def flaky(st):
        calls["n"] += 1
        if calls["n"] == 3:
            raise RuntimeError("injected step failure")
        return inner(st)
    svc2.denoiser.step = flaky
    job = svc2.submit("a stream", plan)
    job._done.wait(300)
    assert job.state == "completed", job.error
    assert job.resumes == 1 and job.resumed_from == 2          # two steps were kept
    assert job.content == want.content
    assert calls["n"] == svc2.steps + 1 and not svc2.latent_pool


def _hybrid_mm_engine():
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.models.qwen3_5 import Qwen35MoeModel
    from uniserve_v1_b200.models.qwen3_vl_vision import Qwen3VLVisionTower, VisionConfig
    cfg = Qwen35MoeModel.tiny_config()
    cfg.mrope_section, cfg.image_token_id = (2, 1, 1), 1000
    model = Qwen35MoeModel(cfg, "cpu", torch.float32).init_random(seed=0)
    vc = VisionConfig(depth=2, hidden_size=32, intermediate_size=48, num_heads=2, patch_size=16,
                      temporal_patch_size=2, spatial_merge_size=2, out_hidden_size=64,
                      num_position_embeddings=16, deepstack_visual_indexes=[])
    tower = Qwen3VLVisionTower(vc, "cpu", torch.float32)
    g = torch.Generator().manual_seed(1)

    class Rand:
        def names(self): return ["patch_embed.proj.weight"]
        def get(self, n):
            shapes = {"patch_embed.proj.weight": (32, 3, 2, 16, 16), "patch_embed.proj.bias": (32,),
                      "pos_embed.weight": (16, 32)}
            if n in shapes:
                return torch.randn(*shapes[n], generator=g) * 0.05
            wide = 32 * 4
            dims = {"attn.qkv.weight": (96, 32), "attn.qkv.bias": (96,), "attn.proj.weight": (32, 32),
                    "attn.proj.bias": (32,), "mlp.linear_fc1.weight": (48, 32),
                    "mlp.linear_fc1.bias": (48,), "mlp.linear_fc2.weight": (32, 48),
                    "mlp.linear_fc2.bias": (32,), "merger.norm.weight": (32,), "merger.norm.bias": (32,),
                    "merger.linear_fc1.weight": (wide, wide), "merger.linear_fc1.bias": (wide,),
                    "merger.linear_fc2.weight": (64, wide), "merger.linear_fc2.bias": (64,)}
            for k, shp in dims.items():
                if n.endswith(k):
                    return torch.randn(*shp, generator=g) * 0.05
            return torch.ones(32) if n.endswith("weight") else torch.zeros(32)     # block norms
    tower.load_state(Rand(), prefix="")
    return DenseStateEngine(model, max_num_seqs=4, max_model_len=512, tower=tower), model, tower


def test_chat_with_an_image_on_the_hybrid_family():
    """An `image_url` part (data URL) is decoded, cut into patch rows, run through the vision
    tower and spliced into the prompt; the answer is the model's own multimodal decoding.
    A deployment without a tower refuses images."""
    import base64
    import io
    import numpy as np
    from PIL import Image
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.models.qwen3_5 import Qwen35MoeModel, Qwen35Multimodal
    from uniserve_v1_b200.models.qwen3_vl_vision import Qwen3VLVisionTower, VisionConfig
    from uniserve_v1_b200.server import images as IM
    eng, model, tower = _hybrid_mm_engine()
    pkg = Package.parse('model = "random:tiny"\nserved_model_name = "hybrid"\n')
    tok = ByteTokenizer(1024, 1023)
    app = create_app(package=pkg, engine=eng, tokenizer=tok, served_model_name="hybrid")
    img = np.random.RandomState(0).randint(0, 256, (64, 96, 3), dtype=np.uint8)
    buf = io.BytesIO()
    Image.fromarray(img).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    body = {"model": "hybrid", "max_tokens": 5, "temperature": 0, "ignore_eos": True,
            "messages": [{"role": "user", "content": [{"type": "text", "text": "what is this? "},
                                                      {"type": "image_url", "image_url": {"url": url}}]}]}
    with TestClient(app) as c:
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 200, r.text
        got = r.json()
        n_img = (64 // 32) * (96 // 32)
        assert got["usage"]["completion_tokens"] == 5
        # the same prompt decoded by the model directly
        rows, grid = IM.preprocess(img)
        rid = next(iter(eng.requests))
        prompt_ids = eng.requests[rid].prompt_ids
        assert prompt_ids.count(1000) == n_img and got["usage"]["prompt_tokens"] == len(prompt_ids)
        want = Qwen35Multimodal(model, tower).generate(prompt_ids, rows, [grid], 5)
        assert eng.requests[rid].output_ids == want
        bad = dict(body, messages=[{"role": "user", "content": [
            {"type": "image_url", "image_url": {"url": "https://example.com/x.png"}}]}])
        assert c.post("/v1/chat/completions", json=bad).status_code == 400
    plain = create_app(package=pkg, engine=DenseStateEngine(model), tokenizer=tok,
                       served_model_name="hybrid")
    with TestClient(plain) as c:
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 400 and "images" in r.json()["error"]["message"]


def test_dense_state_engine_shapes_logits_like_the_paged_engine():
    """Penalties, bias, bans, minimum length and log-probabilities on the hybrid family go
    through the same shaping code as on the paged engine."""
    from uniserve_v1_b200.engine.dense_state import DenseStateEngine
    from uniserve_v1_b200.models.qwen3_5 import Qwen35MoeModel
    model = Qwen35MoeModel(Qwen35MoeModel.tiny_config(), "cpu", torch.float32).init_random(seed=0)
    eng = DenseStateEngine(model, max_num_seqs=4, max_model_len=256)
    pkg = Package.parse('model = "random:tiny"\nserved_model_name = "hybrid"\n')
    app = create_app(package=pkg, engine=eng, tokenizer=ByteTokenizer(1024, 1023),
                     served_model_name="hybrid")
    with TestClient(app) as c:
        base = {"model": "hybrid", "messages": [{"role": "user", "content": "hello"}],
                "max_tokens": 6, "temperature": 0, "ignore_eos": True}
        plain = c.post("/v1/chat/completions", json=base).json()
        lp = c.post("/v1/chat/completions", json=dict(base, logprobs=True, top_logprobs=3)).json()
        assert lp["choices"][0]["message"] == plain["choices"][0]["message"]
        ent = lp["choices"][0]["logprobs"]["content"]
        assert len(ent) == 6 and len(ent[0]["top_logprobs"]) == 3 and ent[0]["logprob"] <= 0.0
        first = eng.requests[next(reversed(eng.requests))].output_ids[0]
        banned = c.post("/v1/chat/completions", json=dict(base, logit_bias={str(first): -100})).json()
        rid = next(reversed(eng.requests))
        assert eng.requests[rid].output_ids[0] != first and banned["usage"]["completion_tokens"] == 6
        rep = c.post("/v1/chat/completions", json=dict(base, repetition_penalty=1.8,
                                                       presence_penalty=1.0)).json()
        assert rep["usage"]["completion_tokens"] == 6


def test_video_frames_become_timestamped_images(tmp_path):
    """A `video_url` part: frames are sampled, cut into temporal patches and enter the prompt as
    one timestamped placeholder group per patch; the rows equal the image path's rows for the
    same frame pair."""
    import cv2
    import numpy as np
    from uniserve_v1_b200.server import images as IM
    from uniserve_v1_b200.server.chat import _flatten_content
    path = str(tmp_path / "clip.avi")
    wr = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*"MJPG"), 8.0, (96, 64))
    assert wr.isOpened()
    rng = np.random.RandomState(0)
    base = rng.randint(0, 256, (64, 96, 3), dtype=np.uint8)
    for i in range(16):
        wr.write(np.roll(base, 4 * i, axis=1))
    wr.release()
    IM.set_media_directory(tmp_path)
    frames, secs = IM.load_video("file://" + path, fps=2.0)
    assert frames.shape == (4, 64, 96, 3) and secs == [0.0, 0.5, 1.0, 1.5]
    rows, grid = IM.preprocess_video(frames)
    assert grid == (2, 4, 6) and rows.shape == (48, 3 * 2 * 16 * 16)
    # temporal patch 0 holds frames 0 and 1: channel-major, then the two frames
    one, g1 = IM.patch_rows(((torch.from_numpy(frames[:2].copy()).permute(0, 3, 1, 2).float() / 255)
                             - 0.5) / 0.5, 16, 2, 2)
    assert g1 == (1, 4, 6) and torch.equal(one, rows[:24])
    assert IM.video_prompt(secs) == ("<0.2 seconds><|vision_start|><|image_pad|><|vision_end|>"
                                     "<1.2 seconds><|vision_start|><|image_pad|><|vision_end|>")
    assert _flatten_content([{"type": "text", "text": "see "},
                             {"type": "video_url", "video_url": {"url": "file://x"}}]) == \
        "see <|vision_start|><|video_pad|><|vision_end|>"
    assert IM.collect_media([{"role": "user", "content": [
        {"type": "video_url", "video_url": {"url": "file://" + path}},
        {"type": "image_url", "image_url": "data:x"}]}]) == [("video", "file://" + path),
                                                              ("image", "data:x")]


def test_chat_with_a_video_on_the_hybrid_family(tmp_path):
    """End to end: a `video_url` file is sampled, every temporal patch becomes a timestamped
    image group of the prompt, and the answer is the model's own decoding of those ids and rows."""
    import cv2
    import numpy as np
    from uniserve_v1_b200.models.qwen3_5 import Qwen35Multimodal
    from uniserve_v1_b200.server import images as IM
    path = str(tmp_path / "clip.avi")
    wr = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*"MJPG"), 8.0, (96, 64))
    base = np.random.RandomState(1).randint(0, 256, (64, 96, 3), dtype=np.uint8)
    for i in range(16):
        wr.write(np.roll(base, 4 * i, axis=1))
    wr.release()
    eng, model, tower = _hybrid_mm_engine()
    pkg = Package.parse('model = "random:tiny"\nserved_model_name = "hybrid"\n'
                        f'[media_config]\ndirectory = "{tmp_path}"\n')
    app = create_app(package=pkg, engine=eng, tokenizer=ByteTokenizer(1024, 1023),
                     served_model_name="hybrid")
    body = {"model": "hybrid", "max_tokens": 4, "temperature": 0, "ignore_eos": True,
            "messages": [{"role": "user", "content": [
                {"type": "text", "text": "what happens? "},
                {"type": "video_url", "video_url": {"url": "file://" + path}}]}]}

    def with_url(url, kind="video_url"):
        return dict(body, messages=[{"role": "user", "content": [
            {"type": "text", "text": "what happens? "}, {"type": kind, kind: {"url": url}}]}])
    with TestClient(app) as c:
        # file:// is read below the media directory only: no traversal, no symbolic link out
        # of it, no host part, and a missing file is the request's own error (400, not 500)
        import os
        outside = tmp_path.parent / "outside.png"
        outside.write_bytes(b"secret")
        os.symlink(outside, tmp_path / "link.png")
        for url, kind in ((f"file://{tmp_path}/../outside.png", "image_url"),
                          (f"file://{tmp_path}/link.png", "image_url"),
                          ("file:///etc/passwd", "image_url"),
                          (f"file://otherhost{path}", "video_url"),
                          (f"file://{tmp_path}/missing.avi", "video_url"),
                          (f"file://{tmp_path}/missing.png", "image_url")):
            bad = c.post("/v1/chat/completions", json=with_url(url, kind))
            assert bad.status_code == 400, (url, bad.text)
            assert bad.json()["error"]["type"] in ("input_error", "invalid_request_error")
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 200, r.text
        rid = next(iter(eng.requests))
        req = eng.requests[rid]
        frames, secs = IM.load_video("file://" + path)
        rows, (gt, gh, gw) = IM.preprocess_video(frames)
        assert req.prompt_ids.count(1000) == gt * (gh // 2) * (gw // 2) == 12
        grids = [(1, gh, gw)] * gt
        want = Qwen35Multimodal(model, tower).generate(req.prompt_ids, rows, grids, 4)
        assert req.output_ids == want and r.json()["usage"]["completion_tokens"] == 4
    # without a media directory every file:// URL is refused
    bare = create_app(package=Package.parse('model = "random:tiny"\nserved_model_name = "hybrid"\n'),
                      engine=_hybrid_mm_engine()[0], tokenizer=ByteTokenizer(1024, 1023),
                      served_model_name="hybrid")
    with TestClient(bare) as c:
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 400 and "media_config.directory" in r.text


def test_mp4_built_in_memory_is_the_file_form_byte_for_byte(tmp_path):
    """`write_mp4` without a path builds the file in memory (pictures encoded in parallel,
    copied into a bytes object of the exact size); with a path it writes the file: the same
    bytes, edge macroblocks and the audio track included."""
    from uniserve_v1_b200.ops import media as M
    g = torch.Generator().manual_seed(0)
    F_, H, W = 5, 48, 70                      # not multiples of 16
    y = torch.randint(0, 256, (F_, H, W), dtype=torch.uint8, generator=g)
    u = torch.randint(0, 256, (F_, H // 2, W // 2), dtype=torch.uint8, generator=g)
    v = torch.randint(0, 256, (F_, H // 2, W // 2), dtype=torch.uint8, generator=g)
    y[1, :3] = 0                              # runs of zero bytes: emulation prevention bytes
    pcm = torch.randint(-1000, 1000, (3200, 2), dtype=torch.int16, generator=g)
    mem = M.write_mp4(y, u, v, 24, pcm, 32000)
    path = tmp_path / "clip.mp4"
    assert M.write_mp4(y, u, v, 24, pcm, 32000, path=str(path)) == b""
    assert isinstance(mem, bytes) and mem == path.read_bytes()
    assert mem[4:8] == b"ftyp" and b"moov" in mem[-4096:] and b"avcC" in mem
    assert M.write_mp4(y, u, v, 24) == M.write_mp4(y, u, v, 24, None)     # video only


def test_media_larger_than_the_deployments_bound_are_refused(tmp_path):
    """`media_config.max_request_bytes` bounds every medium: a `data:` URL is refused before
    it is decoded, a `file://` medium by its size; media within the bound load as before."""
    import base64
    import io
    import numpy as np
    import pytest
    from PIL import Image
    from uniserve_v1_b200.server import images
    buf = io.BytesIO()
    Image.fromarray((np.arange(64 * 64 * 3) % 251).astype(np.uint8).reshape(64, 64, 3)).save(buf, "PNG")
    raw = buf.getvalue()
    url = "data:image/png;base64," + base64.b64encode(raw).decode()
    (tmp_path / "a.png").write_bytes(raw)
    images.set_media_directory(str(tmp_path))
    try:
        images.set_media_limit(len(raw))
        assert images.load_image(url).shape == (64, 64, 3)
        assert images.load_image(f"file://{tmp_path}/a.png").shape == (64, 64, 3)
        images.set_media_limit(len(raw) - 8)
        for u in (url, f"file://{tmp_path}/a.png"):
            with pytest.raises(ValueError, match="larger than the deployment accepts"):
                images.load_image(u)
        with pytest.raises(ValueError, match="larger than the deployment accepts"):
            images.load_video("data:video/mp4;base64," + base64.b64encode(raw).decode())
        with pytest.raises(ValueError, match="larger than the deployment accepts"):
            images.load_video(f"file://{tmp_path}/a.png")
    finally:
        images.set_media_limit(None)
        images.set_media_directory(None)
