"""The released control / routing programs under the metered program host, the control
loop that applies what they write, and the epoch update machine (prepare, switch, trial,
commit / roll back) on CPU engines."""
import json
import time

import pytest
import torch

from uniserve_v1_b200.config.policy import Package
from uniserve_v1_b200.engine.program import ProgramHost
from uniserve_v1_b200.programs import NAMES, source_of


def host(name, **args):
    return ProgramHost(source_of(name), name, args=args)


def test_chunk_program_halves_and_doubles_within_bounds():
    h = host("uniserve:chunk", tpot=0.05, ttft=1.0, low=512, high=8192, pause=60.0)
    r = {"tpot_p99": {"a": 0.08}, "ttft_p99": {"a": 0.2}, "chunk": 2048}
    assert h.call("step", r, 0.0) == {"scheduler_config.chunked_prefill_size": 1024}
    r = {"tpot_p99": {"a": 0.08}, "ttft_p99": {}, "chunk": 512}
    assert h.call("step", r, 0.0) == {}                               # already at `low`
    r = {"tpot_p99": {"a": 0.01}, "ttft_p99": {"a": 2.0}, "chunk": None,
         "max_num_batched_tokens": 4096}
    assert h.call("step", r, 0.0) == {"scheduler_config.chunked_prefill_size": 8192}
    h.call("rolled_back", 10.0)                                       # held back for `pause`
    assert h.call("step", r, 30.0) == {}
    state = h.save_state()
    h2 = host("chunk", tpot=0.05, ttft=1.0, low=512, high=8192, pause=60.0)
    h2.restore_state(state)
    assert h2.call("step", r, 30.0) == {} and h2.call("step", r, 80.0) != {}


def test_expert_order_program_balances_ranks_and_keeps_slots():
    h = host("expert-order", ranks=2, imbalance=1.1)
    tokens = [100, 90, 5, 5, 80, 70, 5, 5]          # rank 0 holds experts 0..3: 200 vs 160
    out = h.call("step", {"tokens": {"3": tokens}, "order": {}}, 0.0)
    order = out["moe_config.expert_order"]["3"]
    assert sorted(order) == list(range(8))
    loads = [sum(tokens[e] for e in order[:4]), sum(tokens[e] for e in order[4:])]
    assert max(loads) < 200 and abs(loads[0] - loads[1]) <= 20
    stay = [e for i, e in enumerate(order) if e == i]
    assert len(stay) >= 4                            # experts that stay keep their slot
    assert h.call("step", {"tokens": {"3": [10] * 8}, "order": {}}, 0.0) == {}


def test_role_and_ttft_and_layout_programs():
    h = host("role", ttft=1.0, tpot=0.05, room=0.2, interval=300.0, keep=1)
    r = {"ttft_p99": 2.0, "tpot_p99": 0.02, "running": {"a": 5, "b": 1, "c": 9},
         "roles": {"a": "decode", "b": "decode", "c": "prefill"}}
    assert h.call("step", r, 1000.0) == {"replicas.b.role": "prefill"}
    assert h.call("step", r, 1100.0) == {}                             # within `interval`
    r["roles"] = {"a": "decode", "c": "prefill"}
    assert h.call("step", r, 2000.0) == {}                             # `keep` one decode replica
    t = host("ttft", rate=1000.0, page=16)
    reps = [{"id": "p0", "role": "prefill", "remaining": 0.5, "queued_prefill_tokens": 4000,
             "running": 2, "reservable_pages": 0},
            {"id": "p1", "role": "prefill", "remaining": 0.0, "queued_prefill_tokens": 100,
             "running": 3, "reservable_pages": 0},
            {"id": "d0", "role": "decode", "running": 7, "reservable_pages": 1000},
            {"id": "d1", "role": "decode", "running": 1, "reservable_pages": 2}]
    got = t.call("route", {"prompt_tokens": 800, "hits": {"p0": 800}}, reps)
    assert got == {"prefill": "p1", "decode": "d0"}                    # d1 cannot hold the pages
    got = t.call("route", {"prompt_tokens": 800, "hits": {"p0": 800}},
                 [dict(reps[0], queued_prefill_tokens=0, remaining=0.0)] + reps[1:])
    assert got["prefill"] == "p0"
    lay = host("layout", layouts={"tp8": {"tensor_parallel_size": 8},
                                  "tp4": {"tensor_parallel_size": 4}},
               bounds=[32], samples=2, margin=0.05, weight=0.5)
    base = {"running_mean": 10.0, "served_window": True}
    for _ in range(2):
        assert lay.call("step", dict(base, token_rate=1000.0,
                                     config={"tensor_parallel_size": 8}), 0.0) == {}
    for _ in range(2):
        lay.call("step", dict(base, token_rate=1500.0, config={"tensor_parallel_size": 4}), 0.0)
    assert lay.call("step", dict(base, token_rate=1000.0, config={"tensor_parallel_size": 8}),
                    0.0) == {"tensor_parallel_size": 4}
    for n in NAMES:
        assert source_of(n)


def test_backend_program_opens_and_closes_a_probe():
    b = host("backend", slowdown=0.1, probe=30.0, interval=600.0, backends=["tcgen05", "simt"],
             op="paged_attention")
    cfg = {"profiling_config.fence_modules": None, "profiling_config.fence_probes": False,
           "profiling_config.fence_probes_off": None}
    slow = {"decode_p50_window": 0.02, "decode_p50_baseline": 0.015, "config": cfg}
    opened = b.call("step", slow, 1000.0)
    assert opened["profiling_config.fence_probes"] is True
    assert b.call("step", slow, 1010.0) == {}                          # the probe is measuring
    closed = b.call("step", dict(slow, probe={"modules": {"Qwen.Attention": 0.004, "Qwen.MoE": 0.01},
                                              "keys": ["d128p16"], "backend": "tcgen05"}), 1031.0)
    assert closed["profiling_config.fence_probes"] is False            # options go back
    assert b.call("step", slow, 1100.0) == {}                          # `interval` between probes


def test_control_loop_applies_a_program_change_and_keeps_state(tmp_path):
    from uniserve_v1_b200.server.control import ControlLoop
    from uniserve_v1_b200.server.observation import ObservationStore
    text = ('model = "random:tiny"\nmax_num_batched_tokens = 4096\n[programs.chunk]\n'
            'source = "uniserve:chunk"\nperiod = "10s"\n'
            'args = { tpot = "50ms", ttft = "1s", low = 512, high = 8192 }\n')
    box = {"pkg": Package.parse(text)}
    obs = ObservationStore()
    now = [1000.0]
    applied = []

    def apply(changes):
        box["pkg"] = box["pkg"].with_options(changes)
        applied.append(changes)
        return True
    loop = ControlLoop(lambda: box["pkg"], obs, apply, str(tmp_path), clock=lambda: now[0])
    assert list(loop.hosts) == ["chunk"]
    for _ in range(20):
        obs.observe("uniserve_tpot_seconds", 0.09, {"replica": "r0"})
    obs.db.execute("update stats set ts = 1005.0")
    assert loop.tick() == []                                           # its period has not passed
    now[0] = 1011.0
    done = loop.tick()
    assert done and applied == [{"scheduler_config.chunked_prefill_size": 4096}]
    assert box["pkg"].scheduler_config.chunked_prefill_size == 4096
    assert (tmp_path / "chunk.state").exists()
    # a program that runs past its fuel is ended; serving options stay as they are
    bad = Package.parse('model = "random:tiny"\n[scheduler_config.policy_budget]\ncall_fuel = 50\n'
                        '[programs.spin]\nsource = "spin.py"\nperiod = "1s"\n', tmp_path)
    (tmp_path / "spin.py").write_text("def step(r, now):\n    while True:\n        pass\n")
    lp = ControlLoop(lambda: bad, obs, lambda c: True, None, clock=lambda: now[0])
    now[0] += 5
    assert lp.tick() == [] and "spin" in lp.ended and not lp.hosts


def _engine(max_len=128):
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    return LLMEngine(model, num_pages=128, max_num_seqs=8, max_model_len=max_len, use_graphs=False)


def test_epoch_update_switches_drains_commits_and_rolls_back():
    """PUT /admin/policy with an epoch-effect change on a deployment that can build engines:
    the target is prepared while serving goes on, a request in flight at the switch still
    completes with the tokens one engine would give, the trial commits; a second update whose
    target fails its first step rolls back to the previous engine; a target that cannot be
    built leaves everything as it was."""
    from fastapi.testclient import TestClient
    from uniserve_v1_b200.server.app import create_app
    from uniserve_v1_b200.server.tokenizer import ByteTokenizer
    base = 'model = "random:tiny"\nserved_model_name = "tiny"\n'
    upd = '[update_config]\ntrial = "0.3s"\ndrain_s = 0.05\n'
    built = []

    def builder(pkg):
        if pkg.max_model_len == 333:
            raise RuntimeError("no memory for the target")
        eng = _engine(max_len=pkg.max_model_len or 128)
        if pkg.max_model_len == 111:
            def boom():
                raise RuntimeError("target broke")
            eng.step = boom
        built.append(eng)
        return eng
    first = _engine()
    app = create_app(package=Package.parse(base + upd), engine=first,
                     tokenizer=ByteTokenizer(1024, 1023), served_model_name="tiny",
                     engine_builder=builder)
    body = {"model": "tiny", "messages": [{"role": "user", "content": "count with me"}],
            "max_tokens": 24, "temperature": 0, "ignore_eos": True}
    with TestClient(app) as c:
        want = c.post("/v1/chat/completions", json=body).json()["choices"][0]["message"]["content"]
        r = c.put("/admin/policy", content=base + "max_model_len = 256\n" + upd)
        assert r.status_code == 202 and r.json()["update"] == "preparing"
        # a request that is admitted around the switch gives the same answer
        got = c.post("/v1/chat/completions", json=body).json()["choices"][0]["message"]["content"]
        assert got == want
        for _ in range(100):
            ph = c.get("/admin/update").json()
            if ph["phase"] == "committed":
                break
            time.sleep(0.05)
        assert ph["phase"] == "committed" and ph["history"] == ["preparing", "switching", "trial",
                                                                 "committed"]
        svc = app.state.s.service
        assert svc.engine is built[0] and app.state.s.package.max_model_len == 256
        # a target that breaks on trial: back to the engine that served before
        r = c.put("/admin/policy", content=base + "max_model_len = 111\n" + upd)
        assert r.status_code == 202
        time.sleep(0.2)
        got = c.post("/v1/chat/completions", json=body).json()["choices"][0]["message"]["content"]
        assert got == want
        for _ in range(100):
            ph = c.get("/admin/update").json()
            if ph["phase"] in ("rolled_back", "committed"):
                break
            time.sleep(0.05)
        assert ph["phase"] == "rolled_back" and "target" in ph["reason"]
        assert svc.engine is built[0] and app.state.s.package.max_model_len == 256
        # a target that cannot be built: abandoned, nothing changed
        r = c.put("/admin/policy", content=base + "max_model_len = 333\n" + upd)
        assert r.status_code == 202
        for _ in range(100):
            ph = c.get("/admin/update").json()
            if ph["phase"] == "abandoned":
                break
            time.sleep(0.05)
        assert ph["phase"] == "abandoned" and svc.engine is built[0]
        events = c.get("/admin/query", params={"q": "select fields from events where kind = 'update'"}
                       ).json()["rows"]
        assert len(events) >= 6


def test_sleep_and_wake_keep_the_queue_and_give_the_same_tokens():
    """POST /admin/sleep frees the KV cache (level 1) and the weights (level 2) while the
    process and its queue stay; a request sent while asleep is answered after /admin/wake with
    the tokens an engine that never slept gives."""
    import threading
    from fastapi.testclient import TestClient
    from uniserve_v1_b200.server.app import create_app
    from uniserve_v1_b200.server.tokenizer import ByteTokenizer
    eng = _engine()
    app = create_app(package=Package.parse('model = "random:tiny"\nserved_model_name = "tiny"\n'),
                     engine=eng, tokenizer=ByteTokenizer(1024, 1023), served_model_name="tiny")
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}],
            "max_tokens": 12, "temperature": 0, "ignore_eos": True}
    with TestClient(app) as c:
        want = c.post("/v1/chat/completions", json=body).json()["choices"][0]["message"]["content"]
        for level in (1, 2):
            r = c.post("/admin/sleep", params={"level": level})
            assert r.status_code == 200 and r.json()["freed_bytes"] > 0
            assert eng.runner.kv_caches is None and c.get("/health").json()["asleep"] == level
            if level == 2 and eng.device.type == "cuda":      # host copies only of GPU weights
                assert eng.model.embed is None
            got = {}
            t = threading.Thread(target=lambda: got.update(
                r=c.post("/v1/chat/completions", json=body).json()))
            t.start()
            time.sleep(0.3)
            assert not got                                    # queued, not refused
            assert c.post("/admin/wake").json()["was"] == level
            t.join(timeout=60)
            assert got["r"]["choices"][0]["message"]["content"] == want
        assert c.post("/admin/sleep", params={"level": 3}).status_code == 400


def test_otlp_push_resends_what_a_refused_push_carried():
    from uniserve_v1_b200.server.export import OtlpPusher
    from uniserve_v1_b200.server.observation import ObservationStore
    obs = ObservationStore()
    sent, refuse = [], [True]

    def post(url, body, timeout):
        if refuse[0]:
            return 503
        sent.append((url, body))
        return 200
    p = OtlpPusher(obs, "http://collector:4318/", deployment="d", post=post)
    obs.inc("uniserve_requests_total", {"outcome": "ok"})
    obs.set("uniserve_running_requests", 3)
    obs.observe("uniserve_ttft_seconds", 0.25, {"replica": "r0"})
    obs.snapshot()
    obs.event("update", phase="committed")
    assert p.push_once() is False and p.failures == 1 and not sent
    obs.observe("uniserve_ttft_seconds", 0.5, {"replica": "r0"})
    refuse[0] = False
    assert p.push_once() is True
    urls = [u for u, _ in sent]
    assert urls == ["http://collector:4318/v1/metrics", "http://collector:4318/v1/logs"]
    metrics = {m["name"]: m for m in
               sent[0][1]["resourceMetrics"][0]["scopeMetrics"][0]["metrics"]}
    assert metrics["uniserve_requests_total"]["sum"]["isMonotonic"] is True
    assert len(metrics["uniserve_ttft_seconds"]["gauge"]["dataPoints"]) == 2     # both observations
    rec = sent[1][1]["resourceLogs"][0]["scopeLogs"][0]["logRecords"][0]
    assert rec["body"]["stringValue"] == "update"
    sent.clear()
    assert p.push_once() is True and not sent                                  # nothing new


def test_kv_events_follow_commits_reuse_and_flush():
    """An engine with a publisher: the pages a prompt fills are announced as BlockStored with
    SGLang's chained hashes, a second request with the same prefix stores only its new pages,
    pages handed out again are BlockRemoved, a flush clears."""
    import msgpack
    import struct
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.server.export import KvEventPublisher, block_digest, block_hash
    eng = _engine()
    frames = []
    eng.blocks.kv_events = KvEventPublisher(None, rank=2, block_size=16, send=frames.append)
    prompt = [(11 * i) % 1000 for i in range(50)]
    sp = SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True)
    eng.generate([prompt], sp)
    batches = [msgpack.unpackb(f[2]) for f in frames]
    assert [struct.unpack(">Q", f[1])[0] for f in frames] == list(range(len(frames)))
    assert frames[0][0] == b"kv-events" and batches[0][2] == 2
    events = [e for b in batches for e in b[1]]
    assert events[0]["type"] == "AllBlocksCleared"
    stored = [e for e in events if e["type"] == "BlockStored"]
    d0 = block_digest(None, prompt[:16])
    d1 = block_digest(d0, prompt[16:32])
    d2 = block_digest(d1, prompt[32:48])
    hashes = [h for e in stored for h in e["block_hashes"]]
    assert hashes[:3] == [block_hash(d0), block_hash(d1), block_hash(d2)]
    assert stored[0]["parent_block_hash"] is None and stored[0]["block_size"] == 16
    assert stored[0]["token_ids"][:16] == prompt[:16] and stored[0]["medium"] == "GPU"
    n0 = len(stored)
    eng.generate([prompt[:32] + [7] * 20], sp)        # shares two pages, fills one new
    events = [e for f in frames for e in msgpack.unpackb(f[2])[1]]
    new = [e for e in events if e["type"] == "BlockStored"][n0:]
    assert new and new[0]["parent_block_hash"] == block_hash(d1)
    eng.blocks.flush()
    eng.blocks.kv_events.flush()
    assert msgpack.unpackb(frames[-1][2])[1][-1]["type"] == "AllBlocksCleared"
