"""Device quotas: the ledger's rules, the engine's reservations, and an epoch update whose target
does not fit (crates/storage-server/src/quota.rs, reference project path, for the rules)."""
import time

import pytest
import torch

from uniserve_v1_b200.config.policy import Package
from uniserve_v1_b200.engine.quota import DeviceQuota, QuotaExceeded, divide


def test_ledger_limits_shared_storage_and_hand_over():
    q = DeviceQuota(1000, "fake:0")
    q.state_fraction("a", 0.9)
    assert q.limit() == 1000                      # nobody holds anything yet
    q.reserve("a", "weights", 400, key="w0")
    assert q.limit() == 900 and q.usage() == 400 and q.room("a") == 500
    q.reserve("a", "cache_segment", 450)
    with pytest.raises(QuotaExceeded) as e:       # 400 + 450 + 100 > 900: refused, nothing changes
        q.reserve("a", "graph_pool", 100)
    assert e.value.limit == 900 and q.usage() == 850 and q.refused == 1
    q.reserve("a", "graph_pool", 50)
    # growing an item is checked, shrinking always succeeds
    with pytest.raises(QuotaExceeded):
        q.reserve("a", "cache_segment", 451)
    assert q.usage() == 900
    q.reserve("a", "cache_segment", 200)
    assert q.usage() == 650
    # a second holder with a smaller fraction: the smaller limit holds while both hold storage
    q.state_fraction("b", 0.7)
    q.reserve("b", "weights", 400, key="w0")      # the same storage: counted once
    assert q.usage() == 650 and q.limit() == 700 and q.usage("b") == 400
    with pytest.raises(QuotaExceeded):
        q.reserve("b", "cache_segment", 51)
    q.reserve("b", "cache_segment", 50)
    assert q.usage() == 700 and q.room("b") == 0
    # the successor takes the predecessor's segment over: no release, no allocation
    assert q.hand_over("a", "b", "cache_segment") == 200
    assert q.usage() == 700 and q.usage("b") == 650
    rep = q.report()
    assert rep["holders"]["b"]["items"] == {"cache_segment": 250, "weights": 400}
    assert rep["holders"]["a"]["items"] == {"graph_pool": 50, "weights": 400}
    assert rep["limit"] == 700 and rep["room"] == 0 and rep["refused"] == 3
    # the predecessor retires: the shared weights stay reserved (b holds them), its pool ends,
    # and its larger fraction no longer matters
    assert q.release("a") == 50
    assert q.usage() == 650 and q.limit() == 700
    assert q.release("b") == 650 and q.usage() == 0 and q.limit() == 1000
    # memory that is allocated already is recorded past the limit, and counted
    q.state_fraction("c", 0.5)
    q.reserve("c", "exclusive", 600, force=True)
    assert q.usage() == 600 and q.report()["forced"] == 1
    with pytest.raises(ValueError):
        q.reserve("c", "pages", 1)
    with pytest.raises(ValueError):
        q.state_fraction("c", 0.0)


def test_division_gives_the_rest_to_kv_pages():
    q = DeviceQuota(10_000, "fake:1")
    pages = divide(q, "e0", 0.8, weights=3000, graph_pool=1000, per_page=100, want_pages=1000,
                   min_pages=4)
    assert pages == 40 and q.usage() == 8000 and q.room("e0") == 0
    # a second engine that shares the weights gets nothing but its minimum, which is refused
    with pytest.raises(QuotaExceeded):
        divide(q, "e1", 0.8, weights=3000, graph_pool=1000, per_page=100, want_pages=1000,
               min_pages=4, weights_key=None)
    assert q.usage() == 8000 and "e1" not in q.report()["holders"]
    q.release("e0")
    assert divide(q, "e2", 0.8, weights=3000, graph_pool=1000, per_page=100, want_pages=10) == 10
    assert q.usage() == 5000


def _engine(quota=None, strict=False, pages=128, max_len=128, model=None):
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    if model is None:
        model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    return LLMEngine(model, num_pages=pages, max_num_seqs=8, max_model_len=max_len,
                     use_graphs=False, quota=quota, quota_strict=strict, mem_fraction_static=0.9)


def test_engine_reserves_sleeps_wakes_and_retires():
    from uniserve_v1_b200.engine.types import SamplingParams
    probe = _engine(DeviceQuota(1 << 40, "fake:2"))
    weights = probe._quota_items["weights"]
    cache = probe._quota_items["cache_segment"]
    assert weights > 0 and cache == 128 * probe.model.kv_bytes_per_page(16)
    # a device with room for one engine and a second cache, but not a third
    total = int((weights + 2 * cache + cache // 2) / 0.9) + 1
    q = DeviceQuota(total, "fake:3")
    first = _engine(q, strict=True, model=probe.model)
    st = first.stats()["quota"]
    assert st["bytes"] == weights + cache and st["limit"] == int(total * 0.9) and st["over"] is None
    second = _engine(q, strict=True, model=probe.model)          # shares the weights
    assert q.usage() == weights + 2 * cache
    with pytest.raises(QuotaExceeded):
        _engine(q, strict=True, model=probe.model)
    assert q.usage() == weights + 2 * cache and len(q.report()["holders"]) == 2
    # an engine that is not strict is recorded all the same, and says what did not fit
    loose = _engine(q, strict=False, model=probe.model)
    assert loose.quota_over and q.report()["forced"] == 1
    assert loose.retire() == cache
    # sleep gives the cache back (level 2: the weights too, once nobody else holds them)
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    want = first.generate([[1, 2, 3, 4, 5]], sp)
    first.sleep(1)
    assert q.usage() == weights + cache and q.usage(first.quota_holder) == weights
    third = _engine(q, strict=True, model=probe.model)           # takes the room
    with pytest.raises(QuotaExceeded):                           # ... so the sleeper stays asleep
        first.wake()
    assert first.asleep == 1
    third.retire()
    first.wake()
    assert q.usage() == weights + 2 * cache and first.generate([[1, 2, 3, 4, 5]], sp) == want
    second.retire()
    first.retire()
    assert q.usage() == 0
    # an engine that is dropped without being retired gives its reservations back too
    gone = _engine(q, strict=True, model=probe.model)
    assert q.usage() == gone._quota_items["weights"] + cache
    del gone
    import gc
    gc.collect()
    assert q.usage() == 0


def test_update_whose_target_does_not_fit_the_quota_is_abandoned():
    """An epoch update builds its target beside the serving engine; a target that the
    device's quota has no room for is refused, the update is abandoned with the ledger's
    reason, the serving engine keeps serving and its reservations are intact; after a
    committed update the previous engine's reservations are gone."""
    from fastapi.testclient import TestClient
    from uniserve_v1_b200.server.app import create_app
    from uniserve_v1_b200.server.tokenizer import ByteTokenizer
    probe = _engine(DeviceQuota(1 << 40, "fake:4"))
    weights, cache = probe._quota_items["weights"], probe._quota_items["cache_segment"]
    q = DeviceQuota(int((weights + 2 * cache + cache // 2) / 0.9) + 1, "fake:5")
    first = _engine(q, strict=True, model=probe.model)
    base = 'model = "random:tiny"\nserved_model_name = "tiny"\n'
    upd = '[update_config]\ntrial = "0.2s"\ndrain_s = 0.05\n'
    built = []

    def builder(pkg):
        big = pkg.max_model_len == 96
        eng = _engine(q, strict=True, pages=384 if big else 128,
                      max_len=pkg.max_model_len or 128, model=probe.model)
        built.append(eng)
        return eng
    app = create_app(package=Package.parse(base + upd), engine=first,
                     tokenizer=ByteTokenizer(1024, 1023), served_model_name="tiny",
                     engine_builder=builder)
    body = {"model": "tiny", "messages": [{"role": "user", "content": "still here"}],
            "max_tokens": 8, "temperature": 0, "ignore_eos": True}

    def settle(c, phases):
        for _ in range(200):
            ph = c.get("/admin/update").json()
            if ph["phase"] in phases:
                return ph
            time.sleep(0.05)
        return ph
    with TestClient(app) as c:
        want = c.post("/v1/chat/completions", json=body).json()["choices"][0]["message"]["content"]
        assert c.put("/admin/policy", content=base + "max_model_len = 96\n" + upd).status_code == 202
        ph = settle(c, ("abandoned", "committed"))
        assert ph["phase"] == "abandoned" and "quota" in ph["reason"] and not built
        assert app.state.s.service.engine is first and q.usage() == weights + cache
        assert c.post("/v1/chat/completions", json=body).json()["choices"][0]["message"]["content"] == want
        # a target that fits: committed, and the previous engine's quota ends with it
        assert c.put("/admin/policy", content=base + "max_model_len = 100\n" + upd).status_code == 202
        ph = settle(c, ("abandoned", "committed", "rolled_back"))
        assert ph["phase"] == "committed" and app.state.s.service.engine is built[0]
        rep = q.report()
        assert list(rep["holders"]) == [built[0].quota_holder]
        assert rep["usage"] == built[0]._quota_items["weights"] + cache
        assert c.post("/v1/chat/completions", json=body).json()["choices"][0]["message"]["content"] == want
        devices = c.get("/admin/quota").json()["devices"]
        assert isinstance(devices, list)


def test_host_tier_leaves_the_nodes_reserve_free(monkeypatch):
    """The host KV tier is sized as a multiple of the device pool within its own budget and
    within what the node has beyond the reserve that stays free of KV pages."""
    from uniserve_v1_b200.engine import engine as E
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    per_page = model.kv_bytes_per_page(16)
    monkeypatch.setattr(E, "_host_available", lambda: float((10 << 30) + 40 * per_page))

    def tier(**kw):
        eng = E.LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=128,
                          use_graphs=False, host_kv_ratio=2.0, quota=DeviceQuota(1 << 40, "fake:6"),
                          **kw)
        return int(getattr(eng.blocks, "host_slots", 0))
    assert tier() == 128                                   # no reserve stated: ratio x pool
    assert tier(host_reserve_gib=1.0) == 128               # plenty beyond the reserve
    assert tier(host_reserve_gib=10.0) == 40               # what the node has beyond it
    assert tier(host_reserve_gib=11.0) == 0                # nothing: no host tier
