"""The real scheduler and block manager against a deterministic fake executor:
chunked prefill, prefix reuse, recompute preemption, limits, priorities, aborts,
failure classes and migration through the engine service."""
import asyncio
import random

import pytest

from uniserve_v1_b200.engine.scheduler import Policy
from uniserve_v1_b200.engine.types import FinishReason, SamplingParams
from uniserve_v1_b200.testing.fakes import FakeEngine, expected_output


def _prompts(n, lo=3, hi=70, seed=0):
    rng = random.Random(seed)
    return [[rng.randrange(1000) for _ in range(rng.randrange(lo, hi))] for _ in range(n)]


def test_outputs_are_exact_under_chunking_and_batching():
    eng = FakeEngine(num_pages=256, max_num_seqs=4, max_num_batched_tokens=24)
    prompts = _prompts(9)
    ids = [eng.add_request(p, SamplingParams(max_tokens=11)) for p in prompts]
    eng.run()
    for rid, p in zip(ids, prompts):
        r = eng.scheduler.requests[rid]
        assert r.output_ids == expected_output(p, 11) and r.finish_reason == FinishReason.LENGTH
    kinds = [k for k, _ in eng.runner.calls]
    assert "prefill" in kinds and "decode" in kinds
    # no chunk exceeds the token budget and at most 31 prompts share a prefill call
    for kind, chunks in eng.runner.calls:
        if kind == "prefill":
            assert sum(c[2] for c in chunks) <= 24 and len(chunks) <= 31
    assert eng.blocks.num_free + eng.blocks.num_cached >= 0 and not eng.scheduler.running


def test_preemption_by_recompute_keeps_tokens_exact():
    # 12 pages of 16 tokens cannot hold 4 long requests at once
    eng = FakeEngine(num_pages=13, max_num_seqs=4, max_num_batched_tokens=64,
                     enable_prefix_cache=False)
    prompts = _prompts(4, 30, 40, seed=1)
    ids = [eng.add_request(p, SamplingParams(max_tokens=40)) for p in prompts]
    eng.run()
    assert eng.scheduler.stats["preemptions"] > 0
    for rid, p in zip(ids, prompts):
        assert eng.scheduler.requests[rid].output_ids == expected_output(p, 40)
    assert eng.blocks.num_free == 12


def test_prefix_cache_reuse_and_salt_isolation():
    eng = FakeEngine(num_pages=64, max_num_seqs=2)
    base = list(range(100, 150))
    a = eng.add_request(base + [1, 2], SamplingParams(max_tokens=3))
    eng.run()
    b = eng.add_request(base + [7, 8, 9], SamplingParams(max_tokens=3))
    eng.run()
    rb = eng.scheduler.requests[b]
    assert rb.num_cached == 48 and rb.output_ids == expected_output(base + [7, 8, 9], 3)
    c = eng.add_request(base + [7, 8, 9], SamplingParams(max_tokens=3), cache_salt="tenant-b")
    eng.run()
    assert eng.scheduler.requests[c].num_cached == 0
    assert eng.scheduler.requests[a].output_ids == expected_output(base + [1, 2], 3)


def test_stop_conditions_and_limits():
    eng = FakeEngine(num_pages=64, max_model_len=40)
    p = _prompts(1, 10, 11)[0]
    full = expected_output(p, 30)
    stop_tok = full[4]
    r1 = eng.add_request(p, SamplingParams(max_tokens=30, stop_token_ids=(stop_tok,)))
    r2 = eng.add_request(p, SamplingParams(max_tokens=30, stop_token_ids=(stop_tok,), min_tokens=8))
    r3 = eng.add_request(p, SamplingParams(max_tokens=100))
    eng.run()
    q = eng.scheduler.requests
    first = full.index(stop_tok)
    assert q[r1].output_ids == full[:first + 1] and q[r1].finish_reason == FinishReason.STOP
    assert len(q[r2].output_ids) >= 8
    assert q[r3].num_tokens == 40 and q[r3].finish_reason == FinishReason.LENGTH
    with pytest.raises(ValueError):
        eng.add_request(list(range(40)), SamplingParams())
    with pytest.raises(ValueError):
        eng.add_request([], SamplingParams())


def test_priority_and_abort():
    class Prio(Policy):
        pass
    eng = FakeEngine(num_pages=64, max_num_seqs=1, policy=Prio())
    lo = eng.add_request([1, 2, 3], SamplingParams(max_tokens=4), priority=0)
    hi = eng.add_request([4, 5, 6], SamplingParams(max_tokens=4), priority=5)
    gone = eng.add_request([7, 8, 9], SamplingParams(max_tokens=4), priority=9)
    assert eng.abort(gone) and not eng.abort(gone)
    order = []
    for o in eng.run():
        if o.finished:
            order.append(o.request_id)
    assert order == [hi, lo]
    assert eng.scheduler.requests[gone].finish_reason == FinishReason.ABORT


def test_numerical_fault_fails_only_its_row():
    eng = FakeEngine(num_pages=64, nan_on={"bad"})
    eng.add_request([1, 2, 3], SamplingParams(max_tokens=5), request_id="bad")
    ok = eng.add_request([4, 5, 6], SamplingParams(max_tokens=5))
    eng.run()
    q = eng.scheduler.requests
    assert q["bad"].finish_reason == FinishReason.ERROR and "numerical_fault" in q["bad"].error
    assert q[ok].output_ids == expected_output([4, 5, 6], 5)


def test_engine_service_migrates_requests_after_worker_failure():
    """A fatal worker failure stops the engine; the service rebuilds it and every
    live request continues from its delivered tokens (bounded by max_migrations)."""
    from uniserve_v1_b200.server.engine_service import EngineService
    made = []

    def factory():
        e = FakeEngine(num_pages=64, max_num_seqs=4)
        made.append(e)
        return e

    first = FakeEngine(num_pages=64, max_num_seqs=4, fail_on={4})
    svc = EngineService(first, None, None, max_migrations=3, engine_factory=factory)

    async def go():
        svc.start()
        prompts = _prompts(3, 5, 20, seed=3)
        qs = [svc.submit(p, SamplingParams(max_tokens=9)) for p in prompts]
        outs = []
        for (rid, q), p in zip(qs, prompts):
            toks = []
            while True:
                o = await asyncio.wait_for(q.get(), 20)
                toks += o.new_token_ids
                if o.finished:
                    assert o.finish_reason == FinishReason.LENGTH, o
                    break
            outs.append((toks, expected_output(p, 9)))
        svc.stop()
        return outs

    for got, want in asyncio.run(go()):
        assert got == want
    assert len(made) == 1


def test_random_workloads_keep_the_books_straight():
    """Property test over random arrival / abort / step interleavings on a small KV pool
    (forcing chunked prefill, prefix reuse and preemption by recompute): every finished
    request carries exactly the tokens a fresh run of its prompt yields, nothing is lost or
    duplicated, and every page returns to the pool."""
    from hypothesis import HealthCheck, given, settings
    from hypothesis import strategies as st
    from uniserve_v1_b200.engine.types import FinishReason, SamplingParams
    from uniserve_v1_b200.testing.fakes import FakeEngine, expected_output

    events = st.lists(st.one_of(
        st.tuples(st.just("add"), st.integers(1, 90), st.integers(1, 12), st.integers(0, 5)),
        st.tuples(st.just("abort"), st.integers(0, 30)),
        st.tuples(st.just("step"), st.integers(1, 4))), min_size=5, max_size=60)

    @settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])
    @given(events, st.integers(0, 3))
    def run(evs, shared_prefix):
        eng = FakeEngine(num_pages=24, page_size=8, max_num_seqs=4, max_model_len=128,
                         max_num_batched_tokens=32)
        total_pages = eng.blocks.num_free
        prompts, outs, finished, aborted = {}, {}, {}, set()
        k = 0

        def drain(out_list):
            for o in out_list:
                outs.setdefault(o.request_id, []).extend(o.new_token_ids)
                if o.finished:
                    finished[o.request_id] = o.finish_reason
        for ev in evs:
            if ev[0] == "add":
                _, plen, max_tok, seed = ev
                base = [7, 7, 7, 7, 7, 7, 7, 7, 9, 9, 9, 9, 9, 9, 9, 9] * shared_prefix
                prompt = (base + [(seed * 31 + j * 17) % 1000 for j in range(plen)])[:100]
                rid = eng.add_request(prompt, SamplingParams(temperature=0.0, max_tokens=max_tok,
                                                             ignore_eos=True))
                prompts[rid] = (prompt, max_tok)
                k += 1
            elif ev[0] == "abort":
                rid = f"r{ev[1]}"
                if rid in prompts and rid not in finished and eng.abort(rid):
                    aborted.add(rid)
            else:
                for _ in range(ev[1]):
                    drain(eng.step())
        drain(eng.run())
        assert not eng.has_work()
        for rid, (prompt, max_tok) in prompts.items():
            want = expected_output(prompt, max_tok)
            got = outs.get(rid, [])
            if rid in aborted:
                assert got == want[:len(got)]
            else:
                assert got == want, (rid, got, want)
                assert finished[rid] == FinishReason.LENGTH
        eng.blocks.flush()
        assert eng.blocks.num_free == total_pages
    run()


def test_scheduling_program_decides_under_a_fuel_budget(tmp_path):
    """A program from the package orders admissions (shortest prompt first) and keeps state
    across a restart; a runaway program is cut by its budget and the default order applies."""
    import torch
    from uniserve_v1_b200.config.policy import Package
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.program import FuelExhausted, ProgramHost, ProgramPolicy
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    (tmp_path / "programs").mkdir()
    (tmp_path / "programs" / "sjf.py").write_text(
        "seen = {'n': 0}\n"
        "def dispatch(waiting, room):\n"
        "    seen['n'] += len(waiting)\n"
        "    return [w['id'] for w in sorted(waiting, key=lambda w: (w['prompt_tokens'], w['arrival']))]\n"
        "def save_state():\n    return seen\n"
        "def restore_state(s):\n    seen.update(s)\n")
    (tmp_path / "programs" / "spin.py").write_text(
        "def dispatch(waiting, room):\n    while True:\n        pass\n")
    (tmp_path / "config.toml").write_text(
        'model = "random:tiny"\n[scheduler_config.policy_budget]\ncall_fuel = 20000\n'
        '[programs.sjf]\nsource = "programs/sjf.py"\n[programs.spin]\nsource = "programs/spin.py"\n')
    pkg = Package.load(tmp_path)
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    sp = SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True)
    prompts = {"long": list(range(40)), "short": list(range(5)), "mid": list(range(17))}

    def first_tokens(policy):
        eng = LLMEngine(model, num_pages=64, max_num_seqs=1, max_model_len=128,
                        use_graphs=False, policy=policy)
        for rid, p in prompts.items():
            eng.add_request(p, sp, request_id=rid)
        order = []
        while eng.has_work():
            for o in eng.step():
                if o.request_id not in order:
                    order.append(o.request_id)
        return order
    assert first_tokens(None) == ["long", "short", "mid"]                    # arrival order
    host = ProgramHost.load(pkg, "sjf")
    pol = ProgramPolicy(host)
    assert first_tokens(pol) == ["short", "mid", "long"] and pol.faults == 0
    assert host.fuel_used > 0 and host.call_fuel == 20000
    again = ProgramHost.load(pkg, "sjf")
    again.restore_state(host.save_state())
    assert again.ns["seen"]["n"] == host.ns["seen"]["n"] > 0
    spin = ProgramPolicy(ProgramHost.load(pkg, "spin"))
    assert first_tokens(spin) == ["long", "short", "mid"] and spin.faults > 0
    import pytest
    with pytest.raises(FuelExhausted):
        spin.host.call("dispatch", [], {})
    with pytest.raises(Exception):
        ProgramHost("import os\n", "escape")                                  # no import machinery


def test_routing_program_picks_replicas_and_falls_back():
    from uniserve_v1_b200.engine.program import ProgramHost
    from uniserve_v1_b200.server.router import ReplicaRouter
    big_to_last = ProgramHost(
        "def route(request, replicas):\n"
        "    if request['bytes'] > 1000:\n"
        "        return replicas[-1]['index']\n"
        "    return min(replicas, key=lambda r: r['in_flight'])['index']\n", "routing", 100000)
    rt = ReplicaRouter(["http://a", "http://b", "http://c"], program=big_to_last)
    rt.replicas[0].in_flight = 2
    assert rt.pick(size=5000).url == "http://c" and rt.pick(size=10).url == "http://b"
    assert rt.pick(size=5000, exclude=[rt.replicas[2]]).url == "http://b"
    bad = ReplicaRouter(["http://a", "http://b"], program=ProgramHost(
        "def route(request, replicas):\n    return 7\n", "routing", 100000))
    bad.replicas[0].in_flight = 1
    assert bad.pick().url == "http://b" and bad.program_faults == 1
    spin = ReplicaRouter(["http://a"], program=ProgramHost(
        "def route(request, replicas):\n    while True:\n        pass\n", "routing", 5000))
    assert spin.pick().url == "http://a" and spin.program_faults == 1
