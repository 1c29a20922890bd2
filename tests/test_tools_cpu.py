"""The evaluation tool against a live server on CPU (tiny model), and its checks."""
import asyncio
import socket
import threading
import time

import pytest
import torch


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.fixture(scope="module")
def live_server():
    import uvicorn
    from uniserve_v1_b200.config.policy import Package
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.server.app import create_app
    from uniserve_v1_b200.server.tokenizer import ByteTokenizer
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    eng = LLMEngine(model, num_pages=512, max_num_seqs=8, max_model_len=512, use_graphs=False)
    pkg = Package.parse('model = "random:tiny"\nserved_model_name = "tiny"\n')
    app = create_app(package=pkg, engine=eng, tokenizer=ByteTokenizer(1024, 1023),
                     served_model_name="tiny")
    port = _free_port()
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    for _ in range(200):
        if server.started:
            break
        time.sleep(0.05)
    assert server.started
    yield f"http://127.0.0.1:{port}"
    server.should_exit = True
    th.join(timeout=10)


def test_eval_run_and_checks(live_server):
    from uniserve_v1_b200.tools import eval as E
    b = asyncio.run(E.run_load(live_server, concurrency=4, requests=8, prompt_tokens=12,
                               max_tokens=6, model="tiny"))
    s = b["summary"]
    assert s["succeeded"] == 8 and s["failed"] == 0 and s["output_tokens"] == 48
    assert s["ttft_s"]["p50"] is not None and s["tpot_s"]["p50"] is not None
    assert all(r["finish_reason"] == "length" for r in b["records"])
    assert E.check_stop(b) == [] and E.check_faults(b) == []
    assert E.compare_bundles(b, b) == []
    slow = {"summary": dict(s, output_tokens_per_s=s["output_tokens_per_s"] * 0.5), "records": []}
    assert any("tokens/s" in f for f in E.compare_bundles(b, slow))
    # non-streaming path
    b2 = asyncio.run(E.run_load(live_server, 2, 2, 8, 4, stream=False, model="tiny"))
    assert b2["summary"]["succeeded"] == 2


def test_eval_plan_and_list(capsys):
    """`plan` prints what `run` would send (the same prompts for the same seed), `list` the
    verbs with what each checks."""
    import json
    from uniserve_v1_b200.tools import eval as E
    assert E.main(["plan", "--requests", "3", "--prompt-tokens", "16", "--seed", "4",
                   "--stop", "END", "--change", "1.5:policy.toml"]) == 0
    plan = json.loads(capsys.readouterr().out)
    assert plan["requests"] == 3 and [i["seed"] for i in plan["items"]] == [4, 5, 6]
    assert plan["body"]["stop"] == ["END"] and plan["changes"] == [{"at_s": 1.5, "file": "policy.toml"}]
    assert E.main(["plan", "--requests", "3", "--prompt-tokens", "16", "--seed", "4"]) == 0
    again = json.loads(capsys.readouterr().out)
    assert [i["prompt_sha256"] for i in again["items"]] == [i["prompt_sha256"] for i in plan["items"]]
    assert E.main(["list"]) == 0
    assert {"run", "plan", "compare", "check-change", "check-stop", "check-faults"} <= \
        set(json.loads(capsys.readouterr().out))


def test_eval_check_rules():
    from uniserve_v1_b200.tools import eval as E
    rec = dict(index=0, ok=True, status=200, error=None, latency_s=1.0, ttft_s=0.1,
               output_tokens=5, prompt_tokens=3, cached_tokens=0, finish_reason="length",
               text="abc END", chunks=5, stop=["END"], max_tokens=8)
    fails = E.check_stop({"records": [rec]})
    assert len(fails) == 2          # stop string present; 'length' short of the budget
    hung = dict(rec, ok=False, status=0, error=None, finish_reason=None)
    assert E.check_faults({"records": [hung]})
    failed = dict(rec, ok=False, status=503, error="engine failed")
    assert E.check_faults({"records": [failed]}) == []
    acc = E.compare_accuracy(1248, 1233, 1319)
    assert acc["pass"] and abs(acc["reference"] - 0.946171) < 1e-6
    assert not E.compare_accuracy(1248, 1100, 1319)["pass"]


def test_profile_session_and_trace(tmp_path):
    """Probes and spans of engine steps land in a session file; the profile tool
    pairs the probes into device ranges and writes a trace."""
    import json
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.profiling import StepProfiler
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.tools import profile as P
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    eng = LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=128, use_graphs=False)
    eng.profiler = StepProfiler("cpu")
    path = str(tmp_path / "rank0.sqlite")
    eng.profiler.open(path, {"model": "tiny"})
    eng.generate([[1, 2, 3, 4, 5]], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    steps = eng.profiler.steps
    eng.profiler.close()
    assert steps >= 4 and eng.profiler.counters()["device_seconds"] > 0
    s = P.load(path)
    assert len(s["spans"]) == steps and len(s["probes"]) == 2 * steps
    assert s["meta"]["model"] == "tiny"
    ranges = P.device_ranges(s["probes"])
    assert len(ranges) == steps and all(r[4] >= r[3] for r in ranges)
    out = tmp_path / "trace.json"
    assert P.main(["trace", path, "-o", str(out)]) == 0
    tr = json.loads(out.read_text())
    assert len(tr["traceEvents"]) == 2 * steps
    assert {e["tid"] for e in tr["traceEvents"]} >= {"device"}


_LAYOUTS = {
    "tp2": "tensor_parallel_size = 2\n",
    # data-parallel attention + expert parallelism: two members, each with half the experts
    "dp_ep2": "data_parallel_size = 2\n[moe_config]\nexpert_parallel = true\n",
    # distributed weight data parallelism: two members that read each other's expert shards
    "dwdp2": 'data_parallel_size = 2\n[moe_config]\nexpert_parallel = true\nexchange = "weights"\n',
    # attention / expert disaggregation: two attention members, one experts-only rank
    "afd": '[moe_config]\nexpert_parallel = true\n[[worker_groups]]\nid = "attention"\n'
           'ranks = ["cuda:0-1"]\n[[worker_groups]]\nid = "experts"\nrole = "experts"\n'
           'ranks = ["cuda:2"]\n',
}


@pytest.mark.parametrize("layout", ["tp2", "dp_ep2", "dwdp2", "afd"])
def test_serve_command_runs_a_two_rank_deployment(tmp_path, layout):
    """`serve` starts the other ranks of the package's layout itself (gloo ranks on CPU
    here) - a tensor-parallel pair, an expert union of two members, or two attention members
    with an experts-only rank - and the deployment answers like a single-rank one."""
    import json
    import os
    import subprocess
    import sys
    import urllib.request
    port = _free_port()
    pkg = tmp_path / "pkg"
    pkg.mkdir()
    head = 'model = "random:tiny"\nserved_model_name = "tiny"\n'
    admin = f'[admin_config]\nhost = "127.0.0.1"\nport = {port}\n'
    body_toml = _LAYOUTS[layout]
    (pkg / "config.toml").write_text(head + (body_toml + admin if not body_toml.startswith("[")
                                             else admin + body_toml))
    env = dict(os.environ, UNISERVE_CPU_RANKS="1")
    env.pop("RANK", None)
    proc = subprocess.Popen([sys.executable, "-m", "uniserve_v1_b200", "serve", str(pkg)], env=env,
                            cwd=os.path.dirname(os.path.dirname(__file__)))
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}],
            "max_tokens": 8, "temperature": 0, "ignore_eos": True}
    try:
        ok = False
        for _ in range(240):
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1) as r:
                    ok = r.status == 200
                    break
            except Exception:
                if proc.poll() is not None:
                    break
                time.sleep(0.5)
        assert ok, "server did not come up"
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions",
                                     data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as r:
            two = json.loads(r.read())
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=30)
        except Exception:
            proc.kill()
    # the same request on an in-process single-rank server
    from fastapi.testclient import TestClient
    from uniserve_v1_b200.config.policy import Package
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.server.app import create_app
    from uniserve_v1_b200.server.tokenizer import load_tokenizer
    cfg = Qwen3MoeConfig.tiny()
    model = Qwen3MoeModel(cfg, "cpu", torch.float32).init_random(seed=0)
    eng = LLMEngine(model, num_pages=512, max_num_seqs=8, max_model_len=512, use_graphs=False)
    app = create_app(package=Package.parse('model = "random:tiny"\nserved_model_name = "tiny"\n'),
                     engine=eng, tokenizer=load_tokenizer(None, cfg.vocab_size, cfg.eos_token_id),
                     served_model_name="tiny")
    with TestClient(app) as c:
        one = c.post("/v1/chat/completions", json=body).json()
    assert two["choices"][0]["message"]["content"] == one["choices"][0]["message"]["content"]
    assert two["usage"]["completion_tokens"] == 8


def test_replica_router_spreads_and_sticks(live_server):
    """Two replicas behind the router: requests spread by load, a cache key sticks to one
    replica, streaming passes through, a dead replica is skipped."""
    import json
    import threading as th
    import urllib.request
    import uvicorn
    from uniserve_v1_b200.server.router import create_router_app
    port = _free_port()
    dead = f"http://127.0.0.1:{_free_port()}"
    app = create_router_app([dead, live_server, live_server])
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error"))
    t = th.Thread(target=server.run, daemon=True)
    t.start()
    for _ in range(200):
        if server.started:
            break
        time.sleep(0.05)
    base = f"http://127.0.0.1:{port}"
    try:
        def post(body):
            req = urllib.request.Request(base + "/v1/chat/completions", data=json.dumps(body).encode(),
                                         headers={"Content-Type": "application/json"})
            with urllib.request.urlopen(req, timeout=60) as r:
                return r.read().decode()
        body = {"model": "tiny", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4,
                "temperature": 0, "ignore_eos": True}
        out = [json.loads(post(body)) for _ in range(3)]
        assert all(o["usage"]["completion_tokens"] == 4 for o in out)
        sse = post(dict(body, stream=True))
        assert sse.strip().endswith("data: [DONE]")
        for _ in range(3):
            post(dict(body, prompt_cache_key="tenant-7"))
        with urllib.request.urlopen(base + "/router/replicas", timeout=10) as r:
            stats = json.loads(r.read())
        assert stats[0]["served"] == 0 and not stats[0]["up"]          # the dead one
        assert stats[1]["served"] + stats[2]["served"] == 7
        with urllib.request.urlopen(base + "/health", timeout=10) as r:
            assert json.loads(r.read())["replicas_up"] == 2
        with urllib.request.urlopen(base + "/v1/models", timeout=10) as r:
            assert json.loads(r.read())["data"][0]["id"] == "tiny"
    finally:
        server.should_exit = True
        t.join(timeout=10)


def test_router_sends_requests_where_their_prefix_is_cached():
    """Two replicas behind a prefix-aware router.  A conversation whose first turn ran on one
    replica continues there (the router asks both replicas how much of the prompt each holds),
    also when that replica is the busier one by index order; a prompt nobody holds goes by
    load; the probe allocates nothing."""
    import json
    import urllib.request
    import uvicorn
    from uniserve_v1_b200.server.router import create_router_app
    a_url, a_srv, a_th, a_eng = _start_chat_server()
    b_url, b_srv, b_th, b_eng = _start_chat_server()
    port = _free_port()
    app = create_router_app([a_url, b_url], prefix_aware=True)
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error"))
    t = threading.Thread(target=server.run, daemon=True)
    t.start()
    for _ in range(200):
        if server.started:
            break
        time.sleep(0.05)
    base = f"http://127.0.0.1:{port}"

    def post(url, body, path="/v1/chat/completions"):
        req = urllib.request.Request(url + path, data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as r:
            return json.loads(r.read())
    story = "once upon a time there was a very long prompt about routing requests " * 3
    turn1 = {"model": "tiny", "max_tokens": 4, "temperature": 0, "ignore_eos": True,
             "messages": [{"role": "user", "content": story}]}
    try:
        # the first turn runs on replica B directly (the router would have picked A)
        first = post(b_url, turn1)
        free_b = b_eng.blocks.num_free
        probe_a = post(a_url, turn1, "/internal/probe")
        probe_b = post(b_url, turn1, "/internal/probe")
        assert probe_a["cached_tokens"] == 0 and probe_b["cached_tokens"] >= 64
        assert probe_b["prompt_tokens"] == probe_a["prompt_tokens"] > 64
        assert b_eng.blocks.num_free == free_b                        # a probe keeps no page
        # the second turn extends the first: it is sent to B, where the prefix is
        turn2 = dict(turn1, messages=turn1["messages"] + [
            {"role": "assistant", "content": first["choices"][0]["message"]["content"] or ""},
            {"role": "user", "content": "and then?"}])
        served_b = b_eng.scheduler.stats["prefill_tokens"]
        out = post(base, turn2)
        assert out["usage"]["completion_tokens"] == 4
        with urllib.request.urlopen(base + "/router/stats", timeout=10) as r:
            st = json.loads(r.read())
        assert st["prefix_hits"] == 1 and st["probes"] == 1
        assert [x["served"] for x in st["replicas"]] == [0, 1]
        # B computed only what the first turn had not cached
        assert b_eng.scheduler.stats["prefill_tokens"] - served_b < probe_b["prompt_tokens"]
        # nobody holds this prompt: by load, lowest index first
        post(base, dict(turn1, messages=[{"role": "user", "content": "something else entirely"}]))
        with urllib.request.urlopen(base + "/router/stats", timeout=10) as r:
            st = json.loads(r.read())
        assert st["prefix_hits"] == 1 and [x["served"] for x in st["replicas"]] == [1, 1]
    finally:
        for srv, th_ in ((server, t), (a_srv, a_th), (b_srv, b_th)):
            srv.should_exit = True
            th_.join(timeout=10)


def test_admin_client(live_server, capsys):
    import json
    from uniserve_v1_b200.__main__ import main
    assert main(["admin", "--url", live_server, "health"]) == 0
    assert json.loads(capsys.readouterr().out)["status"] == "ok"
    assert main(["admin", "--url", live_server, "get-policy"]) == 0
    assert json.loads(capsys.readouterr().out)["config"]["served_model_name"] == "tiny"
    assert main(["admin", "--url", live_server, "query", "select count(*) from events"]) == 0
    assert "rows" in json.loads(capsys.readouterr().out)
    assert main(["admin", "--url", live_server, "query", "drop table events"]) == 1


def test_admin_client_status_watch_and_apply_over_several_nodes(live_server, tmp_path, capsys):
    """The manager's verbs: `status` tables every node (an unreachable one fails the exit
    status), `watch` prints a line per change, `apply` puts a policy on every node and puts
    the nodes already changed back when one refuses."""
    import json
    from uniserve_v1_b200.__main__ import main
    other, other_srv, other_th, _eng = _start_chat_server()
    dead = f"http://127.0.0.1:{_free_port()}"
    try:
        assert main(["admin", "--url", live_server, "--url", other, "status"]) == 0
        rows = json.loads(capsys.readouterr().out)
        assert [r["status"] for r in rows] == ["ok", "ok"] and rows[0]["model"] == "tiny"
        assert main(["admin", "--url", live_server, "--url", dead, "status"]) == 1
        assert json.loads(capsys.readouterr().out)[1]["status"] == "unreachable"
        assert main(["admin", "--url", live_server, "--url", other, "--interval", "0.05",
                     "--count", "3", "watch"]) == 0
        lines = [json.loads(x) for x in capsys.readouterr().out.strip().splitlines()]
        assert len(lines) == 2 and {x["url"] for x in lines} == {live_server, other}

        good = tmp_path / "good.toml"
        good.write_text('model = "random:tiny"\nserved_model_name = "tiny"\n'
                        '[scheduler_config]\nmax_batch = 3\n')
        assert main(["admin", "--url", live_server, "--url", other, "apply", str(good)]) == 0
        capsys.readouterr()
        for u in (live_server, other):
            assert main(["admin", "--url", u, "get-policy"]) == 0
            assert json.loads(capsys.readouterr().out)["config"]["scheduler_config"]["max_batch"] == 3
        # the second node is gone: the first one returns to what it served
        other_srv.should_exit = True
        other_th.join(timeout=10)
        back = tmp_path / "back.toml"
        back.write_text('model = "random:tiny"\nserved_model_name = "tiny"\n'
                        '[scheduler_config]\nmax_batch = 5\n')
        bad = tmp_path / "bad.toml"
        bad.write_text('model = "random:tiny"\nserved_model_name = "tiny"\nno_such_option = 1\n')
        assert main(["admin", "--url", live_server, "apply", str(bad)]) == 1
        capsys.readouterr()
        assert main(["admin", "--url", live_server, "get-policy"]) == 0
        assert json.loads(capsys.readouterr().out)["config"]["scheduler_config"]["max_batch"] == 3
    finally:
        other_srv.should_exit = True
        other_th.join(timeout=10)


def test_block_manager_bounded_exhaustive_check_and_mutants():
    """Every operation sequence up to depth 4 on a 5-page pool keeps the invariants of the
    native block manager; each deliberately broken variant is flagged."""
    from uniserve_v1_b200.engine.block_manager import BlockManager
    from uniserve_v1_b200.tools.verify import explore, mutants
    mk = lambda cls: (lambda pages: cls(pages, page_size=4))
    r = explore(mk(BlockManager), pages=5, depth=4, n_keys=2)
    assert r["violation"] is None and r["sequences"] > 2000
    for name, cls in mutants(BlockManager):
        assert explore(mk(cls), pages=5, depth=4, n_keys=2)["violation"], name


def test_host_tier_contents_enumerated_and_unpinned_mutant_caught():
    """Page contents through the host tier, enumerated: whatever the order of allocations,
    commits, fetches and steps (also from a state where the host tier is full and every fetch
    must evict), a fetched page holds what was committed under its key; a manager that does
    not pin matched host slots is flagged."""
    from uniserve_v1_b200.engine.block_manager import BlockManager
    from uniserve_v1_b200.tools.verify import HOST_FULL, explore_host_tier, host_mutant
    mk = lambda cls: (lambda pages: cls(pages, page_size=4))
    for slots in (1, 2):
        r = explore_host_tier(mk(BlockManager), 4, slots, 4, 2)
        assert r["violation"] is None and r["sequences"] > 1000
    assert explore_host_tier(mk(BlockManager), 4, 1, 4, 2, HOST_FULL)["violation"] is None
    assert explore_host_tier(mk(host_mutant(BlockManager)), 4, 1, 3, 2, HOST_FULL)["violation"]


def _start_chat_server(role="mixed", key=None):
    import uvicorn
    from uniserve_v1_b200.config.policy import Package
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.server.app import create_app
    from uniserve_v1_b200.server.tokenizer import ByteTokenizer
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    eng = LLMEngine(model, num_pages=256, max_num_seqs=8, max_model_len=512, use_graphs=False)
    pkg = Package.parse('model = "random:tiny"\nserved_model_name = "tiny"\n')
    app = create_app(package=pkg, engine=eng, tokenizer=ByteTokenizer(1024, 1023),
                     served_model_name="tiny", role=role, internal_key=key)
    port = _free_port()
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    for _ in range(200):
        if server.started:
            break
        time.sleep(0.05)
    assert server.started
    return f"http://127.0.0.1:{port}", server, th, eng


def test_router_hand_off_legs_have_a_transfer_deadline():
    """A prefill replica that does not answer within the transfer deadline, and a decode
    replica that does not take the frames within it, are answered 504 and counted; the
    router keeps serving."""
    import json
    import urllib.error
    import urllib.request
    import uvicorn
    from fastapi import FastAPI
    from fastapi.responses import Response
    from uniserve_v1_b200.server.router import create_router_app
    import asyncio
    delays = {"prefill": 1.5, "decode": 0.0}
    fake = FastAPI()

    @fake.post("/internal/prefill")
    async def prefill():
        await asyncio.sleep(delays["prefill"])
        return Response(content=b"frames", media_type="application/octet-stream")

    @fake.post("/internal/decode")
    async def decode():
        await asyncio.sleep(delays["decode"])
        return {"choices": [{"message": {"role": "assistant", "content": "ok"}}]}
    servers = []
    ports = [_free_port(), _free_port()]
    apps = [fake, create_router_app([], prefill_urls=[f"http://127.0.0.1:{ports[0]}"],
                                    decode_urls=[f"http://127.0.0.1:{ports[0]}"],
                                    transfer_deadline_s=0.4)]
    for app, port in zip(apps, ports):
        srv = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error"))
        th = threading.Thread(target=srv.run, daemon=True)
        th.start()
        servers.append((srv, th))
    for srv, _ in servers:
        for _ in range(200):
            if srv.started:
                break
            time.sleep(0.05)
    base = f"http://127.0.0.1:{ports[1]}"

    def post():
        req = urllib.request.Request(
            base + "/v1/chat/completions", headers={"Content-Type": "application/json"},
            data=json.dumps({"model": "m", "messages": [{"role": "user", "content": "x"}]}).encode())
        try:
            with urllib.request.urlopen(req, timeout=30) as r:
                return r.status, json.loads(r.read())
        except urllib.error.HTTPError as e:
            return e.code, json.loads(e.read())
    try:
        t0 = time.monotonic()
        code, ans = post()
        assert code == 504 and "prefill" in ans["error"]["message"] and time.monotonic() - t0 < 1.4
        delays.update(prefill=0.0, decode=1.5)
        code, ans = post()
        assert code == 504 and "decode" in ans["error"]["message"]
        delays.update(decode=0.0)
        code, ans = post()
        assert code == 200 and ans["choices"][0]["message"]["content"] == "ok"
        with urllib.request.urlopen(base + "/router/stats", timeout=10) as r:
            st = json.loads(r.read())
        assert st["deadline_misses"] == 2 and st["transfer_deadline_s"] == 0.4
        assert all(x.in_flight == 0 for x in apps[1].state.prefill.replicas + apps[1].state.decode.replicas)
    finally:
        for srv, th in servers:
            srv.should_exit = True
        for srv, th in servers:
            th.join(timeout=10)


def test_router_disaggregates_prefill_and_decode(live_server):
    """A prefill replica and a decode replica behind the router: the answers (plain and
    streamed, greedy and seeded sampling) are those of one replica; the decode replica
    computes no prompt; a request that ends at its first token is answered by the prefill
    replica alone."""
    import json
    import urllib.request
    import uvicorn
    from uniserve_v1_b200.server.router import create_router_app
    pre_url, pre_srv, pre_th, pre_eng = _start_chat_server("prefill", "k3y")
    dec_url, dec_srv, dec_th, dec_eng = _start_chat_server("decode", "k3y")
    port = _free_port()
    app = create_router_app([], prefill_urls=[pre_url], decode_urls=[dec_url],
                            internal_key="k3y")
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error"))
    t = threading.Thread(target=server.run, daemon=True)
    t.start()
    for _ in range(200):
        if server.started:
            break
        time.sleep(0.05)

    def post(base, body):
        req = urllib.request.Request(base + "/v1/chat/completions", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as r:
            return r.read().decode()

    def text_of_stream(sse):
        out = ""
        for line in sse.splitlines():
            if line.startswith("data: ") and line != "data: [DONE]":
                ch = json.loads(line[6:])
                if ch.get("choices"):
                    out += ch["choices"][0]["delta"].get("content") or ""
        return out
    base = f"http://127.0.0.1:{port}"
    try:
        for extra in ({"temperature": 0}, {"temperature": 0.9, "top_p": 0.9, "seed": 5}):
            body = dict({"model": "tiny", "messages": [{"role": "user", "content": "tell me"}],
                         "max_tokens": 9, "ignore_eos": True}, **extra)
            want = json.loads(post(live_server, body))
            got = json.loads(post(base, body))
            assert got["choices"][0]["message"] == want["choices"][0]["message"]
            assert got["usage"]["completion_tokens"] == 9
            assert text_of_stream(post(base, dict(body, stream=True))) == \
                (want["choices"][0]["message"]["content"] or "")
        assert dec_eng.scheduler.stats["prefill_tokens"] <= 8      # one token per imported request
        assert pre_eng.scheduler.stats["decode_tokens"] == 0 and not pre_eng.scheduler.running
        one = json.loads(post(base, {"model": "tiny", "max_tokens": 1, "temperature": 0,
                                     "ignore_eos": True,
                                     "messages": [{"role": "user", "content": "x"}]}))
        assert one["usage"]["completion_tokens"] == 1
        with urllib.request.urlopen(base + "/v1/models", timeout=10) as r:
            assert json.loads(r.read())["data"][0]["id"] == "tiny"

        # the internal routes: absent on a mixed replica, closed without the key, and a
        # pickle stream (what an attacker would send to get code run) is refused as a frame
        import base64
        import pickle
        import urllib.error

        class Boom:
            def __reduce__(self):
                return (os.system, ("touch /tmp/us_handoff_pwned",))
        import os
        evil = base64.b64encode(pickle.dumps(Boom())).decode()
        chat = {"model": "tiny", "messages": [{"role": "user", "content": "x"}], "max_tokens": 2}

        def status(url, body, key=None):
            hdr = {"Content-Type": "application/json"}
            if key:
                hdr["x-uniserve-internal-key"] = key
            rq = urllib.request.Request(url, data=json.dumps(body).encode(), headers=hdr)
            try:
                with urllib.request.urlopen(rq, timeout=30) as r:
                    return r.status, r.read().decode()
            except urllib.error.HTTPError as e:
                return e.code, e.read().decode()
        assert status(live_server + "/internal/decode", {"request": chat, "handoff": evil})[0] == 404
        assert status(dec_url + "/internal/decode", {"request": chat, "handoff": evil})[0] == 401
        assert status(pre_url + "/internal/prefill", chat)[0] == 401
        code, text = status(dec_url + "/internal/decode", {"request": chat, "handoff": evil}, "k3y")
        assert code == 400 and "hand-off" in text
        assert not os.path.exists("/tmp/us_handoff_pwned")

        # a lender of another tensor-parallel degree: the state arrives as one frame per rank
        # (here the prefill replica's frame cut into its two KV heads) and is re-cut on import
        import dataclasses
        from uniserve_v1_b200.engine.handoff import Handoff, pack_frames
        chat9 = {"model": "tiny", "messages": [{"role": "user", "content": "tell me"}],
                 "max_tokens": 9, "ignore_eos": True, "temperature": 0}
        rq = urllib.request.Request(pre_url + "/internal/prefill", data=json.dumps(chat9).encode(),
                                    headers={"Content-Type": "application/json",
                                             "x-uniserve-internal-key": "k3y"})
        with urllib.request.urlopen(rq, timeout=60) as r:
            frame = r.read()
        h = Handoff.from_bytes(frame)
        halves = [dataclasses.replace(h, head_lo=lo, kv=[(k[:, :, lo:lo + 1].contiguous(),
                                                          v[:, :, lo:lo + 1].contiguous())
                                                         for k, v in h.kv]) for lo in (1, 0)]
        two = base64.b64encode(pack_frames([x.to_bytes() for x in halves])).decode()
        code, text = status(dec_url + "/internal/decode", {"request": chat9, "handoff": two}, "k3y")
        assert code == 200, text
        want9 = json.loads(post(live_server, chat9))
        assert json.loads(text)["choices"][0]["message"] == want9["choices"][0]["message"]
        only_one = base64.b64encode(halves[0].to_bytes()).decode()
        code, text = status(dec_url + "/internal/decode", {"request": chat9, "handoff": only_one},
                            "k3y")
        assert code == 400 and "in no frame" in text
    finally:
        for srv, th_ in ((server, t), (pre_srv, pre_th), (dec_srv, dec_th)):
            srv.should_exit = True
            th_.join(timeout=10)


def test_block_manager_replays_a_serving_trace():
    """The block-manager calls of an engine that serves shared prefixes under page pressure
    (preemption, eviction) replay on a fresh manager with the same answers and with the
    invariants intact; a tampered trace is flagged."""
    from uniserve_v1_b200.engine.block_manager import BlockManager
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.tools.verify import record, replay
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    eng = LLMEngine(model, num_pages=14, page_size=4, max_num_seqs=3, max_model_len=64,
                    use_graphs=False)
    trace = record(eng.blocks)
    shared = list(range(100, 113))
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    for tail in ([1, 2, 3], [4, 5], [6], [7, 8, 9, 10]):
        eng.add_request(shared + tail, sp)
    while eng.has_work():
        eng.step()
    eng.generate([shared + [11]], sp)                      # finds the committed prefix again
    kinds = {op[0] for op in trace}
    assert {"allocate", "release", "commit", "match"} <= kinds and len(trace) > 40
    assert eng.scheduler.stats["preemptions"] > 0 or eng.blocks.stats()["evictions"] > 0
    mk = lambda pages: BlockManager(pages, page_size=4)
    assert replay(trace, mk, 14) == {"calls": len(trace), "violation": None}
    i = next(i for i, op in enumerate(trace) if op[0] == "release")
    bad = trace[:i] + [trace[i], trace[i]] + trace[i + 1:]           # a double release
    assert replay(bad, mk, 14)["violation"]


def test_site_protocol_interleavings():
    """The flag / epoch protocol of the fused collectives: no interleaving of 2 or 3 ranks reads a
    stale or overwritten partial or blocks, as long as another site's barrier lies between two
    uses of a buffer; a single site is caught."""
    from uniserve_v1_b200.tools.verify import explore_site_protocol
    assert explore_site_protocol(2, 2, 3)["violation"] is None
    assert explore_site_protocol(3, 2, 2)["violation"] is None
    assert explore_site_protocol(3, 3, 2)["violation"] is None
    bad = explore_site_protocol(2, 1, 2)["violation"]
    assert bad and "finds pass" in bad


def test_ulysses_protocol_interleavings():
    from uniserve_v1_b200.tools.verify import explore_ulysses_protocol
    assert explore_ulysses_protocol(2, 3)["violation"] is None
    assert explore_ulysses_protocol(3, 2)["violation"] is None
    assert explore_ulysses_protocol(2, 2, second_barrier=False)["violation"]


def test_tp_protocol_interleavings():
    from uniserve_v1_b200.tools.verify import explore_tp_protocol
    assert explore_tp_protocol(2, 4)["violation"] is None
    assert explore_tp_protocol(3, 2)["violation"] is None
    assert explore_tp_protocol(2, 3, norm_sites=1)["violation"] is None


def test_eval_check_change_against_control(live_server):
    """A load during which the policy is changed twice (prefix caching off, then on) loses no
    request, no token and no admission against its control; tampered bundles are flagged."""
    import copy
    from uniserve_v1_b200.tools import eval as E
    kw = dict(concurrency=3, requests=9, prompt_tokens=10, max_tokens=5, model="tiny", seed=3)
    control = asyncio.run(E.run_load(live_server, **kw))
    base = 'model = "random:tiny"\nserved_model_name = "tiny"\n'
    off = base + "[kv_cache_config]\nprefix_caching = false\n"
    run = asyncio.run(E.run_load(live_server, changes=[(0.05, off), (0.25, base)], **kw))
    assert len(run["timeline"]) == 2 and all(e["status"] == 200 for e in run["timeline"])
    assert E.check_change(run, control) == []
    lost = copy.deepcopy(run)
    lost["records"][2]["text"] = lost["records"][2]["text"] + "x"
    lost["records"][4]["error"] = "ClientPayloadError: closed"
    lost["timeline"][0]["status"] = 409
    fails = E.check_change(lost, control)
    assert len(fails) == 3 and any("text differs" in f for f in fails)
    late = copy.deepcopy(run)
    w1 = max(e["done_s"] for e in late["timeline"])
    r = late["records"][0]
    r["submit_s"], r["ttft_s"] = late["timeline"][0]["issued_s"] + 0.001, w1 + 30.0
    assert any("inside the change window" in f for f in E.check_change(late, control))


def test_hot_restart_hands_the_listener_to_a_successor(tmp_path):
    """`POST /admin/restart`: a successor process takes the listening socket over, the first
    process finishes and exits, requests before, during and after are answered alike."""
    import json
    import os
    import subprocess
    import sys
    import urllib.request
    port = _free_port()
    pkg = tmp_path / "pkg"
    pkg.mkdir()
    (pkg / "config.toml").write_text('model = "random:tiny"\nserved_model_name = "tiny"\n'
                                     f'[admin_config]\nhost = "127.0.0.1"\nport = {port}\n')
    env = dict(os.environ, UNISERVE_CPU_RANKS="1")
    env.pop("RANK", None)
    proc = subprocess.Popen([sys.executable, "-m", "uniserve_v1_b200", "serve", str(pkg)], env=env,
                            cwd=os.path.dirname(os.path.dirname(__file__)))
    base = f"http://127.0.0.1:{port}"
    body = json.dumps({"model": "tiny", "max_tokens": 8, "temperature": 0, "ignore_eos": True,
                       "messages": [{"role": "user", "content": "hello there, " * 16}]}).encode()
    cached = []

    def get(path):
        with urllib.request.urlopen(base + path, timeout=5) as r:
            return json.loads(r.read())

    def chat():
        req = urllib.request.Request(base + "/v1/chat/completions", data=body,
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as r:
            out = json.loads(r.read())
        cached.append(out["usage"]["prompt_tokens_details"]["cached_tokens"])
        return out["choices"][0]["message"]["content"]
    successor = None
    try:
        for _ in range(240):
            try:
                first = get("/health")["pid"]
                break
            except Exception:
                assert proc.poll() is None, "server ended"
                time.sleep(0.5)
        assert first == proc.pid
        want = chat()
        req = urllib.request.Request(base + "/admin/restart", data=b"", method="POST")
        with urllib.request.urlopen(req, timeout=30) as r:
            out = json.loads(r.read())
        assert r.status == 202 and out["state"] == "starting" and out["successor_pid"]
        successor = out["successor_pid"]
        assert chat() == want                         # whoever accepts it answers
        for _ in range(240):
            try:
                if get("/health")["pid"] == successor and proc.poll() is not None:
                    break
            except Exception:
                pass
            time.sleep(0.5)
        assert proc.poll() is not None, "the first process did not leave"
        assert get("/health")["pid"] == successor and chat() == want
        # the successor read the first process's cached pages before it served: whichever
        # process answered after the first request found the prompt's pages cached - also the
        # successor on the first request it ever saw
        assert cached[0] == 0 and len(cached) >= 3 and all(c >= 64 for c in cached[1:]), cached
    finally:
        if proc.poll() is None:
            proc.terminate()
        if successor:
            try:
                os.kill(successor, 15)
            except ProcessLookupError:
                pass


def test_standby_is_promoted_when_the_serving_process_dies(tmp_path):
    """`profiling_config.standby`: a parked second process with the model loaded takes the
    listening socket when the serving process is killed, serves as generation 1 - starting
    from the serving process's last snapshot of its cached KV pages - and parks a standby of
    its own."""
    import json
    import os
    import signal
    import subprocess
    import sys
    import urllib.request
    port = _free_port()
    pkg = tmp_path / "pkg"
    pkg.mkdir()
    (pkg / "config.toml").write_text('model = "random:tiny"\nserved_model_name = "tiny"\n'
                                     f'[admin_config]\nhost = "127.0.0.1"\nport = {port}\n'
                                     '[profiling_config]\nstandby = true\nstandby_snapshot = 0.3\n')
    env = dict(os.environ, UNISERVE_CPU_RANKS="1")
    env.pop("RANK", None)
    proc = subprocess.Popen([sys.executable, "-m", "uniserve_v1_b200", "serve", str(pkg)], env=env,
                            cwd=os.path.dirname(os.path.dirname(__file__)))
    base = f"http://127.0.0.1:{port}"
    body = json.dumps({"model": "tiny", "max_tokens": 8, "temperature": 0, "ignore_eos": True,
                       "messages": [{"role": "user", "content": "hello there, " * 16}]}).encode()
    cached = []

    def get(path):
        with urllib.request.urlopen(base + path, timeout=5) as r:
            return json.loads(r.read())

    def chat():
        req = urllib.request.Request(base + "/v1/chat/completions", data=body,
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as r:
            out = json.loads(r.read())
        cached.append(out["usage"]["prompt_tokens_details"]["cached_tokens"])
        return out["choices"][0]["message"]["content"]
    pids = []
    try:
        sb = {"state": "none"}
        for _ in range(360):
            try:
                sb = get("/admin/standby")
                if sb["state"] == "parked":
                    break
            except Exception:
                assert proc.poll() is None, "server ended"
            time.sleep(0.5)
        assert sb["state"] == "parked" and sb["pid"] != proc.pid
        pids.append(sb["pid"])
        assert get("/health")["generation"] == 0
        want = chat()
        time.sleep(1.5)                                 # a snapshot of the cached pages is taken
        os.kill(proc.pid, signal.SIGKILL)               # the serving process dies
        proc.wait(timeout=30)
        h = None
        for _ in range(120):
            try:
                h = get("/health")
                if h["pid"] == sb["pid"]:
                    break
            except Exception:
                pass
            time.sleep(0.25)
        assert h and h["pid"] == sb["pid"] and h["generation"] == 1
        assert chat() == want
        # the promoted standby read the last snapshot: its first request finds the prompt cached
        assert cached[0] == 0 and cached[1] >= 64, cached
        for _ in range(360):                            # and it parks its own standby
            nxt = get("/admin/standby")
            if nxt["state"] == "parked":
                break
            time.sleep(0.5)
        assert nxt["state"] == "parked" and nxt["generation"] == 1
        pids.append(nxt["pid"])
    finally:
        if proc.poll() is None:
            proc.kill()
        for p in pids:                                  # the promoted one first: its standby leaves
            try:
                os.kill(p, signal.SIGTERM)
            except ProcessLookupError:
                pass
        time.sleep(1.0)
        for p in pids:
            try:
                os.kill(p, signal.SIGKILL)
            except ProcessLookupError:
                pass


def test_a_dead_rank_takes_the_deployment_through_a_relaunch(tmp_path):
    """The leader of a two-rank deployment watches the rank it started: when that process is
    killed, the leader replaces itself with a fresh `serve` of the next generation on the same
    listening socket, which starts the ranks again and answers as before."""
    import json
    import os
    import signal
    import subprocess
    import sys
    import urllib.request
    port = _free_port()
    pkg = tmp_path / "pkg"
    pkg.mkdir()
    (pkg / "config.toml").write_text('model = "random:tiny"\nserved_model_name = "tiny"\n'
                                     'tensor_parallel_size = 2\n'
                                     f'[admin_config]\nhost = "127.0.0.1"\nport = {port}\n')
    env = dict(os.environ, UNISERVE_CPU_RANKS="1")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    proc = subprocess.Popen([sys.executable, "-m", "uniserve_v1_b200", "serve", str(pkg)], env=env,
                            cwd=os.path.dirname(os.path.dirname(__file__)))
    base = f"http://127.0.0.1:{port}"
    body = json.dumps({"model": "tiny", "messages": [{"role": "user", "content": "hello there"}],
                       "max_tokens": 8, "temperature": 0, "ignore_eos": True}).encode()

    def get(path):
        with urllib.request.urlopen(base + path, timeout=5) as r:
            return json.loads(r.read())

    def chat():
        req = urllib.request.Request(base + "/v1/chat/completions", data=body,
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as r:
            return json.loads(r.read())["choices"][0]["message"]["content"]
    try:
        for _ in range(360):
            try:
                ranks = get("/admin/ranks")
                break
            except Exception:
                assert proc.poll() is None, "server ended"
                time.sleep(0.5)
        assert len(ranks["ranks"]) == 1 and ranks["ranks"][0]["alive"] and ranks["generation"] == 0
        want = chat()
        os.kill(ranks["ranks"][0]["pid"], signal.SIGKILL)
        h = None
        for _ in range(480):
            try:
                h = get("/health")
                if h.get("generation") == 1 and h["status"] == "ok":
                    break
            except Exception:
                pass
            assert proc.poll() is None, "the leader ended instead of relaunching"
            time.sleep(0.5)
        assert h and h["generation"] == 1 and h["pid"] == proc.pid      # the same process, new image
        assert get("/admin/ranks")["ranks"][0]["pid"] != ranks["ranks"][0]["pid"]
        assert chat() == want
    finally:
        if proc.poll() is None:
            proc.terminate()
            try:
                proc.wait(timeout=30)
            except Exception:
                proc.kill()


def test_supervision_backs_off_relaunches_in_a_row(monkeypatch):
    """The first relaunch after a rank's death is immediate; relaunches that follow one
    another wait `restart_s`, doubling up to `restart_max_s`; an image that served longer
    than that starts the count again; `stop` ends a wait."""
    from uniserve_v1_b200.server import restart as R
    assert [R.restart_delay(n, 5.0, 300.0) for n in (0, 1, 2, 3, 7, 50)] == \
        [0.0, 5.0, 10.0, 20.0, 300.0, 300.0]

    class Child:
        pid = 4242

        def __init__(self):
            self.code = None

        def poll(self):
            return self.code

        def terminate(self):
            self.code = -15

        def wait(self, timeout=None):
            return self.code

    class Listener:
        def fileno(self):
            return 0

    class Sup(R.Supervision):
        def _exec(self):
            self.launched = (time.monotonic(), f"{self.relaunches + 1}")

    def run(env, restart_s=0.3, stop_after=None):
        if env is None:
            monkeypatch.delenv(R.RESTARTS_ENV, raising=False)
        else:
            monkeypatch.setenv(R.RESTARTS_ENV, env)
        dead, alive, said = Child(), Child(), []
        sup = Sup([dead, alive], Listener(), ["serve", "pkg"], 0, on_failure=said.append,
                  period=0.02, restart_s=restart_s, restart_max_s=60.0)
        sup.launched = None
        sup.start()
        t0 = time.monotonic()
        dead.code = 9
        if stop_after is not None:
            time.sleep(stop_after)
            sup.stop()
        sup.thread.join(timeout=10)
        assert said and "rank 1" in said[0] and alive.code == -15
        return sup, (sup.launched[0] - t0 if sup.launched else None)
    sup, after = run(None)
    assert after is not None and after < 0.25 and sup.status()["relaunches"] == 0
    sup, after = run(f"1:{time.time():.3f}")
    assert 0.3 <= after < 0.6 and sup.status()["waiting_s"] == 0.3
    sup, after = run(f"2:{time.time():.3f}")
    assert 0.6 <= after < 1.0
    sup, after = run(f"6:{time.time() - 120:.3f}")           # served for two minutes since
    assert after < 0.25 and sup.relaunches == 0
    sup, after = run("garbage")
    assert after < 0.25
    sup, after = run(f"3:{time.time():.3f}", restart_s=5.0, stop_after=0.2)
    assert after is None and sup.status()["waiting_s"] == 20.0


def test_weights_keeper_handle_records_are_plain_data():
    """A device-memory record carries its IPC handle as JSON of integers, booleans and
    base64 byte strings: it round-trips with its kinds intact, and anything else (a pickle
    stream, a nested object, a string) is refused rather than constructed."""
    import base64
    import pickle
    import pytest
    from uniserve_v1_b200.server.weights_keeper import _handle_from_json, _handle_to_json
    handle = (0, b"\x00\x01\xfehandle" * 4, 1 << 20, 256, b"refcount", 7, b"event" * 13, True)
    text = _handle_to_json(handle)
    back = _handle_from_json(text)
    assert back == handle and [type(x) for x in back] == [type(x) for x in handle]
    with pytest.raises(TypeError):
        _handle_to_json((0, 1.5))
    for bad in (base64.b64encode(pickle.dumps(handle)).decode(), '{"b":"AA=="}', '["text"]',
                '[{"b":"AA==","c":1}]', '[[1]]', '[{"b":"not base64!"}]', "[" + "1," * 16 + "1]"):
        with pytest.raises(ValueError):
            _handle_from_json(bad)


def test_weights_keeper_serves_weights_to_restarting_engines(tmp_path):
    """`keep` holds a model's weights in shared memory; engines built by `serve`'s own model
    constructor map them (no second copy, tied tensors stay tied), give the tokens of a model
    that loaded its own weights, and a keeper of another model is refused."""
    import json
    import os
    import subprocess
    import sys
    from uniserve_v1_b200.__main__ import _qwen3_model
    from uniserve_v1_b200.config.policy import Package
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.server.weights_keeper import attach, stop_keeper
    pkg_dir = tmp_path / "pkg"
    pkg_dir.mkdir()
    (pkg_dir / "config.toml").write_text('model = "random:tiny"\nserved_model_name = "tiny"\n')
    sock = str(tmp_path / "w.sock")
    r, w = os.pipe()
    os.set_inheritable(w, True)
    env = dict(os.environ, UNISERVE_CPU_RANKS="1")
    proc = subprocess.Popen([sys.executable, "-m", "uniserve_v1_b200", "keep", str(pkg_dir),
                             "--socket", sock, "--ready-fd", str(w)], env=env, pass_fds=(w,),
                            cwd=os.path.dirname(os.path.dirname(__file__)))
    os.close(w)
    try:
        line = os.read(r, 4096)
        info = json.loads(line.split(b"\n")[0])
        assert info["state"] == "keeping" and info["tensors"] > 10
        pkg = Package.load(str(pkg_dir))
        prompts = [[(3 * i + j) % 1000 for i in range(n)] for j, n in enumerate((9, 30))]
        sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
        _, own, _ = _qwen3_model(pkg, None, torch.device("cpu"), torch.float32, None)
        want = LLMEngine(own, num_pages=64, max_num_seqs=4, max_model_len=128,
                         use_graphs=False).generate(prompts, sp)
        for _ in range(2):                                   # an engine, then its restart
            _, mapped, _ = _qwen3_model(pkg, None, torch.device("cpu"), torch.float32, None, sock)
            assert mapped.weights_from["keeper_pid"] == proc.pid
            assert torch.equal(mapped.embed, own.embed) and mapped.embed.data_ptr() != own.embed.data_ptr()
            assert (mapped.lm_head is mapped.embed) == (own.lm_head is own.embed)
            got = LLMEngine(mapped, num_pages=64, max_num_seqs=4, max_model_len=128,
                            use_graphs=False).generate(prompts, sp)
            assert got == want
        # another model's keeper is refused: the caller loads the weights itself
        from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
        import dataclasses
        other = Qwen3MoeModel(dataclasses.replace(Qwen3MoeConfig.tiny(), num_hidden_layers=1), "cpu",
                              torch.float32)
        assert attach(other, sock) is False
        assert attach(Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32),
                      str(tmp_path / "nobody.sock")) is False
        assert stop_keeper(sock)
        proc.wait(timeout=30)
        assert not os.path.exists(sock)
    finally:
        os.close(r)
        if proc.poll() is None:
            proc.terminate()


def test_profile_session_collectors_and_admin_route(tmp_path):
    """A session with the ``timeline`` collector records the activity of the process beside
    the fence probes (on CPU ranks: host operator records), closes itself after the asked
    number of steps, and is driven over HTTP by ``/admin/profile``; sampling collectors are
    refused by name."""
    import pytest
    from fastapi.testclient import TestClient
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.engine.profiling import StepProfiler, start_session
    from uniserve_v1_b200.engine.types import SamplingParams
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.server.app import create_app
    from uniserve_v1_b200.tools import profile as P
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    eng = LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=128, use_graphs=False)
    path = str(tmp_path / "tl.sqlite")
    st = start_session(eng, ["fence_timeline", "timeline"], path, steps=3)
    assert st["open"] and st["collectors"] == ["fence_timeline", "timeline"]
    eng.generate([[1, 2, 3, 4, 5]], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    assert eng.profiler.session is None                  # closed itself after three steps
    s = P.load(path)
    assert len(s["spans"]) == 3 and len(s["kernels"]) > 0
    assert s["meta"]["collectors"] == "fence_timeline,timeline"
    summ = P.summary([s])
    assert summ["kernels"] and all(v["count"] >= 1 for v in summ["kernels"].values())
    tr = P.to_trace([s])
    assert any(e["tid"].startswith("host_ops:") for e in tr["traceEvents"])
    assert P.main(["timeline", path, "--limit", "5"]) == 0
    with pytest.raises(ValueError, match="sampling"):
        StepProfiler("cpu").open(str(tmp_path / "x.sqlite"), collectors=["pc_sampling"])
    with pytest.raises(ValueError, match="unknown collector"):
        StepProfiler("cpu").open(str(tmp_path / "y.sqlite"), collectors=["everything"])

    from uniserve_v1_b200.server.tokenizer import ByteTokenizer
    app = create_app(engine=eng, tokenizer=ByteTokenizer(256), served_model_name="tiny")
    with TestClient(app) as c:
        assert c.get("/admin/profile").json()["open"] is False
        out = c.post("/admin/profile", json={"collectors": ["fence_timeline"], "steps": 100,
                                             "output": str(tmp_path)}).json()
        assert out["open"] and out["path"].endswith("rank0.sqlite")
        r = c.post("/v1/chat/completions", json={"model": "tiny", "max_tokens": 3,
                                                 "messages": [{"role": "user", "content": "hi"}]})
        assert r.status_code == 200
        assert c.get("/admin/profile").json()["steps_left"] < 100
        assert c.post("/admin/profile", json={"close": True}).json()["open"] is False
        bad = c.post("/admin/profile", json={"collectors": ["pm_sampling"]})
        assert bad.status_code == 400
    assert len(P.load(str(tmp_path / "rank0.sqlite"))["spans"]) >= 1


def test_admin_prefix_cache_saves_and_loads_over_http(tmp_path):
    """`POST /admin/prefix_cache`: one deployment writes its cached pages, another reads them
    and answers the same prompt from the cache."""
    from fastapi.testclient import TestClient
    from uniserve_v1_b200.engine.engine import LLMEngine
    from uniserve_v1_b200.models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    from uniserve_v1_b200.server.app import create_app
    from uniserve_v1_b200.server.tokenizer import ByteTokenizer
    model = Qwen3MoeModel(Qwen3MoeConfig.tiny(), "cpu", torch.float32).init_random(seed=0)
    path = str(tmp_path / "pages.kv")
    chat = {"model": "tiny", "max_tokens": 3, "temperature": 0, "ignore_eos": True,
            "messages": [{"role": "user", "content": "the same long question, " * 8}]}

    def deployment():
        eng = LLMEngine(model, num_pages=64, max_num_seqs=4, max_model_len=512, use_graphs=False)
        return TestClient(create_app(engine=eng, tokenizer=ByteTokenizer(1024, 1023),
                                     served_model_name="tiny"))
    with deployment() as a:
        first = a.post("/v1/chat/completions", json=chat).json()
        assert first["usage"]["prompt_tokens_details"]["cached_tokens"] == 0
        saved = a.post("/admin/prefix_cache", json={"action": "save", "path": path}).json()
        assert saved["pages"] >= 4
        assert a.post("/admin/prefix_cache", json={"action": "erase", "path": path}).status_code == 400
    with deployment() as b:
        got = b.post("/admin/prefix_cache", json={"action": "load", "path": path}).json()
        assert got["pages"] == saved["pages"]
        again = b.post("/v1/chat/completions", json=chat).json()
        assert again["choices"][0]["message"] == first["choices"][0]["message"]
        assert again["usage"]["prompt_tokens_details"]["cached_tokens"] >= 64
        missing = b.post("/admin/prefix_cache", json={"action": "load", "path": path + ".no"}).json()
        assert missing["pages"] == 0 and "refused" in missing
