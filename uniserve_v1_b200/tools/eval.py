"""Measures a serving system through its public HTTP interface.

    python -m uniserve_v1_b200.tools.eval run --url http://127.0.0.1:8000 --concurrency 64 \
        --requests 256 --prompt-tokens 128 --max-tokens 256 --out bundle.json
    python -m uniserve_v1_b200.tools.eval compare reference.json candidate.json
    python -m uniserve_v1_b200.tools.eval check-stop bundle.json
    python -m uniserve_v1_b200.tools.eval check-change run.json control.json
    python -m uniserve_v1_b200.tools.eval check-faults bundle.json

``run`` drives ``POST /v1/chat/completions`` with a closed loop of ``concurrency``
clients (streaming, so the first-token time is observed), validates every
response and writes a *bundle*: one record per request plus a summary (output
tokens/s, request latency, time to first token and time per output token at
p50/p95/p99).  ``compare`` holds a candidate bundle to a reference bundle with a
relative tolerance, or two GSM8K-style accuracy counts to the two-sided 95 %
interval of a difference of proportions.  ``check-stop`` verifies stop handling
(no stop string in any text, finish reasons agree with the budget) and
``check-faults`` that every request of a fault-injection run ended in a clean
terminal state.  Exit status 2 marks a failed validation.

Reference: tools/eval/src/main.rs:1-7, tools/eval/src/check.rs (reference project paths).
"""
from __future__ import annotations

import argparse
import asyncio
import json
import math
import random
import statistics
import sys
import time
from dataclasses import asdict, dataclass, field
from typing import Optional


@dataclass
class Record:
    index: int
    ok: bool = False
    status: int = 0
    error: Optional[str] = None
    latency_s: float = 0.0
    ttft_s: Optional[float] = None
    output_tokens: int = 0
    prompt_tokens: int = 0
    cached_tokens: int = 0
    finish_reason: Optional[str] = None
    text: str = ""
    chunks: int = 0
    stop: list = field(default_factory=list)
    max_tokens: int = 0
    submit_s: float = 0.0          # when the load issued it, from the load's start


def percentile(xs, p):
    if not xs:
        return None
    xs = sorted(xs)
    k = (len(xs) - 1) * p
    lo, hi = math.floor(k), math.ceil(k)
    return xs[lo] + (xs[hi] - xs[lo]) * (k - lo)


def synth_prompt(rng: random.Random, tokens: int) -> str:
    """About ``tokens`` tokens of pronounceable filler (one short word per token)."""
    syll = ["ka", "mi", "to", "ra", "ne", "so", "lu", "vi", "pe", "da", "go", "he"]
    return " ".join(rng.choice(syll) + rng.choice(syll) for _ in range(max(1, tokens)))


async def one_request(session, url, headers, body, rec: Record, timeout_s: float):
    import aiohttp
    t0 = time.perf_counter()
    try:
        async with session.post(url + "/v1/chat/completions", json=body, headers=headers,
                                timeout=aiohttp.ClientTimeout(total=timeout_s)) as resp:
            rec.status = resp.status
            if resp.status != 200:
                rec.error = (await resp.text())[:500]
                return
            if body.get("stream"):
                async for raw in resp.content:
                    line = raw.decode().strip()
                    if not line.startswith("data:"):
                        continue
                    data = line[5:].strip()
                    if data == "[DONE]":
                        break
                    ev = json.loads(data)
                    if "error" in ev:
                        rec.error = json.dumps(ev["error"])[:500]
                        return
                    for ch in ev.get("choices", []):
                        delta = ch.get("delta", {})
                        piece = (delta.get("content") or "") + (delta.get("reasoning") or "")
                        # the first chunk after the role announcement carries the first token,
                        # even when its bytes do not yet form printable text
                        if piece or delta.get("tool_calls") or "role" not in delta:
                            if rec.ttft_s is None and not ch.get("finish_reason"):
                                rec.ttft_s = time.perf_counter() - t0
                        if piece or delta.get("tool_calls"):
                            rec.text += piece
                            rec.chunks += 1
                        if ch.get("finish_reason"):
                            rec.finish_reason = ch["finish_reason"]
                            if rec.ttft_s is None:      # no printable piece was ever streamed
                                rec.ttft_s = time.perf_counter() - t0
                    if ev.get("usage"):
                        u = ev["usage"]
                        rec.output_tokens = u.get("completion_tokens", 0)
                        rec.prompt_tokens = u.get("prompt_tokens", 0)
                        rec.cached_tokens = (u.get("prompt_tokens_details") or {}).get(
                            "cached_tokens", 0)
            else:
                ev = await resp.json()
                ch = ev["choices"][0]
                rec.text = ch["message"].get("content") or ""
                rec.finish_reason = ch.get("finish_reason")
                u = ev.get("usage", {})
                rec.output_tokens = u.get("completion_tokens", 0)
                rec.prompt_tokens = u.get("prompt_tokens", 0)
            rec.ok = rec.finish_reason is not None
    except Exception as e:     # noqa: BLE001 - a load generator records every failure
        rec.error = f"{type(e).__name__}: {e}"
    finally:
        rec.latency_s = time.perf_counter() - t0


async def run_load(url: str, concurrency: int, requests: int, prompt_tokens: int, max_tokens: int,
                   stream: bool = True, api_key: Optional[str] = None, model: str = "default",
                   seed: int = 0, stop: Optional[list] = None, temperature: float = 0.0,
                   timeout_s: float = 600.0, ignore_eos: bool = True,
                   changes: Optional[list] = None) -> dict:
    """``changes``: [(seconds from the start, policy text)] - each is PUT to ``/admin/policy``
    while the load runs; the bundle's ``timeline`` records when each was issued and applied."""
    import aiohttp
    headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}
    records = [Record(i, stop=stop or [], max_tokens=max_tokens) for i in range(requests)]
    # prompts depend on the request's index only, so a run and its control send the same ones
    prompts = [synth_prompt(random.Random(seed * 1000003 + i), prompt_tokens)
               for i in range(requests)]
    timeline: list = []
    queue: asyncio.Queue = asyncio.Queue()
    for r in records:
        queue.put_nowait(r)
    t0 = time.perf_counter()

    async def client(session):
        while True:
            try:
                rec = queue.get_nowait()
            except asyncio.QueueEmpty:
                return
            body = {"model": model, "max_tokens": max_tokens, "temperature": temperature,
                    "stream": stream, "seed": seed + rec.index, "ignore_eos": ignore_eos,
                    "messages": [{"role": "user", "content": prompts[rec.index]}]}
            if stream:
                body["stream_options"] = {"include_usage": True}
            if stop:
                body["stop"] = stop
            rec.submit_s = time.perf_counter() - t0
            await one_request(session, url, headers, body, rec, timeout_s)

    async def changer(session):
        for at, text in sorted(changes or []):
            await asyncio.sleep(max(0.0, at - (time.perf_counter() - t0)))
            ev = {"issued_s": time.perf_counter() - t0}
            try:
                async with session.put(url + "/admin/policy", data=text, headers=dict(
                        headers, **{"Content-Type": "application/toml"})) as resp:
                    ev["status"] = resp.status
                    ev["answer"] = (await resp.text())[:300]
            except Exception as e:     # noqa: BLE001
                ev["status"], ev["answer"] = 0, f"{type(e).__name__}: {e}"
            ev["done_s"] = time.perf_counter() - t0
            timeline.append(ev)

    conn = aiohttp.TCPConnector(limit=0)
    async with aiohttp.ClientSession(connector=conn) as session:
        await asyncio.gather(changer(session), *[client(session) for _ in range(concurrency)])
    wall = time.perf_counter() - t0
    b = bundle_of(records, wall, dict(url=url, concurrency=concurrency, requests=requests,
                                      prompt_tokens=prompt_tokens, max_tokens=max_tokens,
                                      stream=stream, seed=seed))
    b["timeline"] = timeline
    return b


def bundle_of(records, wall_s: float, point: dict) -> dict:
    good = [r for r in records if r.ok]
    lat = [r.latency_s for r in good]
    ttft = [r.ttft_s for r in good if r.ttft_s is not None]
    tpot = [(r.latency_s - r.ttft_s) / max(1, r.output_tokens - 1) for r in good
            if r.ttft_s is not None and r.output_tokens > 1]
    out_tokens = sum(r.output_tokens for r in good)
    pct = lambda xs: {"p50": percentile(xs, .5), "p95": percentile(xs, .95),
                      "p99": percentile(xs, .99),
                      "mean": statistics.fmean(xs) if xs else None}
    return {"point": point, "wall_s": wall_s,
            "summary": {"requests": len(records), "succeeded": len(good),
                        "failed": len(records) - len(good), "output_tokens": out_tokens,
                        "output_tokens_per_s": out_tokens / wall_s if wall_s > 0 else 0.0,
                        "requests_per_s": len(good) / wall_s if wall_s > 0 else 0.0,
                        "latency_s": pct(lat), "ttft_s": pct(ttft), "tpot_s": pct(tpot)},
            "records": [asdict(r) for r in records]}


# ------------------------------------------------------------------ checks ----
def compare_bundles(ref: dict, cand: dict, tolerance: float = 0.05) -> list:
    """Regressions of the candidate against the reference (empty = pass)."""
    fails = []
    rs, cs = ref["summary"], cand["summary"]
    if cs["failed"] > rs["failed"]:
        fails.append(f"failed requests {cs['failed']} > {rs['failed']}")
    if cs["output_tokens_per_s"] < rs["output_tokens_per_s"] * (1 - tolerance):
        fails.append(f"output tokens/s {cs['output_tokens_per_s']:.1f} < "
                     f"{rs['output_tokens_per_s']:.1f} - {tolerance:.0%}")
    for key in ("latency_s", "ttft_s", "tpot_s"):
        a, b = rs[key]["p50"], cs[key]["p50"]
        if a is not None and b is not None and b > a * (1 + tolerance):
            fails.append(f"{key} p50 {b:.4f} > {a:.4f} + {tolerance:.0%}")
    return fails


def compare_accuracy(ref_correct: int, cand_correct: int, n: int) -> dict:
    """Two-sided 95 % interval of the difference of two proportions over the same
    ``n`` problems; the candidate passes when the interval contains zero or lies above it."""
    p1, p2 = ref_correct / n, cand_correct / n
    se = math.sqrt(p1 * (1 - p1) / n + p2 * (1 - p2) / n)
    lo, hi = (p2 - p1) - 1.96 * se, (p2 - p1) + 1.96 * se
    return {"reference": p1, "candidate": p2, "difference": p2 - p1, "interval": [lo, hi],
            "pass": hi >= 0.0}


def check_stop(bundle: dict) -> list:
    fails = []
    for r in bundle["records"]:
        if not r["ok"]:
            continue
        for s in r.get("stop") or []:
            if s and s in r["text"]:
                fails.append(f"request {r['index']}: stop string {s!r} in the text")
        if r["finish_reason"] == "length" and r["max_tokens"] and \
                r["output_tokens"] != r["max_tokens"]:
            fails.append(f"request {r['index']}: finish 'length' at {r['output_tokens']} of "
                         f"{r['max_tokens']} tokens")
        if r["finish_reason"] == "stop" and r["max_tokens"] and \
                r["output_tokens"] > r["max_tokens"]:
            fails.append(f"request {r['index']}: {r['output_tokens']} tokens exceed the budget")
    return fails


def check_change(run: dict, control: dict) -> list:
    """A run whose deployment was changed while it served, against its control (the same load
    without the changes): (1) no failed request - each answered 200 and ended at ``length``
    with exactly its requested tokens; (2) no closed connection; (3) no token lost or
    repeated - each text equals the control's text of the same request; (4) new requests
    were admitted throughout - a request submitted inside the changes' window had its first
    token by the window's end plus the control's 99th-percentile time to first token; and
    every change was accepted."""
    fails = []
    ctl = {r["index"]: r for r in control["records"]}
    for ev in run.get("timeline") or []:
        if ev.get("status") != 200:
            fails.append(f"change at {ev.get('issued_s', 0):.2f} s answered {ev.get('status')}: "
                         f"{ev.get('answer')}")
    win = None
    if run.get("timeline"):
        win = (min(e["issued_s"] for e in run["timeline"]),
               max(e["done_s"] for e in run["timeline"]))
    p99 = (control["summary"]["ttft_s"] or {}).get("p99") or 0.0
    for r in run["records"]:
        i = r["index"]
        if r["error"]:
            fails.append(f"request {i}: connection ended: {r['error']}")
            continue
        if r["status"] != 200 or r["finish_reason"] != "length" or \
                (r["max_tokens"] and r["output_tokens"] != r["max_tokens"]):
            fails.append(f"request {i}: status {r['status']}, finish {r['finish_reason']}, "
                         f"{r['output_tokens']} of {r['max_tokens']} tokens")
            continue
        c = ctl.get(i)
        if c is not None and c["ok"] and c["text"] != r["text"]:
            fails.append(f"request {i}: text differs from the control's")
        if win and win[0] <= r["submit_s"] <= win[1] and r["ttft_s"] is not None and \
                r["submit_s"] + r["ttft_s"] > win[1] + p99 + 1e-3:
            fails.append(f"request {i}: submitted at {r['submit_s']:.2f} s inside the change "
                         f"window, first token only at {r['submit_s'] + r['ttft_s']:.2f} s")
    return fails


def check_faults(bundle: dict) -> list:
    """Every request of a fault-injection run reached a terminal state: a finish
    reason, or an HTTP / stream error that names the failure; none hung."""
    fails = []
    for r in bundle["records"]:
        if r["ok"]:
            continue
        if not r["error"] and r["status"] in (0, 200):
            fails.append(f"request {r['index']}: neither finished nor failed")
        if r["error"] and "TimeoutError" in r["error"]:
            fails.append(f"request {r['index']}: timed out ({r['latency_s']:.1f} s)")
    return fails


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="uniserve-eval", description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("run")
    r.add_argument("--url", required=True)
    r.add_argument("--concurrency", type=int, default=8)
    r.add_argument("--requests", type=int, default=32)
    r.add_argument("--prompt-tokens", type=int, default=128)
    r.add_argument("--max-tokens", type=int, default=128)
    r.add_argument("--no-stream", action="store_true")
    r.add_argument("--api-key")
    r.add_argument("--model", default="default")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--stop", action="append")
    r.add_argument("--temperature", type=float, default=0.0)
    r.add_argument("--out")
    r.add_argument("--change", action="append", default=[], metavar="SECONDS:FILE",
                   help="PUT the policy text of FILE to /admin/policy SECONDS into the load")
    pl = sub.add_parser("plan", help="what `run` would send, without sending it")
    for flag, kw in (("--concurrency", dict(type=int, default=8)), ("--requests", dict(type=int, default=32)),
                     ("--prompt-tokens", dict(type=int, default=128)),
                     ("--max-tokens", dict(type=int, default=128)), ("--seed", dict(type=int, default=0)),
                     ("--model", dict(default="default")), ("--temperature", dict(type=float, default=0.0))):
        pl.add_argument(flag, **kw)
    pl.add_argument("--stop", action="append")
    pl.add_argument("--no-stream", action="store_true")
    pl.add_argument("--change", action="append", default=[], metavar="SECONDS:FILE")
    sub.add_parser("list", help="the verbs and what each checks")
    cc = sub.add_parser("check-change")
    cc.add_argument("run")
    cc.add_argument("control")
    c = sub.add_parser("compare")
    c.add_argument("reference")
    c.add_argument("candidate")
    c.add_argument("--tolerance", type=float, default=0.05)
    a = sub.add_parser("compare-accuracy")
    a.add_argument("reference_correct", type=int)
    a.add_argument("candidate_correct", type=int)
    a.add_argument("n", type=int)
    for name in ("check-stop", "check-faults"):
        s = sub.add_parser(name)
        s.add_argument("bundle")
    args = ap.parse_args(argv)
    if args.cmd == "list":
        print(json.dumps({
            "run": "concurrent chat requests with synthetic prompts; a bundle of per-request "
                   "records (tokens, latencies, finish reasons, usage) and a summary",
            "plan": "the requests `run` would send (prompt digests, seeds, bodies) and its policy changes",
            "compare": "two bundles: same outputs per request index, throughput and latency within a tolerance",
            "compare-accuracy": "two accuracies on n items: difference against the binomial noise",
            "check-change": "a run with policy changes against its control: no request lost or altered by a change",
            "check-stop": "stop strings end the text where they first occur and are not part of it",
            "check-faults": "every request finished or failed with an error body; none hung"}, indent=1))
        return 0
    if args.cmd == "plan":
        import hashlib
        prompts = [synth_prompt(random.Random(args.seed * 1000003 + i), args.prompt_tokens)
                   for i in range(args.requests)]
        plan = {"requests": args.requests, "concurrency": args.concurrency,
                "stream": not args.no_stream,
                "body": {"model": args.model, "max_tokens": args.max_tokens,
                         "temperature": args.temperature, "ignore_eos": True,
                         **({"stop": args.stop} if args.stop else {})},
                "items": [{"index": i, "seed": args.seed + i, "prompt_chars": len(p),
                           "prompt_sha256": hashlib.sha256(p.encode()).hexdigest()[:16]}
                          for i, p in enumerate(prompts)],
                "changes": [{"at_s": float(c.split(":", 1)[0]), "file": c.split(":", 1)[1]}
                            for c in args.change]}
        print(json.dumps(plan, indent=1))
        return 0
    if args.cmd == "run":
        b = asyncio.run(run_load(args.url, args.concurrency, args.requests, args.prompt_tokens,
                                 args.max_tokens, not args.no_stream, args.api_key, args.model,
                                 args.seed, args.stop, args.temperature,
                                 changes=[(float(c.split(":", 1)[0]), open(c.split(":", 1)[1]).read())
                                          for c in args.change]))
        if args.out:
            with open(args.out, "w") as f:
                json.dump(b, f)
        print(json.dumps(b["summary"], indent=1))
        return 0 if b["summary"]["failed"] == 0 else 2
    if args.cmd == "compare":
        fails = compare_bundles(json.load(open(args.reference)), json.load(open(args.candidate)),
                                args.tolerance)
    elif args.cmd == "compare-accuracy":
        res = compare_accuracy(args.reference_correct, args.candidate_correct, args.n)
        print(json.dumps(res))
        return 0 if res["pass"] else 2
    elif args.cmd == "check-change":
        fails = check_change(json.load(open(args.run)), json.load(open(args.control)))
    elif args.cmd == "check-stop":
        fails = check_stop(json.load(open(args.bundle)))
    else:
        fails = check_faults(json.load(open(args.bundle)))
    for f in fails:
        print("FAIL:", f)
    print("pass" if not fails else f"{len(fails)} failure(s)")
    return 0 if not fails else 2


if __name__ == "__main__":
    sys.exit(main())
