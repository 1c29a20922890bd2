"""Data-parallel replicas behind one address.

``data_parallel_size = N`` (or a worker group with ``copies = N``) describes N
independent replicas of a deployment.  Each replica is its own ``serve`` process
(its own GPUs, engine, KV cache); this router is the one address clients talk to.
A request goes to the replica with the fewest requests in flight (ties to the
lowest index); requests that carry ``prompt_cache_key`` stick to one replica so
their prefix pages are found again.  Responses stream through unchanged.
A replica that refuses connections is marked down and retried after a pause;
its request is re-sent once to the next best replica when nothing was streamed
yet.

    python -m uniserve_v1_b200 route --listen 127.0.0.1:8000 \
        --replica http://127.0.0.1:8001 --replica http://127.0.0.1:8002

``--prefix-aware``: requests without a cache key are sent where their prompt prefix is
cached.  The router asks every reachable replica (``POST /internal/probe``: the replica
renders and tokenizes the request and looks its page keys up without allocating) and takes
the one that holds the most tokens, unless it holds fewer than 32 or is more than four
requests busier than the idlest replica; the reference keeps a published cluster directory
for this, here the directory is asked per request.

Roles (``replicas.<id>.role = prefill | decode | mixed``): with ``--prefill URL`` and
``--decode URL`` replicas a chat request is computed up to its first token on a prefill
replica and handed, with the contents of its KV pages, to a decode replica that
streams the answer (``engine/handoff.py``).

Reference behaviour: docs/configuration.md:298, crates/daemon/src/leader.rs:562 (replica
configs), :1834 (submit_routed); reference project paths.
"""
from __future__ import annotations

import asyncio
import hashlib
import json
import time
from typing import Optional

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, Response, StreamingResponse


class Replica:
    def __init__(self, url: str):
        self.url = url.rstrip("/")
        self.in_flight = 0
        self.served = 0
        self.down_until = 0.0

    @property
    def up(self) -> bool:
        return time.monotonic() >= self.down_until


class ReplicaRouter:
    def __init__(self, urls: list, retry_after_s: float = 2.0, program=None):
        """``program``: an ``engine.program.ProgramHost`` whose ``route(request, replicas)``
        returns the index of the replica to use (facts: the request's body size and cache key;
        per replica its index, requests in flight, requests served and whether it is up).  A
        missing, faulting or out-of-range answer falls back to fewest-in-flight."""
        assert urls, "at least one replica"
        self.replicas = [Replica(u) for u in urls]
        self.retry_after_s = retry_after_s
        self.program = program
        self.program_faults = 0
        self.probes = 0            # prefix-aware routing: requests probed / sent to a holder
        self.prefix_hits = 0

    def pick(self, affinity: Optional[str] = None, exclude=(), size: int = 0,
             prefer: Optional[Replica] = None) -> Optional[Replica]:
        live = [r for r in self.replicas if r.up and r not in exclude] or \
            [r for r in self.replicas if r not in exclude]
        if not live:
            return None
        if prefer is not None and prefer in live:
            return prefer
        if self.program is not None and self.program.has("route"):
            try:
                i = self.program.call("route", {"bytes": size, "cache_key": affinity},
                                      [{"index": self.replicas.index(r), "in_flight": r.in_flight,
                                        "served": r.served, "up": r.up} for r in live])
                by_index = {self.replicas.index(r): r for r in live}
                if isinstance(i, int) and i in by_index:
                    return by_index[i]
                self.program_faults += 1
            except Exception:
                self.program_faults += 1
        if affinity:
            h = int.from_bytes(hashlib.sha256(affinity.encode()).digest()[:8], "big")
            return live[h % len(live)]
        return min(live, key=lambda r: (r.in_flight, self.replicas.index(r)))

    def mark_down(self, r: Replica) -> None:
        r.down_until = time.monotonic() + self.retry_after_s

    def stats(self) -> list:
        return [{"url": r.url, "in_flight": r.in_flight, "served": r.served, "up": r.up}
                for r in self.replicas]


def create_router_app(urls: list, api_key: Optional[str] = None,
                      prefill_urls: Optional[list] = None,
                      decode_urls: Optional[list] = None, program=None,
                      internal_key: Optional[str] = None, prefix_aware: bool = False,
                      probe_timeout_s: float = 0.25, prefix_min_tokens: int = 32,
                      prefix_slack: int = 4, transfer_deadline_s: float = 60.0) -> FastAPI:
    """``urls``: replicas of role ``mixed``.  With ``prefill_urls`` and ``decode_urls`` chat
    requests are disaggregated: a prefill replica computes the prompt and the first token
    (``/internal/prefill``), its answer - the request's framed state - goes to a decode
    replica (``/internal/decode``), whose stream is relayed to the client.  ``internal_key``
    is presented on both internal routes; the replicas refuse them without it.  Both legs of
    a hand-off have ``transfer_deadline_s`` to complete - the prefill replica to answer with the
    frames, the decode replica to take them and start its answer; a leg that misses it is
    answered 504 and counted (``storage_config.transfer_deadline_s`` of the reference's
    policy package, 60 s by default)."""
    import aiohttp
    router = ReplicaRouter(urls or (list(prefill_urls or []) + list(decode_urls or [])),
                           program=program)
    pre = ReplicaRouter(prefill_urls) if prefill_urls else None
    dec = ReplicaRouter(decode_urls) if decode_urls else None
    app = FastAPI(title="uniserve_v1_b200 replica router")
    app.state.router, app.state.prefill, app.state.decode = router, pre, dec
    state = {"session": None, "deadline_misses": 0}
    leg = aiohttp.ClientTimeout(total=max(0.001, float(transfer_deadline_s)))

    def _missed(which: str):
        state["deadline_misses"] += 1
        return JSONResponse({"error": {
            "message": f"the {which} replica did not complete its leg of the hand-off within "
                       f"the transfer deadline ({transfer_deadline_s:g} s)",
            "type": "timeout"}}, status_code=504)

    async def session():
        if state["session"] is None:
            state["session"] = aiohttp.ClientSession(
                timeout=aiohttp.ClientTimeout(total=None, sock_connect=5))
        return state["session"]

    @app.on_event("shutdown")
    async def _close():
        if state["session"] is not None:
            await state["session"].close()

    def _headers(req: Request) -> dict:
        keep = ("authorization", "content-type", "accept")
        return {k: v for k, v in req.headers.items() if k.lower() in keep}

    def _internal(req: Request) -> dict:
        return dict(_headers(req), **{"x-uniserve-internal-key": internal_key or ""})

    async def where_cached(body: bytes) -> Optional[Replica]:
        """``prefix_aware``: every reachable replica says how many tokens of the request's
        prompt it holds (``/internal/probe``); the request goes to the best one when it holds
        at least ``prefix_min_tokens`` and is not ``prefix_slack`` requests busier than the
        idlest replica.  Replicas that do not answer in ``probe_timeout_s`` do not count."""
        import asyncio
        s = await session()
        live = [r for r in router.replicas if r.up]
        if len(live) < 2:
            return None

        async def ask(r):
            try:
                async with s.post(r.url + "/internal/probe", data=body,
                                  headers={"content-type": "application/json",
                                           "x-uniserve-internal-key": internal_key or ""},
                                  timeout=aiohttp.ClientTimeout(total=probe_timeout_s)) as up:
                    if up.status != 200:
                        return r, -1
                    return r, int((await up.json()).get("cached_tokens", 0))
            except Exception:
                return r, -1
        got = await asyncio.gather(*[ask(r) for r in live])
        router.probes += 1
        best, tokens = max(got, key=lambda g: (g[1], -g[0].in_flight))
        idlest = min(r.in_flight for r in live)
        if tokens >= prefix_min_tokens and best.in_flight - idlest <= prefix_slack:
            router.prefix_hits += 1
            return best
        return None

    async def forward(req: Request, path: str):
        body = await req.body()
        affinity = None
        if body and req.headers.get("content-type", "").startswith("application/json"):
            try:
                affinity = json.loads(body).get("prompt_cache_key")
            except Exception:
                affinity = None
        prefer = None
        if prefix_aware and not affinity and body and path == "/v1/chat/completions":
            prefer = await where_cached(body)
        tried = []
        s = await session()
        while True:
            r = router.pick(affinity, exclude=tried, size=len(body or b""),
                            prefer=prefer if not tried else None)
            if r is None:
                return JSONResponse({"error": {"message": "no replica is reachable",
                                               "type": "service_unavailable"}}, status_code=503)
            tried.append(r)
            r.in_flight += 1
            try:
                up = await s.request(req.method, r.url + path, data=body or None,
                                     headers=_headers(req), params=dict(req.query_params))
            except aiohttp.ClientConnectionError:
                r.in_flight -= 1
                router.mark_down(r)
                continue
            ctype = up.headers.get("content-type", "application/octet-stream")
            extra = {k: v for k, v in up.headers.items() if k.lower().startswith("x-video-")}
            if ctype.startswith("text/event-stream"):
                async def relay(up=up, r=r):
                    try:
                        async for chunk in up.content.iter_any():
                            yield chunk
                    finally:
                        up.release()
                        r.in_flight -= 1
                        r.served += 1
                return StreamingResponse(relay(), status_code=up.status, media_type=ctype,
                                         headers=extra)
            try:
                data = await up.read()
            finally:
                up.release()
                r.in_flight -= 1
                r.served += 1
            return Response(content=data, status_code=up.status, media_type=ctype, headers=extra)

    async def disaggregated(req: Request):
        import base64
        body = await req.body()
        s = await session()
        p = pre.pick()
        p.in_flight += 1
        try:
            async with s.post(p.url + "/internal/prefill", data=body, headers=_internal(req),
                              timeout=leg) as up:
                blob, status = await up.read(), up.status
                ctype = up.headers.get("content-type", "")
        except asyncio.TimeoutError:
            return _missed("prefill")
        except aiohttp.ClientConnectionError:
            pre.mark_down(p)
            return JSONResponse({"error": {"message": "no prefill replica is reachable",
                                           "type": "service_unavailable"}}, status_code=503)
        finally:
            p.in_flight -= 1
            p.served += 1
        if not ctype.startswith("application/octet-stream"):
            # an error, or a request that its first token already ended
            return Response(content=blob, status_code=status, media_type=ctype or "application/json")
        d = dec.pick()
        d.in_flight += 1
        payload = json.dumps({"request": json.loads(body),
                              "handoff": base64.b64encode(blob).decode()})
        hdr = dict(_internal(req), **{"content-type": "application/json"})
        try:
            # the deadline covers the delivery and the first byte of the answer; the stream
            # that follows is the request's own
            up = await asyncio.wait_for(
                s.post(d.url + "/internal/decode", data=payload, headers=hdr),
                timeout=max(0.001, float(transfer_deadline_s)))
        except asyncio.TimeoutError:
            d.in_flight -= 1
            return _missed("decode")
        except aiohttp.ClientConnectionError:
            d.in_flight -= 1
            dec.mark_down(d)
            return JSONResponse({"error": {"message": "no decode replica is reachable",
                                           "type": "service_unavailable"}}, status_code=503)
        ctype = up.headers.get("content-type", "application/json")

        async def relay():
            try:
                async for chunk in up.content.iter_any():
                    yield chunk
            finally:
                up.release()
                d.in_flight -= 1
                d.served += 1
        return StreamingResponse(relay(), status_code=up.status, media_type=ctype)

    @app.get("/health")
    async def health():
        s = await session()
        ok = 0
        for r in router.replicas:
            try:
                async with s.get(r.url + "/health") as up:
                    ok += up.status == 200
            except Exception:
                router.mark_down(r)
        code = 200 if ok else 503
        return JSONResponse({"status": "ok" if ok else "down", "replicas_up": ok,
                             "replicas": len(router.replicas)}, status_code=code)

    @app.get("/router/replicas")
    async def replicas():
        return router.stats()

    @app.get("/router/stats")
    async def router_stats():
        return {"replicas": router.stats(), "prefix_aware": prefix_aware,
                "probes": router.probes, "prefix_hits": router.prefix_hits,
                "program_faults": router.program_faults,
                "transfer_deadline_s": transfer_deadline_s,
                "deadline_misses": state["deadline_misses"]}

    @app.api_route("/{path:path}", methods=["GET", "POST", "PUT", "DELETE"])
    async def any_route(path: str, req: Request):
        if pre is not None and dec is not None and req.method == "POST" and \
                path == "v1/chat/completions":
            return await disaggregated(req)
        return await forward(req, "/" + path)

    return app
