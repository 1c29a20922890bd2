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

Reference behaviour: docs/configuration.md:298, crates/daemon/src/leader.rs:562 (replica
configs), :1834 (submit_routed); reference project paths.
"""
from __future__ import annotations

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
    def __init__(self, urls: list, retry_after_s: float = 2.0):
        assert urls, "at least one replica"
        self.replicas = [Replica(u) for u in urls]
        self.retry_after_s = retry_after_s

    def pick(self, affinity: Optional[str] = None, exclude=()) -> Optional[Replica]:
        live = [r for r in self.replicas if r.up and r not in exclude] or \
            [r for r in self.replicas if r not in exclude]
        if not live:
            return None
        if affinity:
            h = int.from_bytes(hashlib.sha256(affinity.encode()).digest()[:8], "big")
            return live[h % len(live)]
        return min(live, key=lambda r: (r.in_flight, self.replicas.index(r)))

    def mark_down(self, r: Replica) -> None:
        r.down_until = time.monotonic() + self.retry_after_s

    def stats(self) -> list:
        return [{"url": r.url, "in_flight": r.in_flight, "served": r.served, "up": r.up}
                for r in self.replicas]


def create_router_app(urls: list, api_key: Optional[str] = None) -> FastAPI:
    import aiohttp
    router = ReplicaRouter(urls)
    app = FastAPI(title="uniserve_v1_b200 replica router")
    app.state.router = router
    state = {"session": None}

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

    async def forward(req: Request, path: str):
        body = await req.body()
        affinity = None
        if body and req.headers.get("content-type", "").startswith("application/json"):
            try:
                affinity = json.loads(body).get("prompt_cache_key")
            except Exception:
                affinity = None
        tried = []
        s = await session()
        while True:
            r = router.pick(affinity, exclude=tried)
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

    @app.api_route("/{path:path}", methods=["GET", "POST", "PUT", "DELETE"])
    async def any_route(path: str, req: Request):
        return await forward(req, "/" + path)

    return app
