"""HTTP admission API.

Routes (README.md:89-111 of the reference project): ``GET /health``, ``/version``,
``/v1/models``, ``/v1/capabilities``; ``POST /v1/chat/completions`` (streaming and
not, usage with ``prompt_tokens_details.cached_tokens``, logprobs, tools in JSON
and XML form, reasoning split, stop strings, seed, penalties ...);
``POST /v1/videos/sync``, ``POST/GET/DELETE /v1/videos[/{id}[/content]]``;
``GET/PUT /admin/policy``, ``GET/POST /admin/query``; ``GET /metrics``.
A text deployment registers the chat route, a video deployment the video routes
and ``/v1/capabilities``; anything else answers 404 ``{"detail": "Not Found"}``.
With an API key configured every route but ``/health`` requires it.
"""
from __future__ import annotations

import asyncio
import json
import os
import time
import uuid
from typing import Optional

from fastapi import FastAPI, Request
from fastapi.exceptions import RequestValidationError
from fastapi.responses import JSONResponse, PlainTextResponse, Response, StreamingResponse
from pydantic import ValidationError

from ..config.policy import ConfigError, Package, strongest_effect
from ..engine.types import FinishReason, SamplingParams, StepOutput
from .chat import ChatTemplate, ReasoningSplitter, StopStrings, ToolCallParser
from .engine_service import EngineService, Overloaded
from .observation import ObservationStore
from .protocol import ChatCompletionRequest, VideoGenerationRequest, openai_error
from .tokenizer import IncrementalDecoder

VERSION = "0.1.0"


class _UnsupportedMedia(Exception):
    pass


def _err(status: int, message: str, type_="invalid_request_error", code=None, param=None,
         headers=None):
    return JSONResponse(openai_error(message, type_, code, param), status_code=status,
                        headers=headers)


def lower_sampling(req: ChatCompletionRequest, tokenizer, defaults: dict, max_model_len: int,
                   prompt_len: int, max_logprobs: int = 20) -> SamplingParams:
    """OpenAI fields -> SamplingParams, with the checkpoint's generation_config
    defaults where the request states none (input/sampling.rs, reference)."""
    d = defaults or {}
    temperature = req.temperature if req.temperature is not None else d.get("temperature", 1.0)
    top_p = req.top_p if req.top_p is not None else d.get("top_p", 1.0)
    top_k = req.top_k if req.top_k is not None else d.get("top_k", 0)
    max_tokens = req.max_completion_tokens or req.max_tokens or (max_model_len - prompt_len)
    max_tokens = max(1, min(max_tokens, max_model_len - prompt_len))
    if req.top_logprobs and req.top_logprobs > max_logprobs:
        raise ValueError(f"top_logprobs is at most {max_logprobs}")
    bias = {int(k): float(v) for k, v in (req.logit_bias or {}).items()}
    bad = []
    for w in req.bad_words or []:
        for form in (w, " " + w):
            ids = tokenizer.encode(form)
            if ids:
                bad.append(ids)
    return SamplingParams(
        temperature=temperature, top_k=top_k or 0, top_p=top_p,
        min_p=req.min_p if req.min_p is not None else d.get("min_p", 0.0),
        repetition_penalty=req.repetition_penalty if req.repetition_penalty is not None
        else d.get("repetition_penalty", 1.0),
        frequency_penalty=req.frequency_penalty or 0.0, presence_penalty=req.presence_penalty or 0.0,
        logit_bias=bias or None, allowed_token_ids=req.allowed_token_ids, bad_words_ids=bad or None,
        min_tokens=req.min_tokens or 0, max_tokens=max_tokens, ignore_eos=bool(req.ignore_eos),
        seed=req.seed, stop_token_ids=tuple(req.stop_token_ids or ()),
        logprobs=bool(req.logprobs), top_logprobs=req.top_logprobs or 0)


class ChatRun:
    """One chat request's output path: detokenise -> stop strings -> reasoning
    split -> tool-call parse -> OpenAI chunks."""

    def __init__(self, app_state, req: ChatCompletionRequest, rid: str, prompt_len: int):
        self.s = app_state
        self.req = req
        self.rid = rid
        self.created = int(time.time())
        self.decoder = IncrementalDecoder(app_state.tokenizer,
                                          req.skip_special_tokens is not False)
        stops = [req.stop] if isinstance(req.stop, str) else (req.stop or [])
        self.stops = StopStrings(stops)
        self.reasoning = ReasoningSplitter() if app_state.reasoning else None
        self.tools = ToolCallParser([t.model_dump() for t in req.tools]) \
            if req.tools and req.tool_choice != "none" else None
        self.prompt_len = prompt_len
        self.completion_tokens = 0
        self.cached = 0
        self.finish: Optional[str] = None
        self.content, self.reason_text, self.calls = [], [], []
        self.logprobs = []
        self.stopped_by_string = False

    def _route(self, text: str):
        r_delta, c_delta, calls = "", text, []
        if self.reasoning is not None:
            r_delta, c_delta = self.reasoning.push(text)
        if self.tools is not None and c_delta:
            c_delta, calls = self.tools.push(c_delta)
        return r_delta, c_delta, calls

    def feed(self, out):
        """StepOutput -> list of delta dicts (possibly empty)."""
        deltas = []
        self.cached = out.num_cached_tokens
        if out.new_token_ids and not self.stopped_by_string:
            self.completion_tokens += len(out.new_token_ids)
            text = self.decoder.push(out.new_token_ids)
            if out.logprobs and self.req.logprobs:
                for tok, (lp, rank, tops) in zip(out.new_token_ids, out.logprobs):
                    t = self.s.tokenizer.id_to_token(tok)
                    self.logprobs.append({
                        "token": t, "logprob": lp, "bytes": list(t.encode("utf-8", "replace")),
                        "top_logprobs": [{"token": self.s.tokenizer.id_to_token(i), "logprob": l,
                                          "bytes": list(self.s.tokenizer.id_to_token(i)
                                                        .encode("utf-8", "replace"))}
                                         for i, l in tops]})
            text, hit = self.stops.push(text)
            if hit:
                self.stopped_by_string = True
                self.finish = "stop"
                self.s.service.abort(self.rid)
            r, c, calls = self._route(text)
            d = {}
            if r:
                d["reasoning"] = r
                self.reason_text.append(r)
            if c:
                d["content"] = c
                self.content.append(c)
            if calls:
                d["tool_calls"] = calls
                self.calls.extend(calls)
            if d:
                deltas.append(d)
        if out.finished:
            tail = self.decoder.flush()
            if tail and not self.stopped_by_string:
                tail, _ = self.stops.push(tail)
                tail += self.stops.flush()
                r, c, calls = self._route(tail)
                if self.reasoning is not None:
                    fr, fc = self.reasoning.flush()
                    r += fr
                    c += fc
                if self.tools is not None:
                    c += self.tools.flush()
                d = {}
                if r:
                    d["reasoning"] = r
                    self.reason_text.append(r)
                if c:
                    d["content"] = c
                    self.content.append(c)
                if calls:
                    d["tool_calls"] = calls
                    self.calls.extend(calls)
                if d:
                    deltas.append(d)
            if self.finish is None:
                if out.finish_reason == FinishReason.LENGTH:
                    self.finish = "length"
                elif out.finish_reason == FinishReason.ERROR:
                    self.finish = "error"
                elif out.finish_reason == FinishReason.ABORT:
                    self.finish = "stop"
                else:
                    self.finish = "tool_calls" if self.calls else "stop"
        return deltas

    def usage(self):
        return {"prompt_tokens": self.prompt_len, "completion_tokens": self.completion_tokens,
                "total_tokens": self.prompt_len + self.completion_tokens,
                "prompt_tokens_details": {"cached_tokens": self.cached}}

    def chunk(self, delta: dict, finish=None, usage=None):
        c = {"id": self.rid, "object": "chat.completion.chunk", "created": self.created,
             "model": self.req.model,
             "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
        if self.req.logprobs and self.logprobs and delta:
            c["choices"][0]["logprobs"] = {"content": self.logprobs[-1:]}
        if usage is not None:
            c["usage"] = usage
        return c

    def response(self):
        msg = {"role": "assistant", "content": "".join(self.content) or None}
        if self.reason_text:
            msg["reasoning"] = "".join(self.reason_text)
        if self.calls:
            msg["tool_calls"] = [{k: v for k, v in c.items() if k != "index"} for c in self.calls]
        choice = {"index": 0, "message": msg, "finish_reason": self.finish}
        if self.req.logprobs:
            choice["logprobs"] = {"content": self.logprobs}
        return {"id": self.rid, "object": "chat.completion", "created": self.created,
                "model": self.req.model, "choices": [choice], "usage": self.usage()}


class AppState:
    pass


def create_app(*, package: Optional[Package] = None, engine=None, tokenizer=None,
               served_model_name: str = "model", video_service=None, generation_defaults=None,
               reasoning: bool = True, engine_factory=None, drafter=None,
               role: str = "mixed", internal_key: Optional[str] = None,
               engine_builder=None, state_dir: Optional[str] = None) -> FastAPI:
    """Builds the application.  ``engine`` (an LLMEngine) registers the chat route;
    ``video_service`` registers the video routes and ``/v1/capabilities``.  ``role`` =
    ``prefill`` / ``decode`` also mounts ``/internal/prefill`` / ``/internal/decode`` for a
    disaggregating router; those routes require ``internal_key`` (header
    ``x-uniserve-internal-key``) and exist on no other deployment.  ``engine_builder(package)``
    builds an engine for a changed package: with it, a change of effect ``epoch`` /
    ``generation`` / ``storage`` runs as an epoch update (prepare, switch, trial, commit or
    roll back; ``server/updates.py``) instead of being refused.  Control programs of the
    package (``server/control.py``) run once a second beside the server."""
    if role not in ("mixed", "prefill", "decode"):
        raise ConfigError("role", f"unknown role {role!r}")
    if role != "mixed" and not internal_key:
        raise ConfigError("role", "a prefill or decode replica needs an internal key "
                                  "(the router presents it on /internal/*)")
    app = FastAPI(title="uniserve-b200", docs_url=None, redoc_url=None, openapi_url=None)
    s = AppState()
    s.package = package or Package.parse(f'model = "local/{served_model_name}"\n')
    from . import images as _images
    _images.set_media_directory(s.package.media_config.directory)
    _images.set_media_limit(int(s.package.media_config.max_request_bytes))
    s.served = s.package.served_model_name or served_model_name
    s.tokenizer = tokenizer
    s.template = ChatTemplate(getattr(tokenizer, "chat_template", None)) if tokenizer else None
    s.obs = ObservationStore()
    s.engine = engine
    s.video = video_service
    s.reasoning = reasoning
    s.defaults = generation_defaults or getattr(tokenizer, "generation_config", {}) or {}
    s.inflight = 0
    s.started = time.time()
    s.service = None
    if engine is not None:
        sc = s.package.scheduler_config
        if drafter is None and s.package.speculative_config.num_draft_tokens > 0 and \
                hasattr(engine, "speculative_step") and \
                (hasattr(engine, "scheduler") or hasattr(engine, "states")):
            # `speculative_config.num_draft_tokens` without a drafter of the model's own:
            # prompt-lookup drafting (single-process engines; replicated engines step plainly)
            from ..engine.speculation import NgramDrafter
            drafter = NgramDrafter(k=int(s.package.speculative_config.num_draft_tokens))
        s.service = EngineService(engine, s.obs, sc.max_queued_requests,
                                  s.package.migration_config.max_migrations, engine_factory,
                                  drafter=drafter)
    app.state.s = s

    @app.on_event("startup")
    async def _start():
        if s.service:
            s.service.start()
        if s.video:
            s.video.start()
        oc = s.package.observation_config
        if oc.otlp_endpoint:                   # the store is pushed to an OTLP collector
            from .export import OtlpPusher
            s.otlp = OtlpPusher(s.obs, oc.otlp_endpoint, deployment=s.served,
                                period=max(1.0, float(oc.fine_bucket) * 10))
            s.otlp.start()
        blocks = getattr(s.engine, "blocks", None)
        if oc.kv_events and blocks is not None and blocks.kv_events is None:
            from .export import KvEventPublisher
            blocks.kv_events = KvEventPublisher(oc.kv_events, block_size=blocks.page_size)

    @app.on_event("shutdown")
    async def _stop():
        if s.service:
            s.service.stop(float(s.package.server_config.shutdown_timeout))
        if s.video:
            s.video.stop()
        if getattr(s, "otlp", None) is not None:
            s.otlp.stop()
        blocks = getattr(s.engine, "blocks", None)
        if blocks is not None and getattr(blocks, "kv_events", None) is not None:
            blocks.kv_events.close()

    # ------------------------------------------------------------ middleware --
    @app.middleware("http")
    async def gate(request: Request, call_next):
        t0 = time.monotonic()
        cfg = s.package.server_config
        rid = request.headers.get("x-request-id", "")
        if not rid or len(rid.encode()) > cfg.max_request_id:
            rid = uuid.uuid4().hex
        request.state.request_id = rid
        path = request.url.path
        if cfg.api_key and path != "/health":
            auth = request.headers.get("authorization", "")
            if auth != f"Bearer {cfg.api_key}":
                s.obs.inc("uniserve_http_requests_total", {"path": path, "status": "401"})
                return _err(401, "invalid or missing API key", "authentication_error")
        cl = request.headers.get("content-length")
        if cl and cl.isdigit() and int(cl) > cfg.max_request_body and not path.startswith("/v1/videos"):
            return _err(413, "request body too large")
        if cl and cl.isdigit() and path.startswith("/v1/videos") and \
                int(cl) > int(s.package.media_config.max_request_bytes):
            return _err(413, "request body too large")       # media routes: their own bound
        generating = path in ("/v1/chat/completions", "/v1/videos/sync")
        if generating and cfg.max_concurrent_requests is not None \
                and s.inflight >= cfg.max_concurrent_requests:
            s.obs.inc("uniserve_http_requests_total", {"path": path, "status": "503"})
            return _err(503, "too many concurrent requests", "overloaded",
                        headers={"Retry-After": str(max(1, int(cfg.retry_after)))})
        if generating:
            s.inflight += 1
        try:
            if cfg.request_timeout and not generating:
                resp = await asyncio.wait_for(call_next(request), float(cfg.request_timeout))
            else:
                resp = await call_next(request)
        except asyncio.TimeoutError:
            return _err(504, "request timed out", "timeout")
        finally:
            if generating:
                s.inflight -= 1
        if cfg.request_id_headers:
            resp.headers["X-Request-Id"] = rid
        s.obs.inc("uniserve_http_requests_total", {"path": path, "status": str(resp.status_code)})
        s.obs.observe("uniserve_http_request_seconds", time.monotonic() - t0, {"path": path})
        return resp

    @app.exception_handler(RequestValidationError)
    async def _bad(request, exc):
        e = exc.errors()[0]
        loc = ".".join(str(x) for x in e.get("loc", []) if x != "body")
        return _err(400, f"{loc}: {e.get('msg')}", param=loc or None)

    # ----------------------------------------------------------------- basics --
    @app.get("/health")
    async def health():
        ok = (s.service is None or (s.service.thread.is_alive() and not s.engine.failed))
        body = {"status": "ok" if ok else "failed", "uptime_seconds": time.time() - s.started,
                "pid": os.getpid(), "generation": int(getattr(app.state, "generation", 0)),
                "asleep": int(getattr(s.engine, "asleep", 0) or 0),
                "routes": sorted(r.path for r in app.routes if hasattr(r, "path"))}
        return JSONResponse(body, status_code=200 if ok else 503)

    @app.get("/version")
    async def version():
        import torch
        return {"version": VERSION, "torch": torch.__version__, "target": "sm_100a"}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": s.served, "object": "model",
                                            "created": int(s.started), "owned_by": "uniserve",
                                            "root": s.package.model or s.package.model_dir}]}

    @app.get("/metrics")
    async def metrics():
        return PlainTextResponse(s.obs.prometheus())

    # ------------------------------------------------------------------- chat --
    if engine is not None:
        def _internal_ok(request: Request) -> bool:
            import hmac
            got = request.headers.get("x-uniserve-internal-key", "")
            return hmac.compare_digest(got.encode(), internal_key.encode())

        if role == "prefill":
            @app.post("/internal/prefill")
            async def chat_prefill(request: Request):
                """Prefill role: the chat request runs to its first token; the answer is the
                request's framed state (``application/octet-stream``) for a decode replica, or
                the ordinary completion when the first token already ended it."""
                if not _internal_ok(request):
                    return _err(401, "invalid or missing internal key", "authentication_error")
                return await _chat(request, role="prefill")

        if role == "decode":
            @app.post("/internal/decode")
            async def chat_decode(request: Request):
                """Decode role: body {"request": <chat request>, "handoff": <base64 state>}.
                The state is the explicit frame of ``Handoff.to_bytes`` (a JSON header and raw
                tensor bytes); every field is checked against this engine before a page is
                written."""
                import base64
                from ..engine.handoff import handoffs_from_bytes
                if not _internal_ok(request):
                    return _err(401, "invalid or missing internal key", "authentication_error")
                try:
                    body = await request.json()
                    raw = base64.b64decode(body["handoff"], validate=True)
                    # one frame per rank of the lending deployment; this side re-cuts the KV
                    # heads for its own ranks
                    hs = handoffs_from_bytes(raw)
                    for h in hs:
                        h.validate_for(s.engine)
                    chat_body = body["request"]
                except Exception as e:
                    return _err(400, f"hand-off body: {e}")
                return await _chat(request, body=chat_body, handoff=(hs, raw))

        @app.post("/internal/probe")
        async def prefix_probe(request: Request):
            """How much of a chat request's prompt this replica already holds: the router of a
            replicated deployment asks every replica and sends the request where its prefix
            pages are (the cluster directory, asked instead of published).  Text requests
            only; nothing is allocated.  With an internal key configured the route needs it."""
            if internal_key and not _internal_ok(request):
                return _err(401, "invalid or missing internal key", "authentication_error")
            try:
                req = ChatCompletionRequest.model_validate(await request.json())
                msgs = [m.model_dump(exclude_none=True) for m in req.messages]
                tools = [t.model_dump(exclude_none=True) for t in req.tools] if req.tools else None
                prompt = s.template.render(msgs, tools, True, **(req.chat_template_kwargs or {}))
                ids = s.tokenizer.encode(prompt)
            except Exception as e:
                return _err(400, f"probe: {e}")
            salt = req.cache_salt or req.prompt_cache_key

            def look(e):
                blocks = getattr(e, "blocks", None)       # engines without a paged cache hold nothing
                # a look-up touches the cache's recency order: on a replicated (multi-rank)
                # engine only commands that every rank applies may do that
                if blocks is None or not hasattr(blocks, "peek_prefix") or hasattr(e, "bus"):
                    return 0
                return blocks.peek_prefix(blocks.page_keys(ids, salt)) * blocks.page_size
            cached = await asyncio.to_thread(s.service.call, look)
            return {"cached_tokens": int(cached), "prompt_tokens": len(ids),
                    "in_flight": s.inflight}

        @app.post("/v1/chat/completions")
        async def chat(request: Request):
            return await _chat(request)

        async def _chat(request: Request, role: Optional[str] = None, body=None, handoff=None):
            try:
                req = ChatCompletionRequest.model_validate(body if body is not None
                                                           else await request.json())
            except ValidationError as e:
                err = e.errors()[0]
                loc = ".".join(str(x) for x in err["loc"])
                return _err(400, f"{loc}: {err['msg']}", param=loc)
            except json.JSONDecodeError:
                return _err(400, "request body is not JSON")
            if req.model != s.served and req.model not in (s.package.adapters or {}):
                return _err(404, f"model {req.model!r} is not served", "not_found_error",
                            "model_not_found", "model")
            if s.package.paused:
                return _err(503, "the deployment is paused", "overloaded",
                            headers={"Retry-After": "1"})
            if req.tool_choice == "required" or isinstance(req.tool_choice, dict):
                return _err(400, "tool_choice 'required' and a named function need guided decoding, "
                                 "which this deployment does not serve", param="tool_choice")
            try:
                msgs = [m.model_dump(exclude_none=True) for m in req.messages]
                tools = [t.model_dump(exclude_none=True) for t in req.tools] if req.tools else None
                prompt = s.template.render(msgs, tools, True, **(req.chat_template_kwargs or {}))
            except Exception as e:
                return _err(400, f"chat template: {e}", param="messages")
            media = None
            from . import images as IM
            urls = IM.collect_media(msgs)
            if urls:
                mm = getattr(s.engine, "mm", None)
                if mm is None:
                    return _err(400, "this deployment does not take images", param="messages")
                vc = mm.tower.cfg

                def decode_media(prompt):
                    pre = []
                    for kind, u in urls:
                        if kind == "image":
                            pre.append(IM.preprocess(IM.load_image(u), vc.patch_size,
                                                     vc.temporal_patch_size, vc.spatial_merge_size))
                            continue
                        # a video is a run of timestamped images, one per temporal patch
                        frames, secs = IM.load_video(u)
                        rows, (gt, gh, gw) = IM.preprocess_video(
                            frames, vc.patch_size, vc.temporal_patch_size, vc.spatial_merge_size)
                        per = gh * gw
                        pre.extend((rows[i * per:(i + 1) * per], (1, gh, gw)) for i in range(gt))
                        prompt = prompt.replace("<|vision_start|><|video_pad|><|vision_end|>",
                                                IM.video_prompt(secs, vc.temporal_patch_size), 1)
                    return pre, prompt
                try:
                    # file reads and decoding leave the event loop
                    pre, prompt = await asyncio.to_thread(decode_media, prompt)
                except (ValueError, OSError) as e:
                    return _err(400, str(e), type_="input_error", param="messages")
                grids = [g for _, g in pre]
                img_tok = s.engine.model.cfg.image_token_id
                ids = []
                pieces = prompt.split("<|image_pad|>")
                for i, piece in enumerate(pieces):
                    ids.extend(s.tokenizer.encode(piece))
                    if i < len(pieces) - 1:
                        ids.append(img_tok)
                ids = IM.expand_placeholders(ids, img_tok, grids, vc.spatial_merge_size)
                import torch as _torch
                media = (_torch.cat([r for r, _ in pre]), grids)
            else:
                ids = s.tokenizer.encode(prompt)
            max_len = s.engine.config.max_model_len
            if len(ids) + 1 > max_len:
                return _err(400, f"the prompt has {len(ids)} tokens; the context holds {max_len}",
                            code="context_length_exceeded", param="messages")
            try:
                params = lower_sampling(req, s.tokenizer, s.defaults, max_len, len(ids),
                                        s.package.max_logprobs)
            except ValueError as e:
                return _err(400, str(e))
            try:
                rid, q = s.service.submit(ids, params, "chatcmpl-" + request.state.request_id,
                                          req.priority or 0, req.cache_salt or req.prompt_cache_key,
                                          lend=role == "prefill", handoff=handoff, media=media)
            except Overloaded as e:
                return _err(503, str(e), "overloaded", headers={"Retry-After": "1"})
            run = ChatRun(s, req, rid, len(ids))
            if role == "prefill":
                while True:
                    out = await q.get()
                    if out.handoff is not None:
                        return Response(out.handoff, media_type="application/octet-stream",
                                        headers={"x-uniserve-request-id": rid})
                    run.feed(out)
                    if out.finished:
                        if out.error:
                            return _err(500, out.error, "server_error")
                        return JSONResponse(run.response(), headers={"x-uniserve-finished": "1"})
            # tokens the lending engine already produced open the answer
            seeded = list(handoff[0][0].output_ids) if handoff is not None else []
            first = StepOutput(rid, seeded, False) if seeded else None

            if not req.stream:
                try:
                    if first is not None:
                        run.feed(first)
                    while True:
                        out = await q.get()
                        run.feed(out)
                        if out.finished:
                            if out.error:
                                return _err(500, out.error, "server_error")
                            break
                except asyncio.CancelledError:
                    s.service.abort(rid)
                    raise
                return JSONResponse(run.response())

            async def sse():
                keep = float(s.package.server_config.stream_keep_alive)
                yield "data: " + json.dumps(run.chunk({"role": "assistant", "content": ""})) + "\n\n"
                try:
                    if first is not None:
                        for d in run.feed(first):
                            yield "data: " + json.dumps(run.chunk(d)) + "\n\n"
                    while True:
                        try:
                            out = await asyncio.wait_for(q.get(), keep)
                        except asyncio.TimeoutError:
                            yield ": keep-alive\n\n"
                            continue
                        for d in run.feed(out):
                            yield "data: " + json.dumps(run.chunk(d)) + "\n\n"
                        if out.finished:
                            if out.error:
                                yield "data: " + json.dumps(openai_error(out.error, "server_error")) + "\n\n"
                            break
                    yield "data: " + json.dumps(run.chunk({}, run.finish)) + "\n\n"
                    if req.stream_options and req.stream_options.include_usage:
                        c = run.chunk({}, None, run.usage())
                        c["choices"] = []
                        yield "data: " + json.dumps(c) + "\n\n"
                    yield "data: [DONE]\n\n"
                except asyncio.CancelledError:
                    s.service.abort(rid)
                    raise

            return StreamingResponse(sse(), media_type="text/event-stream",
                                     headers={"Cache-Control": "no-cache"})

    # ------------------------------------------------------------------ video --
    if video_service is not None:
        from .video_rules import VideoRuleError, capabilities, plan_request

        @app.get("/v1/capabilities")
        async def caps():
            c = capabilities(video_service.sizes, video_service.max_seconds, video_service.steps)
            c["tasks"] = list(video_service.tasks)
            c["model"] = s.served
            return c

        async def _parse_video(request: Request):
            ctype = request.headers.get("content-type", "")
            if ctype.startswith("multipart/form-data"):
                # every field is a text part of its own name; file parts and repeated fields
                # are refused (media travel as URLs in ``input_references``)
                form = await request.form()
                data = {}
                for k, v in form.multi_items():
                    if not isinstance(v, str):
                        raise VideoRuleError(k, "file parts are not accepted: name media by URL "
                                                "in input_references")
                    if k in data:
                        raise VideoRuleError(k, "the field is repeated")
                    try:
                        data[k] = json.loads(v) if k in ("input_references", "extra_params") else v
                    except ValueError:
                        raise VideoRuleError(k, "not JSON")
                for k in ("num_frames", "fps", "seed", "num_inference_steps"):
                    if k in data:
                        data[k] = int(data[k])
            elif ctype.startswith("application/json") or not ctype:
                data = await request.json()
            else:
                raise _UnsupportedMedia(ctype)
            req = VideoGenerationRequest.model_validate(data)
            if req.model != s.served:
                raise LookupError(req.model)
            return req, plan_request(req, video_service.sizes, video_service.max_seconds,
                                     video_service.steps, served_tasks=video_service.tasks)

        def _video_error(e):
            if isinstance(e, _UnsupportedMedia):
                return _err(415, "use application/json or multipart/form-data")
            if isinstance(e, ValidationError):
                err = e.errors()[0]
                loc = ".".join(str(x) for x in err["loc"])
                return _err(400, f"{loc}: {err['msg']}", param=loc)
            if isinstance(e, VideoRuleError):
                return _err(400, f"{e.param}: {e}", param=e.param)
            if isinstance(e, LookupError):
                return _err(404, f"model {e.args[0]!r} is not served", "not_found_error",
                            "model_not_found", "model")
            return _err(400, str(e))

        @app.post("/v1/videos/sync")
        async def videos_sync(request: Request):
            try:
                req, plan = await _parse_video(request)
            except Exception as e:
                return _video_error(e)
            job = video_service.submit(req.prompt, plan)
            await job.wait()
            if job.state != "completed":
                if (job.error or "").startswith("input_error"):     # the request's own media
                    return _err(400, job.error, param="input_references")
                return _err(500, job.error or "generation failed", "server_error")
            return Response(job.content, media_type="video/mp4",
                            headers={"x-video-size": f"{plan.width}x{plan.height}",
                                     "x-video-num-frames": str(plan.num_frames),
                                     "x-video-fps": str(plan.fps),
                                     "x-video-seed": str(plan.seed)})

        @app.post("/v1/videos")
        async def videos_create(request: Request):
            try:
                req, plan = await _parse_video(request)
            except Exception as e:
                return _video_error(e)
            return JSONResponse(video_service.submit(req.prompt, plan).record(), status_code=200)

        @app.get("/v1/videos")
        async def videos_list():
            return {"object": "list", "data": [j.record() for j in video_service.jobs()]}

        @app.get("/v1/videos/{job_id}")
        async def videos_get(job_id: str):
            j = video_service.get(job_id)
            return j.record() if j else _err(404, "no such video job", "not_found_error")

        @app.get("/v1/videos/{job_id}/content")
        async def videos_content(job_id: str):
            j = video_service.get(job_id)
            if j is None:
                return _err(404, "no such video job", "not_found_error")
            if j.state != "completed":
                return _err(409, f"the job is {j.state}", "conflict")
            return Response(j.content, media_type="video/mp4")

        @app.delete("/v1/videos/{job_id}")
        async def videos_delete(job_id: str):
            return ({"id": job_id, "deleted": True} if video_service.delete(job_id)
                    else _err(404, "no such video job", "not_found_error"))

    # ------------------------------------------------------------------ admin --
    @app.get("/admin/policy")
    async def get_policy():
        from ..config.policy import dump_toml
        return {"config": s.package.raw, "layout": s.package.layout(),
                "revision": s.obs.revision, "toml": dump_toml(s.package.raw)}

    def apply_package(new: Package, writer: str = "admin"):
        """Applies a parsed package: in place for step / order effects, as an epoch update
        when an engine builder exists, refused otherwise.  Returns (status, body)."""
        changes = s.package.diff(new)
        eff = strongest_effect(changes)
        names = [c[0] for c in changes]
        if eff not in (None, "step", "order"):
            upd = getattr(s.service, "update", None) if s.service else None
            if engine_builder is None or s.service is None or eff == "daemon":
                return 409, openai_error(
                    f"the change needs effect `{eff}`, which a running process cannot apply "
                    f"in place: restart the deployment with the new package", "conflict",
                    None, changes[0][0] if changes else None)
            if upd is not None and not upd.done:
                return 409, openai_error(f"an update is {upd.phase}", "conflict")
            from .updates import EpochUpdate
            old = s.package
            uc = new.update_config

            def on_phase(phase, why):
                if phase == "switching":
                    s.package = new
                    s.served = new.served_model_name or s.served
                    s.obs.revision += 1
                elif phase in ("rolled_back", "abandoned"):
                    s.package = old
                s.obs.event("update", "", phase=phase, reason=why, writer=writer, changes=names)
                if phase == "switching":
                    s.engine = s.service.engine
            rb = uc.rollback
            upd = EpochUpdate(lambda: engine_builder(new), trial_s=float(uc.trial),
                              drain_s=float(uc.drain_s), failure_rate=rb.failure_rate,
                              step_time_regression=rb.step_time_regression,
                              throughput_regression=rb.throughput_regression, on_phase=on_phase)
            s.service.begin_update(upd)
            return 202, {"applied": names, "effect": eff, "update": upd.phase}
        s.package = new
        s.served = new.served_model_name or s.served
        if s.service:
            s.service.paused = bool(new.paused)
            s.service.wake.set()
            if s.engine is not None and hasattr(s.engine, "blocks"):
                s.engine.blocks.enable_prefix_cache = bool(new.kv_cache_config.prefix_caching)
                if any(c[0] == "flush" for c in changes):
                    s.engine.blocks.flush()
                cps = new.scheduler_config.chunked_prefill_size
                if cps and hasattr(s.engine, "config"):
                    s.engine.config.chunked_prefill_size = int(cps)
        s.obs.revision += 1
        s.obs.event("policy", "", changes=names, effect=eff, writer=writer)
        return 200, {"applied": names, "effect": eff, "revision": s.obs.revision}

    s.apply_package = apply_package

    @app.put("/admin/policy")
    async def put_policy(request: Request):
        text = (await request.body()).decode()
        try:
            new = Package.parse(text)
        except ConfigError as e:
            return _err(400, str(e), param=e.path)
        status, body = apply_package(new)
        return JSONResponse(body, status_code=status)

    @app.post("/admin/restart")
    async def admin_restart():
        """Hot restart: a successor process takes the listening socket over; this one finishes
        the requests it took and exits (single-process deployments started by `serve`)."""
        hr = getattr(app.state, "restart", None)
        if hr is None:
            return _err(409, "this deployment cannot hand its listener over (several ranks, a "
                             "unix socket, or not started by `serve`)")
        out = await asyncio.to_thread(hr.begin)
        s.obs.event("restart", **{k: v for k, v in out.items() if v is not None})
        return JSONResponse(out, status_code=202)

    @app.get("/admin/ranks")
    async def admin_ranks():
        sup = getattr(app.state, "supervision", None)
        return sup.status() if sup is not None else {"ranks": [], "failed": None}

    @app.get("/admin/quota")
    async def admin_quota():
        """The devices' quota ledgers: limit, usage and every engine's reservations by item
        (weights, cache segment, graph pool), with refusals counted."""
        from ..engine.quota import all_reports
        return {"devices": all_reports()}

    @app.get("/admin/standby")
    async def admin_standby():
        sb = getattr(app.state, "standby", None)
        return sb.status() if sb is not None else {"state": "none"}

    @app.get("/admin/restart")
    async def admin_restart_status():
        hr = getattr(app.state, "restart", None)
        return hr.status() if hr is not None else {"state": None}

    @app.get("/admin/profile")
    async def get_profile():
        """State of the engine's profile session and its always-on counters."""
        if s.service is None:
            return _err(409, "this deployment has no engine")
        prof = getattr(s.engine, "profiler", None)
        return prof.state() if prof is not None else {"open": False}

    @app.post("/admin/profile")
    async def post_profile(request: Request):
        """Opens a profile session: ``{"collectors": ["fence_timeline", "timeline"], "steps": n,
        "seconds": t, "output": path}``; it closes itself after ``steps`` engine steps or
        ``seconds``.  ``{"close": true}`` ends the open session."""
        if s.service is None:
            return _err(409, "this deployment has no engine")
        if hasattr(s.engine, "bus"):
            return _err(409, "a multi-rank deployment runs its ranks in lock step: a session on "
                             "the leader alone would change its step sequence")
        try:
            body = await request.json()
        except Exception:
            body = {}
        from ..engine.profiling import start_session

        def act(e):
            if body.get("close"):
                if getattr(e, "profiler", None) is not None:
                    e.profiler.close()
                    return e.profiler.state()
                return {"open": False}
            return start_session(e, body.get("collectors") or ["fence_timeline"],
                                 body.get("output"), steps=body.get("steps"),
                                 seconds=body.get("seconds"),
                                 rank=getattr(getattr(e.model, "ctx", None), "rank", 0))
        try:
            out = await asyncio.to_thread(s.service.call, act)
        except ValueError as ex:
            return _err(400, str(ex), param="collectors")
        s.obs.event("profile", **{k: v for k, v in out.items() if k in ("open", "path")})
        return out

    @app.post("/admin/prefix_cache")
    async def admin_prefix_cache(request: Request):
        """``{"action": "save" | "load", "path": FILE}``: writes the cached KV pages to a file
        or reads such a file into the cache (a restart by hand keeps its prefixes)."""
        if s.service is None or not hasattr(s.engine, "blocks"):
            return _err(409, "this deployment has no paged engine")
        if hasattr(s.engine, "bus"):
            return _err(409, "a multi-rank deployment keeps its ranks' caches in step: its "
                             "prefix cache is not written or read from outside")
        try:
            body = await request.json()
            action, path = body["action"], str(body["path"])
        except Exception:
            return _err(400, 'body: {"action": "save" | "load", "path": FILE}')
        from ..engine.prefix_store import load_prefix_cache, save_prefix_cache
        if action == "save":
            fn = lambda e: save_prefix_cache(e, path, int(body.get("max_bytes", 1 << 30)))
        elif action == "load":
            fn = lambda e: load_prefix_cache(e, path, remove=bool(body.get("remove", False)))
        else:
            return _err(400, "action is save or load", param="action")
        try:
            out = await asyncio.to_thread(s.service.call, fn)
        except OSError as e:
            return _err(400, str(e), param="path")
        s.obs.event("prefix_cache", action=action, pages=out.get("pages", 0))
        return out

    @app.post("/admin/sleep")
    async def admin_sleep(level: int = 1):
        """Frees the KV cache and graphs (level 1) and the weights too (level 2); requests in
        flight recompute after ``/admin/wake``, new ones queue meanwhile."""
        if s.service is None or not hasattr(s.engine, "sleep"):
            return _err(409, "this deployment has no engine that can sleep")
        if level not in (1, 2):
            return _err(400, "level is 1 or 2", param="level")
        out = await asyncio.to_thread(s.service.call, lambda e: e.sleep(level))
        s.obs.event("sleep", **out)
        return out

    @app.post("/admin/wake")
    async def admin_wake():
        if s.service is None or not hasattr(s.engine, "wake"):
            return _err(409, "this deployment has no engine that can sleep")
        out = await asyncio.to_thread(s.service.call, lambda e: e.wake())
        s.service.wake.set()
        s.obs.event("wake", **out)
        return out

    @app.get("/admin/update")
    async def get_update():
        upd = getattr(s.service, "update", None) if s.service else None
        if upd is None:
            return {"phase": None}
        return {"phase": upd.phase, "reason": upd.reason, "history": upd.history}

    # control programs of the package: read the store, write options through apply_package
    from .control import ControlLoop

    def _apply_options(changes: dict) -> bool:
        try:
            new = s.package.with_options(changes)
        except ConfigError:
            return False
        status, _ = apply_package(new, writer="program")
        return status in (200, 202)
    s.control = ControlLoop(lambda: s.package, s.obs, _apply_options, state_dir)

    @app.on_event("startup")
    async def _start_control():
        if not s.control.hosts:
            return

        async def loop():
            while True:
                await asyncio.sleep(1.0)
                try:
                    await asyncio.to_thread(s.control.tick)
                except Exception:
                    pass
        s.control_task = asyncio.create_task(loop())

    @app.api_route("/admin/query", methods=["GET", "POST"])
    async def query(request: Request):
        q = request.query_params.get("q")
        if q is None and request.method == "POST":
            q = (await request.body()).decode()
        if not q:
            return _err(400, "state the SQL as ?q= or as the request body")
        try:
            return s.obs.query(q)
        except Exception as e:
            return _err(400, str(e))

    return app
