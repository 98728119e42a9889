"""HTTP API: OpenAI chat completions (streaming SSE and non-streaming), models, health, stats, console snapshot,
and the Anthropic Messages surface (`/v1/messages`, `/v1/messages/count_tokens`) mapped onto the same scheduler.

The HTTP handlers never touch the model: they tokenise, build a `Request`, hand it to the serving thread through
`ServingLoop.submit` and stream what the scheduler emits.  `/health` reports unavailable as soon as the wire or
the scheduler thread has failed (reference: cuteafd-api/src/openai.rs:308-353 routes, :241-265 NativeRequest,
openai/health.rs, gateway/anthropic.rs:25-26).
"""
import asyncio
import json
import queue
import threading
import time
import uuid

from ..loader.tokenizer import StreamDecoder, load_tokenizer
from ..ref.sampler import SamplingParams
from .scheduler import Request, Scheduler

KEEPALIVE_S = 15.0


def render_chat(messages, system=None) -> str:
    """Minimal role-tagged prompt rendering (model-specific chat templates plug in here)."""
    parts = []
    if system:
        parts.append(f"<|system|>\n{system}\n")
    for m in messages:
        content = m.get("content")
        if isinstance(content, list):
            content = "".join(p.get("text", "") for p in content if isinstance(p, dict))
        parts.append(f"<|{m.get('role', 'user')}|>\n{content}\n")
    parts.append("<|assistant|>\n")
    return "".join(parts)


class ServingLoop:
    """Owns the scheduler on one thread; HTTP tasks talk to it through thread-safe queues."""

    def __init__(self, scheduler: Scheduler, health=None):
        self.sched, self.health = scheduler, health
        self.inbox: queue.Queue = queue.Queue(maxsize=64)
        self.cancels: queue.Queue = queue.Queue()
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.stop_flag = False
        self.died = None
        self.started = time.time()

    def start(self):
        self.thread.start()
        return self

    def stop(self):
        self.stop_flag = True
        self.thread.join(timeout=5)

    def submit(self, req: Request) -> bool:
        if self.died or self.sched.fatal:
            return False
        try:
            self.inbox.put_nowait(req)
            return True
        except queue.Full:
            return False

    def cancel(self, rid: str):
        self.cancels.put(rid)

    def _run(self):
        try:
            while not self.stop_flag:
                moved = False
                while True:
                    try:
                        self.sched.submit(self.inbox.get_nowait())
                        moved = True
                    except queue.Empty:
                        break
                while True:
                    try:
                        self.sched.cancel(self.cancels.get_nowait())
                    except queue.Empty:
                        break
                if self.health is not None and not self.health.live and not self.sched.fatal:
                    self.sched.fail_all(self.health.cause)
                if not self.sched.step() and not moved:
                    time.sleep(0.001)
        except Exception as e:      # the scheduler thread dying takes the server to unavailable, clients are told
            self.died = f"scheduler thread: {e}"
            self.sched.fail_all(self.died)

    def healthy(self) -> bool:
        return self.died is None and not self.sched.fatal and (self.health is None or self.health.live)


try:        # imported at module level so FastAPI can resolve the handlers' parameter annotations
    from fastapi import FastAPI, Header, HTTPException, Request as HttpRequest
    from fastapi.responses import JSONResponse, StreamingResponse
except ImportError:      # pragma: no cover - the HTTP layer is optional
    FastAPI = None


def build_app(loop: ServingLoop, *, model_id: str = "cuteafd-b200", tokenizer=None, api_keys=None, max_output: int = 4096):
    if FastAPI is None:
        raise RuntimeError("fastapi is not installed")

    tok = tokenizer or load_tokenizer(None)
    app = FastAPI(title="cuteafd-b200")

    def auth(authorization, x_api_key=None):
        if not api_keys:
            return
        key = (authorization or "").removeprefix("Bearer ").strip() or (x_api_key or "")
        if key not in api_keys:
            raise HTTPException(401, "invalid API key")

    def sampling_from(body: dict) -> SamplingParams:
        try:
            return SamplingParams(temperature=float(body.get("temperature", 0.0) or 0.0), top_p=float(body.get("top_p", 1.0) or 1.0),
                                  top_k=int(body.get("top_k", 0) or 0), min_p=float(body.get("min_p", 0.0) or 0.0),
                                  seed=int(body.get("seed", 0) or 0)).validate()
        except ValueError as e:
            raise HTTPException(400, str(e))

    def start_generation(prompt_ids, body, max_tokens):
        if not loop.healthy():
            raise HTTPException(503, loop.died or loop.sched.fatal or "unavailable")
        events: asyncio.Queue = asyncio.Queue()
        aloop = asyncio.get_running_loop()
        rid = uuid.uuid4().hex[:16]

        def on_token(toks, done, reason):
            aloop.call_soon_threadsafe(events.put_nowait, (toks, done, reason))
        req = Request(rid, prompt_ids, max_tokens=max(1, min(max_tokens, max_output)), sampling=sampling_from(body),
                      eos_id=getattr(tok, "eos_id", None), on_token=on_token)
        if not loop.submit(req):
            raise HTTPException(429, "admission queue is full")
        return rid, events

    @app.get("/health")
    async def health():
        ok = loop.healthy()
        return JSONResponse({"status": "ok" if ok else "unavailable", "cause": loop.died or loop.sched.fatal}, status_code=200 if ok else 503)

    @app.get("/v1/models")
    async def models(authorization: str = Header(None)):
        auth(authorization)
        return {"object": "list", "data": [{"id": model_id, "object": "model", "owned_by": "cuteafd-b200"}]}

    @app.get("/v1/stats")
    async def stats():
        return dict(loop.sched.snapshot(), uptime_s=round(time.time() - loop.started, 1), healthy=loop.healthy())

    @app.get("/v1/console/snapshot")
    async def console():
        s = loop.sched
        return {"lanes": [{"rid": a.req.rid, "prompt": len(a.req.prompt), "prefilled": a.prefilled, "generated": len(a.out),
                           "cache_hit": a.cache_hit} for a in s.active], "queue": len(s.queue), "stats": s.snapshot()}

    @app.post("/v1/chat/completions")
    async def chat(http: HttpRequest, authorization: str = Header(None)):
        auth(authorization)
        body = await http.json()
        msgs = body.get("messages")
        if not isinstance(msgs, list) or not msgs:
            raise HTTPException(400, "messages must be a non-empty list")
        prompt_ids = tok.encode(render_chat(msgs))
        max_tokens = int(body.get("max_completion_tokens") or body.get("max_tokens") or 256)
        rid, events = start_generation(prompt_ids, body, max_tokens)
        created, cid = int(time.time()), "chatcmpl-" + rid

        async def gather():
            ids, reason = [], None
            while True:
                toks, done, reason = await events.get()
                ids += toks
                if done:
                    return ids, reason
        if not body.get("stream"):
            ids, reason = await gather()
            if reason and reason.startswith(("error", "unavailable")):
                raise HTTPException(503 if "unavailable" in reason or "transport" in reason else 500, reason)
            return {"id": cid, "object": "chat.completion", "created": created, "model": model_id,
                    "choices": [{"index": 0, "message": {"role": "assistant", "content": tok.decode(ids)}, "finish_reason": reason}],
                    "usage": {"prompt_tokens": len(prompt_ids), "completion_tokens": len(ids), "total_tokens": len(prompt_ids) + len(ids)}}

        async def sse():
            dec = StreamDecoder(tok)
            def chunk(delta, finish=None):
                return "data: " + json.dumps({"id": cid, "object": "chat.completion.chunk", "created": created, "model": model_id,
                                              "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}) + "\n\n"
            yield chunk({"role": "assistant"})
            try:
                while True:
                    try:
                        toks, done, reason = await asyncio.wait_for(events.get(), KEEPALIVE_S)
                    except asyncio.TimeoutError:
                        yield ": keepalive\n\n"
                        continue
                    text = dec.push(toks) if toks else ""
                    if text:
                        yield chunk({"content": text})
                    if done:
                        yield chunk({}, reason)
                        yield "data: [DONE]\n\n"
                        return
            finally:
                loop.cancel(rid)
        return StreamingResponse(sse(), media_type="text/event-stream")

    @app.post("/v1/messages/count_tokens")
    async def count_tokens(http: HttpRequest, authorization: str = Header(None), x_api_key: str = Header(None)):
        auth(authorization, x_api_key)
        body = await http.json()
        return {"input_tokens": len(tok.encode(render_chat(body.get("messages", []), body.get("system"))))}

    @app.post("/v1/messages")
    async def messages(http: HttpRequest, authorization: str = Header(None), x_api_key: str = Header(None)):
        auth(authorization, x_api_key)
        body = await http.json()
        if "max_tokens" not in body:
            raise HTTPException(400, "max_tokens is required")
        prompt_ids = tok.encode(render_chat(body.get("messages", []), body.get("system") if isinstance(body.get("system"), str) else None))
        rid, events = start_generation(prompt_ids, body, int(body["max_tokens"]))
        ids, reason = [], None
        while True:
            toks, done, reason = await events.get()
            ids += toks
            if done:
                break
        if reason and reason.startswith(("error", "unavailable")):
            raise HTTPException(503, reason)
        return {"id": "msg_" + rid, "type": "message", "role": "assistant", "model": model_id,
                "content": [{"type": "text", "text": tok.decode(ids)}], "stop_reason": "end_turn" if reason == "stop" else "max_tokens",
                "usage": {"input_tokens": len(prompt_ids), "output_tokens": len(ids)}}

    return app
