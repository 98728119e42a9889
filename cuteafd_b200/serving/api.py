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
from .chat_templates import ChatTemplate, parse_completion, template_for
from .constraints import ChoiceConstraint, constraint_from_request, tool_choice_constraint
from .scheduler import Request, Scheduler

KEEPALIVE_S = 15.0


def render_chat(messages, system=None) -> str:
    """Role-tagged prompt of the plain template (models without a chat template, byte tokenizer)."""
    return ChatTemplate().render(messages, system=system)


def _anthropic_to_openai(body: dict) -> tuple[list, list]:
    """Anthropic Messages content blocks -> OpenAI-style messages and tool specs (gateway/anthropic.rs mapping)."""
    msgs = []
    for m in body.get("messages", []):
        content = m.get("content")
        if not isinstance(content, list):
            msgs.append({"role": m.get("role", "user"), "content": content})
            continue
        text, calls, images = [], [], False
        for b in content:
            kind = b.get("type")
            if kind == "text":
                text.append(b.get("text", ""))
            elif kind == "image":                   # stays a content part: the vision front end takes it out of the prompt
                text.append(b)
                images = True
            elif kind == "tool_use":
                calls.append({"id": b.get("id"), "function": {"name": b.get("name"), "arguments": b.get("input", {})}})
            elif kind == "tool_result":
                inner = b.get("content")
                if isinstance(inner, list):
                    inner = "".join(x.get("text", "") for x in inner if isinstance(x, dict))
                msgs.append({"role": "tool", "tool_call_id": b.get("tool_use_id"), "content": inner or ""})
        if text or calls:
            msg = {"role": m.get("role", "user"),
                   "content": [x if isinstance(x, dict) else {"type": "text", "text": x} for x in text] if images else "".join(text)}
            if calls:
                msg["tool_calls"] = calls
            msgs.append(msg)
    tools = [{"type": "function", "function": {"name": t.get("name"), "description": t.get("description", ""),
                                               "parameters": t.get("input_schema") or {"type": "object", "properties": {}}}}
             for t in body.get("tools") or [] if t.get("name")]
    return msgs, tools


def _cut_at_stop(text: str, stops) -> tuple[str, bool]:
    cut = min((i for i in (text.find(s) for s in stops if s) if i >= 0), default=-1)
    return (text[:cut], True) if cut >= 0 else (text, False)


DASHBOARD_HTML = """<!doctype html><meta charset=utf-8><title>cuteafd-b200 console</title>
<style>body{font:13px ui-monospace,monospace;margin:1.5em;background:#111;color:#ddd}h1{font-size:15px}table{border-collapse:collapse}
td,th{padding:2px 10px;text-align:right;border-bottom:1px solid #333}th{color:#8bf}#ev{white-space:pre;color:#9c9;max-height:16em;overflow:auto}
.bar{display:inline-block;height:9px;background:#4a8}</style>
<h1>cuteafd-b200 console</h1><div id=top></div><h1>lanes</h1><table id=lanes></table><h1>draft acceptance by position</h1><div id=acc></div>
<h1>recent requests</h1><table id=recent></table><h1>events</h1><div id=ev></div>
<script>
const row=(cells,tag='td')=>'<tr>'+cells.map(c=>`<${tag}>${c}</${tag}>`).join('')+'</tr>';
async function tick(){try{const s=await (await fetch('/v1/console/snapshot')).json(),st=s.stats;
top.textContent=`active ${st.active}  queued ${st.queued}  generated ${st.generated}  steps ${st.steps}  prefix hits ${st.prefix?st.prefix.hits:'-'}  free pages ${st.free_pages}  graphs ${st.graphs?st.graphs.captures:'-'}`;
lanes.innerHTML=row(['request','prompt','prefilled','generated','cache hit'],'th')+s.lanes.map(l=>row([l.rid,l.prompt,l.prefilled,l.generated,l.cache_hit])).join('');
acc.innerHTML=(st.draft_acceptance_by_position||[]).map((a,i)=>a==null?'':`#${i+1} <span class=bar style="width:${Math.round(a*200)}px"></span> ${(a*100).toFixed(0)}%<br>`).join('');
recent.innerHTML=row(['request','prompt','generated','cache hit','finish'],'th')+s.recent.slice().reverse().map(r=>row([r.rid,r.prompt,r.generated,r.cache_hit,r.reason])).join('');
}catch(e){top.textContent='unreachable: '+e}}
setInterval(tick,1000);tick();
const es=new EventSource('/v1/console/events');es.onmessage=m=>{ev.textContent=(m.data+'\n'+ev.textContent).slice(0,6000)};
</script>"""


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


def build_app(loop: ServingLoop, *, model_id: str = "cuteafd-b200", tokenizer=None, api_keys=None, max_output: int = 4096, template=None,
              usage=None, enable_bench: bool = False, thermal=None, gateway: bool = True, model_aliases: dict | None = None,
              allow_origin: str | None = None, search=None, record_path: str | None = None, vision=None):
    """`usage`: a `UsageStore` that gets one row per finished request and backs `/usage`.  `enable_bench` turns on the
    probe header `x-cuteafd-probe` (JSON: `skip_cache`, `no_drafts`, `token_ids`) that benchmarks use to pin what a
    request exercises (cuteafd-api/src/openai/probe.rs).  `thermal`: object with `.sample()` for `/v1/thermal`.
    `gateway` adds the surfaces other clients speak, mapped onto the same scheduler: Anthropic Messages and OpenAI
    Responses (`/v1/responses`, stored responses with `previous_response_id` chaining); `model_aliases` lists
    official model names that clients may ask for and that are answered by the served model (gateway/models.rs).  `search`: a
    provider for `/v1/alpha/search` (see `gateway_extras.SearchProvider`); `record_path`: every request / response pair of the
    JSON endpoints is appended to this JSONL file (`gateway_extras.replay` plays such a file back).  `vision`: a
    `serving.vision.VisionFrontEnd`; with it image content parts (OpenAI `image_url` / `input_image`, Anthropic `image`) are encoded by
    the tower and take the place of placeholder tokens in the prompt; without it they are refused."""
    if FastAPI is None:
        raise RuntimeError("fastapi is not installed")

    tok = tokenizer or load_tokenizer(None)
    tmpl = template or template_for(model_id)
    vocab_size = getattr(tok, "vocab_size", None)
    app = FastAPI(title="cuteafd-b200")

    def chat_options(body: dict):
        """(thinking, stop strings) of a request."""
        kw = body.get("chat_template_kwargs") or {}
        thinking = bool(kw.get("enable_thinking", kw.get("thinking", False)) or (body.get("thinking") or {}).get("type") == "enabled")
        stop = body.get("stop") or body.get("stop_sequences") or []
        stop = [stop] if isinstance(stop, str) else [x for x in stop if isinstance(x, str)]
        return thinking, list(tmpl.stop_strings) + stop

    def constraint_for(body: dict, prompt_len: int):
        if vocab_size is None:
            return None
        eos = getattr(tok, "eos_id", None)
        try:
            c = constraint_from_request(body, tok, vocab_size, prompt_len, eos)
        except ValueError as e:          # a grammar or pattern that does not compile is the client's error
            raise HTTPException(400, f"invalid response format: {e}") from None
        if c is None and isinstance(body.get("guided_choice"), list):
            c = ChoiceConstraint(tok, vocab_size, prompt_len, [str(x) for x in body["guided_choice"]], eos)
        if c is None and body.get("tools") and body.get("tool_choice") not in (None, "auto", "none"):
            c = tool_choice_constraint(body, tmpl, tok, vocab_size, prompt_len, eos)      # "required" / a named function
        return c

    def auth(authorization, x_api_key=None):
        if not api_keys:
            return
        key = (authorization or "").removeprefix("Bearer ").strip() or (x_api_key or "")
        if key not in api_keys:
            raise HTTPException(401, "invalid API key")
        return key

    def sampling_from(body: dict) -> SamplingParams:
        try:
            return SamplingParams(temperature=float(body.get("temperature", 0.0) or 0.0), top_p=float(body.get("top_p", 1.0) or 1.0),
                                  top_k=int(body.get("top_k", 0) or 0), min_p=float(body.get("min_p", 0.0) or 0.0),
                                  seed=int(body.get("seed", 0) or 0)).validate()
        except ValueError as e:
            raise HTTPException(400, str(e))

    gen_meta: dict = {}

    def key_of(authorization, x_api_key=None):
        k = (authorization or "").removeprefix("Bearer ").strip() or (x_api_key or "")
        return (k[:6] + "...") if k else "-"

    def account(rid, key, t0, t_first, n_prompt, n_out, finish):
        if usage is None:
            return
        now = time.time()
        hit = gen_meta.pop(rid, {}).get("hit", 0)
        usage.record(rid, model_id, key, n_prompt, n_out, hit, ((t_first or now) - t0) * 1e3, (now - t0) * 1e3, finish or "")

    def probe_of(http) -> dict:
        if not enable_bench:
            return {}
        try:
            d = json.loads(http.headers.get("x-cuteafd-probe") or "{}")
            return d if isinstance(d, dict) else {}
        except json.JSONDecodeError:
            raise HTTPException(400, "x-cuteafd-probe is not JSON")

    async def build_prompt(msgs, **render_kw):
        """(prompt ids, image rows of the request or None)."""
        image_kinds = ("image_url", "input_image", "image", "input_audio")
        has_image = any(isinstance(m, dict) and isinstance(m.get("content"), list)
                        and any(isinstance(p, dict) and p.get("type") in image_kinds for p in m["content"]) for m in msgs)
        if not has_image:
            return tok.encode(tmpl.render(msgs, **render_kw)), None
        if vision is None:
            raise HTTPException(400, "this server has no vision tower: image / audio inputs are not accepted")
        try:
            return await asyncio.to_thread(vision.prepare, msgs, lambda m: tmpl.render(m, **render_kw), tok.encode)
        except (ValueError, OSError) as e:          # undecodable image, too many images, remote URL
            raise HTTPException(400, f"invalid image / audio input: {e}") from None

    def start_generation(prompt_ids, body, max_tokens, constraint=None, probe=None, embeds=None):
        if not loop.healthy():
            raise HTTPException(503, loop.died or loop.sched.fatal or "unavailable")
        events: asyncio.Queue = asyncio.Queue()
        aloop = asyncio.get_running_loop()
        rid = uuid.uuid4().hex[:16]

        meta = gen_meta[rid] = {}

        def on_token(toks, done, reason):
            if "hit" not in meta:        # runs on the scheduler thread while the request is still active
                meta["hit"] = next((a.cache_hit for a in loop.sched.active if a.req.rid == rid), 0)
            aloop.call_soon_threadsafe(events.put_nowait, (toks, done, reason))
        req = Request(rid, prompt_ids, max_tokens=max(1, min(max_tokens, max_output)), sampling=sampling_from(body),
                      eos_id=getattr(tok, "eos_id", None), stop_ids=tuple(getattr(tok, "stop_ids", ()) or ()), on_token=on_token,
                      constraint=constraint, embeds=embeds,
                      use_cache=embeds is None and not (probe or {}).get("skip_cache", False), allow_drafts=not (probe or {}).get("no_drafts", False))
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
        names = [model_id] + [n for n in (model_aliases or {}) if n != model_id]
        return {"object": "list", "data": [{"id": n, "object": "model", "owned_by": "cuteafd-b200"} for n in names]}

    @app.get("/v1/stats")
    async def stats():
        return dict(loop.sched.snapshot(), uptime_s=round(time.time() - loop.started, 1), healthy=loop.healthy())

    @app.get("/v1/thermal")
    async def thermal_ep():
        if thermal is None:
            return {"available": False}
        s = thermal.sample()
        if hasattr(thermal, "report"):          # window summaries: was the last minute / ten minutes / two hours throttled, and why
            now = time.time()
            s["windows"] = {f"{w}s": thermal.report.window(now - w) for w in (60, 600, 7200)}
        return s

    @app.get("/v1/fabric")
    async def fabric_ep():
        from ..utils.thermal import fabric_snapshot
        return fabric_snapshot()

    @app.get("/usage")
    async def usage_ep(authorization: str = Header(None)):
        auth(authorization)
        if usage is None:
            raise HTTPException(404, "usage accounting is off")
        return {"totals": usage.totals(), "daily": usage.daily(), "by_key": usage.by_key()}

    @app.get("/v1/console/snapshot")
    async def console():
        s = loop.sched
        return {"lanes": [{"rid": a.req.rid, "prompt": len(a.req.prompt), "prefilled": a.prefilled, "generated": len(a.out),
                           "cache_hit": a.cache_hit} for a in list(s.active)], "queue": len(s.queue), "stats": s.snapshot(),
                "recent": list(getattr(s, "recent", []))}

    @app.get("/v1/console/events")
    async def console_events(http: HttpRequest):
        """Server-sent stream of scheduler events (decode rounds, finished requests); the scheduler only records events
        while at least one viewer is connected."""
        s = loop.sched

        async def stream():
            s.watchers += 1
            last = None
            try:
                yield "retry: 2000\n\n"
                while not await http.is_disconnected():
                    evs = list(s.events)
                    start = 0
                    if last is not None:
                        for i in range(len(evs) - 1, -1, -1):
                            if evs[i] is last:
                                start = i + 1
                                break
                    for e in evs[start:]:
                        yield "data: " + json.dumps(e) + "\n\n"
                    if evs:
                        last = evs[-1]
                    await asyncio.sleep(0.25)
            finally:
                s.watchers -= 1
        return StreamingResponse(stream(), media_type="text/event-stream")

    @app.get("/")
    async def dashboard():
        from fastapi.responses import HTMLResponse
        return HTMLResponse(DASHBOARD_HTML)

    def openai_calls(calls):
        return [{"id": c["id"], "type": "function", "function": {"name": c["name"], "arguments": json.dumps(c["arguments"], ensure_ascii=False)}}
                for c in calls]

    async def collect(events):
        ids, reason = [], None
        while True:
            toks, done, reason = await events.get()
            ids += toks
            if done:
                return ids, reason

    @app.post("/v1/chat/completions")
    async def chat(http: HttpRequest, authorization: str = Header(None)):
        auth(authorization)
        body = await http.json()
        msgs = body.get("messages")
        if not isinstance(msgs, list) or not msgs:
            raise HTTPException(400, "messages must be a non-empty list")
        thinking, stops = chat_options(body)
        tools = body.get("tools") if body.get("tool_choice") != "none" else None
        probe = probe_of(http)
        ids_given = probe.get("token_ids")
        if isinstance(ids_given, list) and ids_given:
            prompt_ids, embeds = [int(x) for x in ids_given], None
        else:
            prompt_ids, embeds = await build_prompt(msgs, tools=tools, thinking=thinking)
        max_tokens = int(body.get("max_completion_tokens") or body.get("max_tokens") or 256)
        t0, key = time.time(), key_of(authorization)
        rid, events = start_generation(prompt_ids, body, max_tokens, constraint_for(body, len(prompt_ids)), probe, embeds)
        created, cid = int(time.time()), "chatcmpl-" + rid

        if not body.get("stream"):
            ids, reason = await collect(events)
            if reason and reason.startswith(("error", "unavailable", "busy", "queue full")):
                raise HTTPException(429 if reason.startswith(("busy", "queue full")) else (503 if "unavailable" in reason or "transport" in reason else 500), reason)
            text, stopped = _cut_at_stop(tok.decode(ids), stops)
            parsed = parse_completion(tmpl, text, thinking)
            account(rid, key, t0, None, len(prompt_ids), len(ids), reason)
            message = {"role": "assistant", "content": parsed["content"]}
            if parsed["reasoning"]:
                message["reasoning_content"] = parsed["reasoning"]
            if parsed["tool_calls"]:
                message["tool_calls"] = openai_calls(parsed["tool_calls"])
            finish = "tool_calls" if parsed["tool_calls"] else ("stop" if stopped else reason)
            return {"id": cid, "object": "chat.completion", "created": created, "model": served_name(body),
                    "choices": [{"index": 0, "message": message, "finish_reason": finish}],
                    "usage": {"prompt_tokens": len(prompt_ids), "completion_tokens": len(ids), "total_tokens": len(prompt_ids) + len(ids)}}

        async def sse():
            dec, parser = StreamDecoder(tok), tmpl.parser(thinking)
            held, n_calls, n_out, t_first = "", 0, 0, None
            hold = max((len(x) for x in stops), default=1) - 1         # text that may still become a stop string stays back

            def chunk(delta, finish=None, usage=None):
                d = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": served_name(body),
                     "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
                if usage:
                    d["usage"] = usage
                return "data: " + json.dumps(d) + "\n\n"

            def deltas(evs):
                nonlocal n_calls
                out = []
                for kind, x in evs:
                    if kind == "content" and x:
                        out.append(chunk({"content": x}))
                    elif kind == "reasoning" and x:
                        out.append(chunk({"reasoning_content": x}))
                    elif kind == "tool_call":
                        out.append(chunk({"tool_calls": [dict(openai_calls([x])[0], index=n_calls)]}))
                        n_calls += 1
                return out
            yield chunk({"role": "assistant"})
            try:
                while True:
                    try:
                        toks, done, reason = await asyncio.wait_for(events.get(), KEEPALIVE_S)
                    except asyncio.TimeoutError:
                        yield ": keepalive\n\n"
                        continue
                    n_out += len(toks)
                    if toks and t_first is None:
                        t_first = time.time()
                    held += dec.push(toks) if toks else ""
                    cut, stopped = _cut_at_stop(held, stops)
                    if stopped or done:
                        for c in deltas(parser.push(cut) + parser.finish()):
                            yield c
                        finish = "tool_calls" if n_calls else ("stop" if stopped else reason)
                        account(rid, key, t0, t_first, len(prompt_ids), n_out, finish)
                        usage = {"prompt_tokens": len(prompt_ids), "completion_tokens": n_out, "total_tokens": len(prompt_ids) + n_out}
                        yield chunk({}, finish, usage if (body.get("stream_options") or {}).get("include_usage") else None)
                        yield "data: [DONE]\n\n"
                        return
                    safe = len(held) - hold
                    if safe > 0:
                        for c in deltas(parser.push(held[:safe])):
                            yield c
                        held = held[safe:]
            finally:
                loop.cancel(rid)
        return StreamingResponse(sse(), media_type="text/event-stream")

    aliases = dict(model_aliases or {})

    def served_name(body):
        """The name echoed back: a known alias is accepted as is, anything else is answered under the served id."""
        asked = body.get("model")
        return asked if asked in aliases or asked == model_id else model_id

    if allow_origin:
        @app.middleware("http")
        async def cors(request, call_next):
            if request.method == "OPTIONS":
                resp = JSONResponse({})
            else:
                resp = await call_next(request)
            resp.headers["access-control-allow-origin"] = allow_origin
            resp.headers["access-control-allow-headers"] = "authorization, content-type, x-api-key, anthropic-version"
            resp.headers["access-control-allow-methods"] = "GET, POST, DELETE, OPTIONS"
            return resp

    if not gateway:
        return app

    # ------------------------------------------------------------------ OpenAI Responses
    # response id -> {"response": ..., "messages": conversation including the answer, "owner": API key that created it}.
    # Bounded (the oldest entries go first) and scoped: a response is visible only to the key that stored it.
    stored: dict = {}

    def stored_entry(response_id, owner):
        e = stored.get(response_id)
        if e is None or e["owner"] != owner:
            raise HTTPException(404, f"no stored response {response_id}")
        stored[response_id] = stored.pop(response_id)       # most recently used last
        return e

    def responses_messages(body, owner=None):
        msgs = []
        prev = body.get("previous_response_id")
        if prev:
            msgs += stored_entry(prev, owner)["messages"]
        inp = body.get("input")
        if isinstance(inp, str):
            msgs.append({"role": "user", "content": inp})
        for item in inp if isinstance(inp, list) else []:
            kind = item.get("type", "message")
            if kind == "message":
                content = item.get("content")
                if isinstance(content, list):
                    if any(isinstance(p, dict) and p.get("type") == "input_image" for p in content):     # kept as parts for the vision front end
                        content = [p if p.get("type") == "input_image" else {"type": "text", "text": p.get("text", "")}
                                   for p in content if isinstance(p, dict)]
                    else:
                        content = "".join(p.get("text", "") for p in content if isinstance(p, dict))
                msgs.append({"role": item.get("role", "user"), "content": content})
            elif kind == "function_call":
                msgs.append({"role": "assistant", "content": "", "tool_calls": [{"id": item.get("call_id"), "function": {
                    "name": item.get("name"), "arguments": item.get("arguments", "{}")}}]})
            elif kind == "function_call_output":
                msgs.append({"role": "tool", "tool_call_id": item.get("call_id"), "content": str(item.get("output", ""))})
        tools = [{"type": "function", "function": {"name": t.get("name"), "description": t.get("description", ""), "parameters": t.get("parameters")}}
                 for t in body.get("tools") or [] if t.get("type") == "function" and t.get("name")]
        return msgs, tools

    def response_object(rid, body, parsed, n_in, n_out, status="completed"):
        out = []
        if parsed["reasoning"]:
            out.append({"type": "reasoning", "id": "rs_" + rid, "summary": [{"type": "summary_text", "text": parsed["reasoning"]}]})
        if parsed["content"] or not parsed["tool_calls"]:
            out.append({"type": "message", "id": "msg_" + rid, "role": "assistant", "status": "completed",
                        "content": [{"type": "output_text", "text": parsed["content"], "annotations": []}]})
        for c in parsed["tool_calls"]:
            out.append({"type": "function_call", "id": "fc_" + c["id"][5:], "call_id": c["id"], "name": c["name"],
                        "arguments": json.dumps(c["arguments"], ensure_ascii=False), "status": "completed"})
        return {"id": "resp_" + rid, "object": "response", "created_at": int(time.time()), "status": status, "model": served_name(body),
                "output": out, "output_text": parsed["content"], "previous_response_id": body.get("previous_response_id"),
                "usage": {"input_tokens": n_in, "output_tokens": n_out, "total_tokens": n_in + n_out}}

    @app.post("/v1/responses")
    async def responses(http: HttpRequest, authorization: str = Header(None)):
        owner = auth(authorization)
        body = await http.json()
        msgs, tools = responses_messages(body, owner)
        if not msgs:
            raise HTTPException(400, "input is required")
        thinking, stops = chat_options(body)
        if (body.get("reasoning") or {}).get("effort") not in (None, "none", "minimal"):
            thinking = True
        prompt_ids, embeds = await build_prompt(msgs, tools=tools or None, system=body.get("instructions"), thinking=thinking)
        t0, key = time.time(), key_of(authorization)
        rf = {"response_format": (body.get("text") or {}).get("format")} if isinstance((body.get("text") or {}).get("format"), dict) else {}
        rid, events = start_generation(prompt_ids, body, int(body.get("max_output_tokens") or 256), constraint_for(rf, len(prompt_ids)), None, embeds)

        def finish(ids, reason):
            text, _ = _cut_at_stop(tok.decode(ids), stops)
            parsed = parse_completion(tmpl, text, thinking)
            account(rid, key, t0, None, len(prompt_ids), len(ids), reason)
            resp = response_object(rid, body, parsed, len(prompt_ids), len(ids), "completed" if reason != "length" else "incomplete")
            if body.get("store", True):
                answer = {"role": "assistant", "content": parsed["content"]}
                if parsed["tool_calls"]:
                    answer["tool_calls"] = openai_calls(parsed["tool_calls"])
                stored[resp["id"]] = {"response": resp, "messages": msgs + [answer], "owner": owner}
                while len(stored) > 256:
                    stored.pop(next(iter(stored)))
            return resp, parsed
        if not body.get("stream"):
            ids, reason = await collect(events)
            if reason and reason.startswith(("error", "unavailable", "busy", "queue full")):
                raise HTTPException(503, reason)
            return finish(ids, reason)[0]

        async def sse():
            seq = 0

            def ev(name, data):
                nonlocal seq
                seq += 1
                return f"event: {name}\ndata: " + json.dumps(dict(data, type=name, sequence_number=seq)) + "\n\n"
            shell = response_object(rid, body, {"reasoning": "", "content": "", "tool_calls": []}, len(prompt_ids), 0, "in_progress")
            shell["output"] = []
            yield ev("response.created", {"response": shell})
            dec, parser, ids = StreamDecoder(tok), tmpl.parser(thinking), []
            held = ""
            hold = max((len(x) for x in stops), default=1) - 1
            try:
                while True:
                    try:
                        toks, done, reason = await asyncio.wait_for(events.get(), KEEPALIVE_S)
                    except asyncio.TimeoutError:
                        yield ": keepalive\n\n"
                        continue
                    ids += toks
                    held += dec.push(toks) if toks else ""
                    cut, stopped = _cut_at_stop(held, stops)
                    final = stopped or done
                    safe = len(cut) if final else len(held) - hold
                    if safe > 0:
                        for kind, x in parser.push(held[:safe]) + (parser.finish() if final else []):
                            if kind == "content" and x:
                                yield ev("response.output_text.delta", {"item_id": "msg_" + rid, "output_index": 0, "content_index": 0, "delta": x})
                            elif kind == "reasoning" and x:
                                yield ev("response.reasoning_summary_text.delta", {"item_id": "rs_" + rid, "output_index": 0, "summary_index": 0, "delta": x})
                        held = held[safe:]
                    if final:
                        resp, parsed = finish(ids, "stop" if stopped else reason)
                        for i, item in enumerate(resp["output"]):
                            yield ev("response.output_item.done", {"output_index": i, "item": item})
                        yield ev("response.completed", {"response": resp})
                        return
            finally:
                loop.cancel(rid)
        return StreamingResponse(sse(), media_type="text/event-stream")

    @app.get("/v1/responses/{response_id}")
    async def get_response(response_id: str, authorization: str = Header(None)):
        return stored_entry(response_id, auth(authorization))["response"]

    @app.delete("/v1/responses/{response_id}")
    async def delete_response(response_id: str, authorization: str = Header(None)):
        stored_entry(response_id, auth(authorization))
        stored.pop(response_id, None)
        return {"id": response_id, "object": "response", "deleted": True}

    async def anthropic_prompt(body):
        msgs, tools = _anthropic_to_openai(body)
        system = body.get("system")
        if isinstance(system, list):
            system = "".join(b.get("text", "") for b in system if isinstance(b, dict))
        thinking, stops = chat_options(body)
        ids, embeds = await build_prompt(msgs, tools=tools or None, system=system or None, thinking=thinking)
        return ids, thinking, stops, embeds

    @app.post("/v1/messages/count_tokens")
    async def count_tokens(http: HttpRequest, authorization: str = Header(None), x_api_key: str = Header(None)):
        auth(authorization, x_api_key)
        return {"input_tokens": len((await anthropic_prompt(await http.json()))[0])}

    @app.post("/v1/messages")
    async def messages(http: HttpRequest, authorization: str = Header(None), x_api_key: str = Header(None)):
        auth(authorization, x_api_key)
        body = await http.json()
        if "max_tokens" not in body:
            raise HTTPException(400, "max_tokens is required")
        prompt_ids, thinking, stops, embeds = await anthropic_prompt(body)
        t0, key = time.time(), key_of(authorization, x_api_key)
        rid, events = start_generation(prompt_ids, body, int(body["max_tokens"]), None, None, embeds)
        mid = "msg_" + rid

        def blocks_of(parsed):
            out = []
            if parsed["reasoning"]:
                out.append({"type": "thinking", "thinking": parsed["reasoning"]})
            if parsed["content"] or not parsed["tool_calls"]:
                out.append({"type": "text", "text": parsed["content"]})
            out += [{"type": "tool_use", "id": "toolu_" + c["id"][5:], "name": c["name"], "input": c["arguments"]} for c in parsed["tool_calls"]]
            return out

        def stop_reason(parsed, stopped, reason):
            return "tool_use" if parsed["tool_calls"] else ("stop_sequence" if stopped and body.get("stop_sequences") else
                                                            ("end_turn" if stopped or reason == "stop" else "max_tokens"))
        if not body.get("stream"):
            ids, reason = await collect(events)
            if reason and reason.startswith(("error", "unavailable", "busy", "queue full")):
                raise HTTPException(503, reason)
            text, stopped = _cut_at_stop(tok.decode(ids), stops)
            parsed = parse_completion(tmpl, text, thinking)
            account(rid, key, t0, None, len(prompt_ids), len(ids), reason)
            return {"id": mid, "type": "message", "role": "assistant", "model": model_id, "content": blocks_of(parsed),
                    "stop_reason": stop_reason(parsed, stopped, reason), "stop_sequence": None,
                    "usage": {"input_tokens": len(prompt_ids), "output_tokens": len(ids)}}

        async def sse():
            """Anthropic event stream; blocks are emitted whole-block-at-a-time per parser event."""
            def ev(name, data):
                return f"event: {name}\ndata: " + json.dumps(dict(data, type=name)) + "\n\n"
            yield ev("message_start", {"message": {"id": mid, "type": "message", "role": "assistant", "model": model_id, "content": [],
                                                   "stop_reason": None, "usage": {"input_tokens": len(prompt_ids), "output_tokens": 0}}})
            dec, parser = StreamDecoder(tok), tmpl.parser(thinking)
            held, n_out, index, open_kind, any_call = "", 0, -1, None, False
            hold = max((len(x) for x in stops), default=1) - 1

            def emit(evs):
                nonlocal index, open_kind, any_call
                out = []
                for kind, x in evs:
                    want = {"content": "text", "reasoning": "thinking", "tool_call": "tool_use"}[kind]
                    if kind != "tool_call" and not x:
                        continue
                    if open_kind is not None and (open_kind != want or want == "tool_use"):
                        out.append(ev("content_block_stop", {"index": index}))
                        open_kind = None
                    if open_kind is None:
                        index += 1
                        start = ({"type": "text", "text": ""} if want == "text" else {"type": "thinking", "thinking": ""} if want == "thinking"
                                 else {"type": "tool_use", "id": "toolu_" + x["id"][5:], "name": x["name"], "input": {}})
                        out.append(ev("content_block_start", {"index": index, "content_block": start}))
                        open_kind = want
                    if want == "text":
                        out.append(ev("content_block_delta", {"index": index, "delta": {"type": "text_delta", "text": x}}))
                    elif want == "thinking":
                        out.append(ev("content_block_delta", {"index": index, "delta": {"type": "thinking_delta", "thinking": x}}))
                    else:
                        any_call = True
                        out.append(ev("content_block_delta", {"index": index, "delta": {"type": "input_json_delta",
                                                                                       "partial_json": json.dumps(x["arguments"], ensure_ascii=False)}}))
                return out
            try:
                while True:
                    try:
                        toks, done, reason = await asyncio.wait_for(events.get(), KEEPALIVE_S)
                    except asyncio.TimeoutError:
                        yield ev("ping", {})
                        continue
                    n_out += len(toks)
                    held += dec.push(toks) if toks else ""
                    cut, stopped = _cut_at_stop(held, stops)
                    if stopped or done:
                        for c in emit(parser.push(cut) + parser.finish()):
                            yield c
                        if open_kind is not None:
                            yield ev("content_block_stop", {"index": index})
                        sr = "tool_use" if any_call else ("end_turn" if stopped or reason == "stop" else "max_tokens")
                        account(rid, key, t0, None, len(prompt_ids), n_out, sr)
                        yield ev("message_delta", {"delta": {"stop_reason": sr, "stop_sequence": None}, "usage": {"output_tokens": n_out}})
                        yield ev("message_stop", {})
                        return
                    safe = len(held) - hold
                    if safe > 0:
                        for c in emit(parser.push(held[:safe])):
                            yield c
                        held = held[safe:]
            finally:
                loop.cancel(rid)
        return StreamingResponse(sse(), media_type="text/event-stream")

    if gateway:
        from .gateway_extras import install_gateway_extras
        install_gateway_extras(app, tok=tok, tmpl=tmpl, auth=auth, start_generation=start_generation, collect=collect, loop=loop,
                               served_name=served_name, search=search, record_path=record_path, build_prompt=build_prompt,
                               audio=vision is not None and getattr(vision, "audio_tower", None) is not None)
    return app
