"""HTTP surface against the fake runner (no GPU): OpenAI chat (plain + SSE), models, stats, health, Anthropic messages,
auth, failure to 503."""
import json

import pytest

fastapi = pytest.importorskip("fastapi")
from fastapi.testclient import TestClient

from cuteafd_b200.engine.kv import PagePool
from cuteafd_b200.parallel.health import Health
from cuteafd_b200.serving.api import ServingLoop, build_app
from cuteafd_b200.serving.prefix import PrefixCache
from cuteafd_b200.serving.runner import FakeRunner
from cuteafd_b200.serving.scheduler import Scheduler


@pytest.fixture
def client():
    pool = PagePool(256)
    runner = FakeRunner(vocab=96)
    runner.next_token = lambda prefix: 32 + (sum(prefix[-3:]) % 60)          # printable bytes
    health = Health()
    loop = ServingLoop(Scheduler(runner, pool, prefix=PrefixCache(pool)), health).start()
    c = TestClient(build_app(loop, api_keys={"sekret"}))
    c.loop, c.health_obj = loop, health
    yield c
    loop.stop()


H = {"Authorization": "Bearer sekret"}


def test_chat_completion_and_usage(client):
    r = client.post("/v1/chat/completions", headers=H, json={"messages": [{"role": "user", "content": "hi there"}], "max_tokens": 12})
    assert r.status_code == 200
    j = r.json()
    assert j["choices"][0]["finish_reason"] == "length" and j["usage"]["completion_tokens"] == 12
    assert len(j["choices"][0]["message"]["content"]) == 12
    assert client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}]}).status_code == 401
    assert client.post("/v1/chat/completions", headers=H, json={"messages": []}).status_code == 400
    assert client.post("/v1/chat/completions", headers=H, json={"messages": [{"role": "user", "content": "x"}], "temperature": 9}).status_code == 400


def test_streaming_matches_non_streaming(client):
    body = {"messages": [{"role": "user", "content": "stream me"}], "max_tokens": 10}
    plain = client.post("/v1/chat/completions", headers=H, json=body).json()["choices"][0]["message"]["content"]
    text, finish = "", None
    with client.stream("POST", "/v1/chat/completions", headers=H, json=dict(body, stream=True)) as r:
        for line in r.iter_lines():
            if line.startswith("data: ") and line != "data: [DONE]":
                ch = json.loads(line[6:])["choices"][0]
                text += ch["delta"].get("content", "")
                finish = ch["finish_reason"] or finish
    assert text == plain and finish == "length"


def test_models_stats_console_and_anthropic(client):
    assert client.get("/v1/models", headers=H).json()["data"][0]["id"] == "cuteafd-b200"
    r = client.post("/v1/messages", headers={"x-api-key": "sekret"}, json={"max_tokens": 5, "system": "be brief", "messages": [{"role": "user", "content": "yo"}]})
    assert r.status_code == 200 and r.json()["usage"]["output_tokens"] == 5 and r.json()["content"][0]["type"] == "text"
    assert client.post("/v1/messages", headers={"x-api-key": "sekret"}, json={"messages": []}).status_code == 400
    n = client.post("/v1/messages/count_tokens", headers={"x-api-key": "sekret"}, json={"messages": [{"role": "user", "content": "abc"}]}).json()
    assert n["input_tokens"] > 3
    s = client.get("/v1/stats").json()
    assert s["finished"] >= 1 and s["healthy"] and "prefix" in s
    assert "lanes" in client.get("/v1/console/snapshot").json()


def test_wire_failure_turns_the_server_unavailable(client):
    assert client.get("/health").status_code == 200
    client.health_obj.record_failure("expert rank 3 stopped answering")
    import time
    time.sleep(0.05)
    assert client.get("/health").status_code == 503
    r = client.post("/v1/chat/completions", headers=H, json={"messages": [{"role": "user", "content": "x"}]})
    assert r.status_code == 503


def _scripted_client(script: str, model: str):
    """Server whose fake model recites `script` (then end of sequence) after any prompt."""
    from cuteafd_b200.serving.chat_templates import template_for
    pool = PagePool(512)
    runner = FakeRunner(vocab=258)
    data = script.encode()
    state = {}

    def next_token(prefix):
        n0 = state.setdefault("prompt", len(prefix))             # the first call sees exactly the prompt
        i = len(prefix) - n0
        return data[i] if i < len(data) else 257
    runner.next_token = next_token
    loop = ServingLoop(Scheduler(runner, pool), Health()).start()
    return TestClient(build_app(loop, model_id=model, template=template_for(model))), loop


def test_tool_calls_reasoning_and_stop_strings_in_chat_completions():
    script = "<think>\nuse the tool\n</think>\n\nOn it.\n<tool_call>\n{\"name\": \"get_weather\", \"arguments\": {\"city\": \"Oslo\"}}\n</tool_call><|im_end|>"
    c, loop = _scripted_client(script, "qwen3-235b")
    try:
        body = {"messages": [{"role": "user", "content": "weather?"}], "max_tokens": 200,
                "tools": [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object"}}}]}
        m = c.post("/v1/chat/completions", json=body).json()["choices"][0]
        assert m["finish_reason"] == "tool_calls" and m["message"]["content"] == "On it." and m["message"]["reasoning_content"].strip() == "use the tool"
        call = m["message"]["tool_calls"][0]
        assert call["function"]["name"] == "get_weather" and json.loads(call["function"]["arguments"]) == {"city": "Oslo"}
    finally:
        loop.stop()
    c, loop = _scripted_client(script, "qwen3-235b")
    try:
        text, reasoning, calls, finish = "", "", [], None
        with c.stream("POST", "/v1/chat/completions", json=dict(body, stream=True)) as r:
            for line in r.iter_lines():
                if line.startswith("data: ") and line != "data: [DONE]":
                    ch = json.loads(line[6:])["choices"][0]
                    text += ch["delta"].get("content", "")
                    reasoning += ch["delta"].get("reasoning_content", "")
                    calls += ch["delta"].get("tool_calls", [])
                    finish = ch["finish_reason"] or finish
        assert finish == "tool_calls" and text.strip() == "On it." and reasoning.strip() == "use the tool" and "<" not in text
        assert calls[0]["function"]["name"] == "get_weather" and calls[0]["index"] == 0
    finally:
        loop.stop()
    c, loop = _scripted_client("alpha beta STOP gamma", "plain")
    try:
        m = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "max_tokens": 50, "stop": ["STOP"]}).json()["choices"][0]
        assert m["message"]["content"] == "alpha beta " and m["finish_reason"] == "stop"
    finally:
        loop.stop()


def test_json_mode_masks_the_fake_model_into_json(client):
    from cuteafd_b200.serving.constraints import JsonPrefix
    client.loop.sched.runner.vocab = 258
    r = client.post("/v1/chat/completions", headers=H, json={"messages": [{"role": "user", "content": "json please"}], "max_tokens": 40,
                                                             "response_format": {"type": "json_object"}}).json()["choices"][0]
    text = r["message"]["content"]
    assert text.lstrip().startswith("{") and JsonPrefix("object").feed_text(text)
    if r["finish_reason"] == "stop":
        assert isinstance(json.loads(text), dict)


def test_anthropic_tools_and_event_stream():
    script = "Checking.<tool_call>get_weather\n<arg_key>city</arg_key>\n<arg_value>Oslo</arg_value>\n</tool_call>"
    body = {"max_tokens": 200, "messages": [{"role": "user", "content": [{"type": "text", "text": "weather?"}]}],
            "tools": [{"name": "get_weather", "description": "w", "input_schema": {"type": "object"}}]}
    c, loop = _scripted_client(script, "glm-5")
    try:
        j = c.post("/v1/messages", json=body).json()
        assert j["stop_reason"] == "tool_use" and [b["type"] for b in j["content"]] == ["text", "tool_use"]
        assert j["content"][1]["name"] == "get_weather" and j["content"][1]["input"] == {"city": "Oslo"}
    finally:
        loop.stop()
    c, loop = _scripted_client(script, "glm-5")
    try:
        names, text, partial = [], "", ""
        with c.stream("POST", "/v1/messages", json=dict(body, stream=True)) as r:
            for line in r.iter_lines():
                if line.startswith("event: "):
                    names.append(line[7:])
                elif line.startswith("data: "):
                    d = json.loads(line[6:])
                    if d["type"] == "content_block_delta":
                        text += d["delta"].get("text", "")
                        partial += d["delta"].get("partial_json", "")
                    if d["type"] == "message_delta":
                        assert d["delta"]["stop_reason"] == "tool_use"
        assert names[0] == "message_start" and names[-1] == "message_stop" and names.count("content_block_start") == 2
        assert text == "Checking." and json.loads(partial) == {"city": "Oslo"}
    finally:
        loop.stop()


def test_usage_accounting_probe_header_and_usage_command(tmp_path):
    import io
    from cuteafd_b200 import cli
    from cuteafd_b200.serving.usage import UsageStore, synthetic_history
    pool = PagePool(256)
    runner = FakeRunner(vocab=96)
    cache = PrefixCache(pool)
    loop = ServingLoop(Scheduler(runner, pool, prefix=cache), Health()).start()
    store = UsageStore(str(tmp_path / "usage.sqlite"))
    c = TestClient(build_app(loop, usage=store, enable_bench=True, api_keys={"sekret-key-1"}))
    try:
        long_prompt = "p" * 300
        body = {"messages": [{"role": "user", "content": long_prompt}], "max_tokens": 4}
        for _ in range(2):
            assert c.post("/v1/chat/completions", headers={"Authorization": "Bearer sekret-key-1"}, json=body).status_code == 200
        u = c.get("/usage", headers={"Authorization": "Bearer sekret-key-1"}).json()
        assert u["totals"]["requests"] == 2 and u["totals"]["completion_tokens"] == 8 and u["totals"]["cache_hit_tokens"] >= 256
        assert u["by_key"][0]["api_key"] == "sekret..."                                   # keys are stored truncated
        hits = cache.stats["hits"]
        probe = {"x-cuteafd-probe": json.dumps({"skip_cache": True, "no_drafts": True}), "Authorization": "Bearer sekret-key-1"}
        assert c.post("/v1/chat/completions", headers=probe, json=body).status_code == 200
        assert cache.stats["hits"] == hits                                                # the probe bypassed the prefix cache
        ids = {"x-cuteafd-probe": json.dumps({"token_ids": [40, 41, 42]}), "Authorization": "Bearer sekret-key-1"}
        assert c.post("/v1/chat/completions", headers=ids, json=body).json()["usage"]["prompt_tokens"] == 3
        assert c.get("/v1/thermal").status_code == 200
    finally:
        loop.stop()
    buf = io.StringIO()
    assert store.export_csv(buf, "1h") == 4 and buf.getvalue().splitlines()[0].startswith("id,time,model")
    assert cli.main(["usage", "export-csv", "--dir", str(tmp_path), "--out", str(tmp_path / "u.csv")]) == 0
    assert len((tmp_path / "u.csv").read_text().splitlines()) == 5
    assert cli.main(["usage", "clear", "--dir", str(tmp_path)]) == 0
    assert UsageStore(str(tmp_path / "usage.sqlite")).totals()["requests"] == 0
    demo = UsageStore()
    synthetic_history(demo, days=3, per_day=5)
    assert demo.totals()["requests"] == 15 and len(demo.daily()) >= 3


def test_responses_surface_stores_chains_and_streams():
    c, loop = _scripted_client("Hello there.", "plain")
    try:
        r1 = c.post("/v1/responses", json={"model": "cuteafd-b200", "input": "hi", "instructions": "be brief", "max_output_tokens": 50}).json()
        assert r1["status"] == "completed" and r1["output_text"] == "Hello there." and r1["output"][0]["content"][0]["type"] == "output_text"
        assert c.get("/v1/responses/" + r1["id"]).json()["id"] == r1["id"]
        # the follow-up renders the stored conversation in front of the new input
        r2 = c.post("/v1/responses", json={"input": [{"type": "message", "role": "user", "content": [{"type": "input_text", "text": "again"}]}],
                                           "previous_response_id": r1["id"], "max_output_tokens": 50}).json()
        assert r2["previous_response_id"] == r1["id"] and r2["usage"]["input_tokens"] > r1["usage"]["input_tokens"]
        assert c.post("/v1/responses", json={"input": "x", "previous_response_id": "resp_missing"}).status_code == 404
        assert c.delete("/v1/responses/" + r1["id"]).json()["deleted"] and c.get("/v1/responses/" + r1["id"]).status_code == 404
    finally:
        loop.stop()
    c, loop = _scripted_client("Hello there.", "plain")
    try:
        names, text, final = [], "", None
        with c.stream("POST", "/v1/responses", json={"input": "hi", "stream": True, "max_output_tokens": 50}) as r:
            for line in r.iter_lines():
                if line.startswith("event: "):
                    names.append(line[7:])
                elif line.startswith("data: "):
                    d = json.loads(line[6:])
                    text += d.get("delta", "") if d["type"] == "response.output_text.delta" else ""
                    final = d["response"] if d["type"] == "response.completed" else final
        assert names[0] == "response.created" and names[-1] == "response.completed" and text == "Hello there." == final["output_text"]
    finally:
        loop.stop()


def test_model_aliases_cors_and_gateway_off():
    pool = PagePool(64)
    loop = ServingLoop(Scheduler(FakeRunner(vocab=96), pool), Health()).start()
    try:
        c = TestClient(build_app(loop, model_aliases={"gpt-4o": "served", "claude-x": "served"}, allow_origin="https://ui.example"))
        ids = [m["id"] for m in c.get("/v1/models").json()["data"]]
        assert ids == ["cuteafd-b200", "gpt-4o", "claude-x"]
        r = c.post("/v1/chat/completions", json={"model": "gpt-4o", "messages": [{"role": "user", "content": "x"}], "max_tokens": 2})
        assert r.json()["model"] == "gpt-4o" and r.headers["access-control-allow-origin"] == "https://ui.example"
        assert c.post("/v1/chat/completions", json={"model": "unknown", "messages": [{"role": "user", "content": "x"}], "max_tokens": 2}).json()["model"] == "cuteafd-b200"
        off = TestClient(build_app(loop, gateway=False))
        assert off.post("/v1/messages", json={"max_tokens": 2, "messages": [{"role": "user", "content": "x"}]}).status_code == 404
        assert off.post("/v1/responses", json={"input": "x"}).status_code == 404
        assert off.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "max_tokens": 2}).status_code == 200
    finally:
        loop.stop()


def test_console_dashboard_snapshot_and_scheduler_observability(client, tmp_path, monkeypatch):
    assert "cuteafd-b200 console" in client.get("/").text
    s = client.loop.sched
    s.watchers += 1                                           # as if a dashboard were connected
    client.post("/v1/chat/completions", headers=H, json={"messages": [{"role": "user", "content": "observe me"}], "max_tokens": 6})
    snap = client.get("/v1/console/snapshot").json()
    assert snap["recent"][-1]["generated"] == 6 and snap["stats"]["phases"]["run"]["n"] >= 1
    kinds = {e["kind"] for e in s.events}
    assert {"decode", "finish"} <= kinds
    s.watchers -= 1
    n = len(s.events)
    client.post("/v1/chat/completions", headers=H, json={"messages": [{"role": "user", "content": "nobody watches"}], "max_tokens": 3})
    assert len(s.events) == n                                 # no viewers: nothing recorded


def test_speculation_trace_and_acceptance_by_position(tmp_path, monkeypatch):
    from cuteafd_b200.serving.scheduler import NgramDrafter, Request
    path = tmp_path / "spec.jsonl"
    monkeypatch.setenv("CUTEAFD_SPECULATION_TRACE", str(path))
    pool = PagePool(128)
    runner = FakeRunner(vocab=50)
    runner.next_token = lambda prefix: prefix[-4]             # period-4 stream: the n-gram drafter predicts it
    sched = Scheduler(runner, pool, drafter=NgramDrafter(), max_draft=3)
    sched.submit(Request("r", [1, 2, 3, 4] * 6, max_tokens=24))
    sched.run_until_idle()
    snap = sched.snapshot()
    assert snap["drafted"] > 0 and snap["accepted"] > 0 and snap["draft_acceptance_by_position"][0] is not None
    lines = [json.loads(l) for l in path.read_text().splitlines()]
    assert lines and all(l["rid"] == "r" and 0 <= l["accepted"] <= l["drafted"] for l in lines)
    assert sum(l["drafted"] for l in lines) == snap["drafted"]


def test_fabric_endpoint_without_gpus(client):
    r = client.get("/v1/fabric")
    assert r.status_code == 200 and "available" in r.json()


def test_tool_choice_forces_a_call_with_schema_checked_arguments():
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"], "additionalProperties": False}}}]
    body = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 120, "tools": tools,
            "tool_choice": {"type": "function", "function": {"name": "get_weather"}}}
    # a model that wants to chat is forced into the call format ...
    c, loop = _scripted_client("Sure, happy to help!", "qwen3-235b")
    try:
        loop.sched.runner.vocab = 258
        m = c.post("/v1/chat/completions", json=body).json()["choices"][0]
        raw = (m["message"]["content"] or "") + json.dumps(m["message"].get("tool_calls", []))
        assert "get_weather" in raw and "Sure" not in raw
    finally:
        loop.stop()
    # ... and a model that already writes a valid call passes through unchanged
    script = '<tool_call>\n{"name": "get_weather", "arguments": {"city": "Oslo"}}\n</tool_call>'
    c, loop = _scripted_client(script, "qwen3-235b")
    try:
        loop.sched.runner.vocab = 258
        m = c.post("/v1/chat/completions", json=dict(body, tool_choice="required")).json()["choices"][0]
        assert m["finish_reason"] == "tool_calls" and json.loads(m["message"]["tool_calls"][0]["function"]["arguments"]) == {"city": "Oslo"}
    finally:
        loop.stop()


def test_stored_responses_belong_to_the_key_that_created_them():
    """A response id is no capability: another API key can neither read it, chain onto it, nor delete it."""
    from cuteafd_b200.serving.chat_templates import template_for
    runner = FakeRunner(vocab=258)
    runner.next_token = lambda prefix: 257 if len(prefix) % 7 == 0 else 65
    loop = ServingLoop(Scheduler(runner, PagePool(512)), Health()).start()
    try:
        c = TestClient(build_app(loop, model_id="plain", template=template_for("plain"), api_keys={"alice", "bob"}))
        a, b = {"authorization": "Bearer alice"}, {"authorization": "Bearer bob"}
        r1 = c.post("/v1/responses", json={"input": "hi", "max_output_tokens": 20}, headers=a).json()
        assert c.get("/v1/responses/" + r1["id"], headers=a).status_code == 200
        assert c.get("/v1/responses/" + r1["id"], headers=b).status_code == 404
        assert c.post("/v1/responses", json={"input": "more", "previous_response_id": r1["id"], "max_output_tokens": 20}, headers=b).status_code == 404
        assert c.delete("/v1/responses/" + r1["id"], headers=b).status_code == 404
        assert c.post("/v1/responses", json={"input": "more", "previous_response_id": r1["id"], "max_output_tokens": 20}, headers=a).status_code == 200
        assert c.delete("/v1/responses/" + r1["id"], headers=a).json()["deleted"]
    finally:
        loop.stop()
