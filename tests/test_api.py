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
