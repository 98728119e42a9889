"""Gateway extras against the fake runner (no GPU): Realtime WebSocket text turns, the search endpoint with the in-memory
provider, request recording and replay."""
import json

import pytest
from fastapi.testclient import TestClient

from cuteafd_b200.engine.kv import PagePool
from cuteafd_b200.parallel.health import Health
from cuteafd_b200.serving.api import ServingLoop, build_app
from cuteafd_b200.serving.gateway_extras import CorpusProvider, replay
from cuteafd_b200.serving.runner import FakeRunner
from cuteafd_b200.serving.scheduler import Scheduler


def _loop(script: bytes | None = None):
    runner = FakeRunner(vocab=258)
    if script is None:
        runner.next_token = lambda prefix: 97 + (sum(prefix[-3:]) % 26)           # lower-case letters, deterministic
    else:
        state = {}

        def next_token(prefix):
            n0 = state.setdefault("prompt", len(prefix))
            i = len(prefix) - n0
            return script[i] if i < len(script) else 257
        runner.next_token = next_token
    return ServingLoop(Scheduler(runner, PagePool(512)), Health()).start()


def test_realtime_websocket_text_turn():
    loop = _loop(b"Hello there.")
    try:
        c = TestClient(build_app(loop, api_keys={"k1"}))
        with c.websocket_connect("/v1/realtime", headers={"Authorization": "Bearer k1"}) as ws:
            assert json.loads(ws.receive_text())["type"] == "session.created"
            ws.send_text(json.dumps({"type": "session.update", "session": {"instructions": "be brief", "max_response_output_tokens": 32}}))
            upd = json.loads(ws.receive_text())
            assert upd["type"] == "session.updated" and upd["session"]["instructions"] == "be brief"
            ws.send_text(json.dumps({"type": "conversation.item.create",
                                     "item": {"type": "message", "role": "user", "content": [{"type": "input_text", "text": "hi"}]}}))
            assert json.loads(ws.receive_text())["type"] == "conversation.item.created"
            ws.send_text(json.dumps({"type": "response.create"}))
            kinds, text, done = [], "", None
            while done is None:
                ev = json.loads(ws.receive_text())
                kinds.append(ev["type"])
                if ev["type"] == "response.text.delta":
                    text += ev["delta"]
                if ev["type"] == "response.done":
                    done = ev
            assert kinds[0] == "response.created" and "response.text.done" in kinds
            assert text == "Hello there." and done["response"]["status"] == "completed"
            assert done["response"]["output"][0]["content"][0]["text"] == "Hello there." and done["response"]["usage"]["output_tokens"] >= 12
            # audio items and unknown events are refused with an error event, the connection stays usable
            ws.send_text(json.dumps({"type": "conversation.item.create", "item": {"type": "message", "content": [{"type": "input_audio", "audio": "x"}]}}))
            assert json.loads(ws.receive_text())["type"] == "error"
            ws.send_text(json.dumps({"type": "input_audio_buffer.append", "audio": "x"}))
            assert json.loads(ws.receive_text())["type"] == "error"
        with pytest.raises(Exception):           # a wrong key is refused at the handshake
            with c.websocket_connect("/v1/realtime", headers={"Authorization": "Bearer nope"}):
                pass
    finally:
        loop.stop()


def test_search_endpoint_with_the_corpus_provider():
    loop = _loop()
    try:
        docs = [{"title": "NVLink 5", "url": "doc://nvlink", "text": "NVLink 5 gives every GPU 900 GB/s per direction through NVSwitch."},
                {"title": "HBM3e", "url": "doc://hbm", "text": "Each B200 has 180 GB of HBM3e."}]
        c = TestClient(build_app(loop, search=CorpusProvider(docs)))
        r = c.post("/v1/alpha/search", json={"query": "nvswitch bandwidth per direction", "max_results": 3}).json()
        assert r["results"] and r["results"][0]["url"] == "doc://nvlink" and "900 GB/s" in r["results"][0]["snippet"]
        assert c.post("/v1/alpha/search", json={"query": ""}).status_code == 400
        assert TestClient(build_app(loop)).post("/v1/alpha/search", json={"query": "x"}).status_code == 501
    finally:
        loop.stop()


def test_record_and_replay(tmp_path):
    path = str(tmp_path / "rec.jsonl")
    loop = _loop()
    try:
        c = TestClient(build_app(loop, record_path=path))
        body = {"messages": [{"role": "user", "content": "count"}], "max_tokens": 12, "temperature": 0}
        first = c.post("/v1/chat/completions", json=body).json()
        c.post("/v1/chat/completions", json=dict(body, stream=True))
        c.post("/v1/responses", json={"input": "hello", "max_output_tokens": 8})
        lines = [json.loads(l) for l in open(path)]
        assert [l["path"] for l in lines] == ["/v1/chat/completions", "/v1/chat/completions", "/v1/responses"]
        assert lines[0]["response"]["choices"][0]["message"]["content"] == first["choices"][0]["message"]["content"]
        assert isinstance(lines[1]["response"], list) and lines[1]["response"][0]["object"] == "chat.completion.chunk"
        # replay against the same deterministic model matches; against a model that answers differently it does not
        rep = replay(build_app(loop), path)
        assert rep == {"requests": 3, "matched": 3, "mismatches": []}
    finally:
        loop.stop()
    other = _loop(b"something else")
    try:
        rep = replay(build_app(other), path)
        assert rep["requests"] == 3 and rep["matched"] == 0 and len(rep["mismatches"]) == 3
    finally:
        other.stop()


def test_realtime_websocket_takes_microphone_audio_when_an_audio_tower_is_loaded():
    """`input_audio_buffer.append` / `.commit` turn PCM from the socket into a user item; the response's prompt carries the audio
    placeholders and the tower's rows, exactly like an `input_audio` part of the chat surface."""
    import base64

    import numpy as np
    import torch

    from cuteafd_b200.ref.audio import AudioSpec
    from cuteafd_b200.serving.vision import VisionFrontEnd

    class FakeAudio:
        device = None
        spec = AudioSpec(out_hidden=8, n_mels=16)
        encodes = 0

        def encode(self, clips):
            self.encodes += 1
            return [torch.ones(c.shape[0] // 4, 8, dtype=torch.bfloat16) for c in clips]

    loop = _loop(b"I heard you.")
    seen = []
    runner = loop.sched.runner
    real_run = runner.run
    runner.run = lambda rows: (seen.extend((r.state.req.embeds, list(r.tokens)) for r in rows), real_run(rows))[1]
    audio = FakeAudio()
    try:
        c = TestClient(build_app(loop, vision=VisionFrontEnd(None, audio_tower=audio, audio_pad_id=250, audio_start_id=251, audio_end_id=252)))
        pcm = (np.sin(np.arange(24000) * 0.03) * 9000).astype("<i2").tobytes()              # one second at the socket's 24 kHz
        with c.websocket_connect("/v1/realtime") as ws:
            assert json.loads(ws.receive_text())["type"] == "session.created"
            for i in range(0, len(pcm), 16000):
                ws.send_text(json.dumps({"type": "input_audio_buffer.append", "audio": base64.b64encode(pcm[i:i + 16000]).decode()}))
            ws.send_text(json.dumps({"type": "input_audio_buffer.commit"}))
            assert json.loads(ws.receive_text())["type"] == "input_audio_buffer.committed"
            created = json.loads(ws.receive_text())
            assert created["type"] == "conversation.item.created" and created["item"]["content"][0]["type"] == "input_audio"
            ws.send_text(json.dumps({"type": "input_audio_buffer.commit"}))                  # nothing buffered any more
            assert json.loads(ws.receive_text())["type"] == "error"
            ws.send_text(json.dumps({"type": "response.create"}))
            text, done = "", None
            while done is None:
                ev = json.loads(ws.receive_text())
                if ev["type"] == "response.text.delta":
                    text += ev["delta"]
                if ev["type"] == "response.done":
                    done = ev
            assert text == "I heard you." and done["response"]["status"] == "completed"
        assert audio.encodes == 1
        emb, toks = next(s for s in seen if s[0] is not None)
        assert toks.count(250) == 25 and emb["rows"].shape == (25, 8)                          # 1 s -> 100 frames at 16 kHz -> 25 tokens
        assert [toks[p] for p in emb["positions"]] == [250] * 25
    finally:
        loop.stop()
