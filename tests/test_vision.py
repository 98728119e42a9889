"""Vision tower oracle: patch ordering, resize rule, rotary table, merge-group layout (CPU)."""
import torch

from cuteafd_b200.ref.vision import (VisionSpec, init_vision_weights, patch_order, position_rows, rgb_to_patches, rope_table, smart_grid,
                                     vision_forward)


def test_patch_order_walks_merge_groups():
    ys, xs = patch_order(4, 6, 2)
    assert list(zip(ys[:8].tolist(), xs[:8].tolist())) == [(0, 0), (0, 1), (1, 0), (1, 1), (0, 2), (0, 3), (1, 2), (1, 3)]
    assert sorted(zip(ys.tolist(), xs.tolist())) == [(y, x) for y in range(4) for x in range(6)]


def test_rgb_patches_follow_the_order_and_the_lut():
    spec = VisionSpec(patch=4, merge=2, image_mean=(0.5, 0.4, 0.3), image_std=(0.2, 0.25, 0.5))
    g = torch.Generator().manual_seed(0)
    rgb = torch.randint(0, 256, (8, 16, 3), generator=g, dtype=torch.uint8)
    p = rgb_to_patches(rgb, spec)
    assert p.shape == (2 * 4, 48)
    ys, xs = patch_order(2, 4, 2)
    for row in (0, 3, 5):
        y0, x0 = int(ys[row]) * 4, int(xs[row]) * 4
        for c, py, px in ((0, 0, 0), (1, 2, 3), (2, 3, 1)):
            want = (float(rgb[y0 + py, x0 + px, c]) / 255 - spec.image_mean[c]) / spec.image_std[c]
            assert abs(float(p[row, c * 16 + py * 4 + px]) - want) < 1e-6


def test_smart_grid_keeps_whole_merge_groups_and_token_bounds():
    spec = VisionSpec(patch=16, merge=2, min_tokens=4, max_tokens=64)
    for h, w in ((10, 10), (640, 480), (4000, 300), (37, 1999)):
        gh, gw = smart_grid(h, w, spec)
        assert gh % 2 == 0 and gw % 2 == 0
        assert 4 <= gh * gw // 4 <= 64 or gh * gw // 4 <= 64 + max(gh, gw)       # rounding may overshoot by less than a row of groups
    assert smart_grid(640, 480, VisionSpec(patch=16, merge=2, max_tokens=4096)) == (40, 30)


def test_rope_table_splits_rows_and_columns():
    spec = VisionSpec(head_dim=16, merge=2)
    cs = rope_table(2, 4, spec)
    ys, xs = patch_order(2, 4, 2)
    assert cs.shape == (8, 16)
    # angle 0 of the row half follows y, angle 0 of the column half follows x (inverse frequency 1)
    assert torch.allclose(cs[:, 0], ys.float().cos()) and torch.allclose(cs[:, 8], ys.float().sin())
    assert torch.allclose(cs[:, 4], xs.float().cos()) and torch.allclose(cs[:, 12], xs.float().sin())


def test_position_table_resample_is_identity_on_its_own_grid():
    spec = VisionSpec(hidden=8, pos_grid=4, merge=2)
    t = torch.randn(16, 8)
    r = position_rows(t, 4, 4, spec)
    ys, xs = patch_order(4, 4, 2)
    assert torch.allclose(r, t.reshape(4, 4, 8)[ys, xs], atol=1e-6)


def test_forward_is_invariant_to_which_image_shares_the_batch_and_depends_on_all_patches():
    for kw in (dict(), dict(norm="rmsnorm", mlp="swiglu", qk_norm=True, pos_grid=3)):
        spec = VisionSpec(hidden=32, depth=2, n_heads=2, head_dim=16, intermediate=48, patch=4, out_hidden=24, **kw)
        w = init_vision_weights(spec, 1)
        g = torch.Generator().manual_seed(2)
        rgb = torch.randint(0, 256, (16, 8, 3), generator=g, dtype=torch.uint8)
        p = rgb_to_patches(rgb, spec)
        out = vision_forward(spec, w, p, 4, 2)
        assert out.shape == (2, 24) and torch.isfinite(out).all()
        p2 = p.clone()
        p2[-1] += 1.0                                     # the last patch belongs to the second merge group
        out2 = vision_forward(spec, w, p2, 4, 2)
        assert (out2[0] - out[0]).abs().max() > 1e-6      # bidirectional: the first group's row sees it too


# ---------------------------------------------------------------- image inputs of the API (fake tower, fake runner)
def _png(w, h, seed=0):
    import io

    import numpy as np
    from PIL import Image
    rng = np.random.default_rng(seed)
    buf = io.BytesIO()
    Image.fromarray(rng.integers(0, 256, (h, w, 3), dtype=np.uint8)).save(buf, format="PNG")
    return buf.getvalue()


class _FakeTower:
    device = None

    def __init__(self, spec):
        self.spec, self.encodes, self.seen = spec, 0, []

    def encode(self, images):
        self.encodes += 1
        self.seen += [tuple(im.shape) for im in images]
        P, m = self.spec.patch, self.spec.merge
        return [torch.zeros((im.shape[0] // P) * (im.shape[1] // P) // m ** 2, self.spec.out_hidden, dtype=torch.bfloat16) for im in images]


def test_expand_prompt_places_pads_between_the_text_pieces():
    from cuteafd_b200.serving.vision import IMAGE_MARK, expand_prompt, split_images
    msgs = [{"role": "user", "content": [{"type": "text", "text": "ab"}, {"type": "image_url", "image_url": {"url": "data:image/png;base64,QUJD"}},
                                         {"type": "text", "text": "cd"}, {"type": "image", "source": {"type": "base64", "data": "QUJD"}}]},
            {"role": "assistant", "content": "ok"}]
    out, images = split_images(msgs)
    assert len(images) == 2 and images[1] == b"ABC"
    assert out[0]["content"][1] == {"type": "text", "text": IMAGE_MARK} and out[1] is msgs[1]
    enc = lambda s: [ord(c) for c in s]
    ids, pos = expand_prompt("ab" + IMAGE_MARK + "cd" + IMAGE_MARK, [3, 2], enc, 900, 901, 902)
    assert ids == [97, 98, 900, 901, 901, 901, 902, 99, 100, 900, 901, 901, 902]
    assert pos == [3, 4, 5, 10, 11]


def test_chat_with_image_parts_runs_the_tower_and_bypasses_the_prefix_cache():
    import base64

    import pytest
    pytest.importorskip("fastapi")
    from fastapi.testclient import TestClient

    from cuteafd_b200.engine.kv import PagePool
    from cuteafd_b200.parallel.health import Health
    from cuteafd_b200.ref.vision import VisionSpec
    from cuteafd_b200.serving.api import ServingLoop, build_app
    from cuteafd_b200.serving.prefix import PrefixCache
    from cuteafd_b200.serving.runner import FakeRunner
    from cuteafd_b200.serving.scheduler import Scheduler
    from cuteafd_b200.serving.vision import VisionFrontEnd
    spec = VisionSpec(patch=16, merge=2, out_hidden=8, max_tokens=64)
    tower = _FakeTower(spec)
    pool = PagePool(256)
    runner = FakeRunner(vocab=96)
    runner.next_token = lambda prefix: 32 + (sum(prefix[-3:]) % 60)
    seen = []
    real_run = runner.run
    runner.run = lambda rows: (seen.extend((r.state.req.embeds, list(r.tokens), r.state.req.use_cache) for r in rows), real_run(rows))[1]
    cache = PrefixCache(pool)
    loop = ServingLoop(Scheduler(runner, pool, prefix=cache), Health()).start()
    try:
        url = "data:image/png;base64," + base64.b64encode(_png(96, 64)).decode()
        plain = TestClient(build_app(loop))
        body = {"model": "m", "max_tokens": 4, "messages": [{"role": "user", "content": [{"type": "text", "text": "what is this? "},
                                                                                      {"type": "image_url", "image_url": {"url": url}}]}]}
        assert plain.post("/v1/chat/completions", json=body).status_code == 400            # no tower: refused, not ignored
        c = TestClient(build_app(loop, vision=VisionFrontEnd(tower, pad_id=90, start_id=91, end_id=92)))
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 200, r.text
        assert tower.encodes == 1 and tower.seen == [(64, 96, 3)]                         # 96 x 64 pixels = 6 x 4 patches = 6 tokens
        emb, toks, use_cache = next(s for s in seen if s[0] is not None)
        assert toks.count(90) == 6 and toks.count(91) == 1 and toks.count(92) == 1
        assert emb["rows"].shape == (6, 8) and [toks[p] for p in emb["positions"]] == [90] * 6
        assert use_cache is False and cache.stats["hits"] == 0
        assert r.json()["usage"]["prompt_tokens"] == len(toks)
        # Anthropic surface: base64 image block
        a = c.post("/v1/messages", json={"model": "m", "max_tokens": 3, "messages": [{"role": "user", "content": [
            {"type": "image", "source": {"type": "base64", "media_type": "image/png", "data": base64.b64encode(_png(32, 32, 1)).decode()}},
            {"type": "text", "text": "describe"}]}]})
        assert a.status_code == 200, a.text
        assert tower.encodes == 2
        bad = c.post("/v1/chat/completions", json={"model": "m", "messages": [{"role": "user", "content": [
            {"type": "image_url", "image_url": {"url": "https://example.com/cat.png"}}]}]})
        assert bad.status_code == 400 and "not fetched" in bad.text
    finally:
        loop.stop()


def test_vision_snapshot_round_trip(tmp_path):
    """`visual.*` tensors written the way checkpoints ship them (patch convolution with a temporal axis, gate / up / down MLP) read
    back into masters that give the same tower output."""
    import json

    from cuteafd_b200.loader.vision_checkpoint import read_vision_masters, vision_spec_from_snapshot, write_vision_snapshot
    for kw in (dict(pos_grid=3), dict(norm="rmsnorm", mlp="swiglu", qk_norm=True, qkv_bias=False)):
        spec = VisionSpec(hidden=32, depth=2, n_heads=2, head_dim=16, intermediate=48, patch=4, out_hidden=24, **kw)
        w = init_vision_weights(spec, 7)
        d = tmp_path / ("a" if "pos_grid" in kw else "b")
        d.mkdir()
        write_vision_snapshot(d / "model-vision.safetensors", spec, w)
        (d / "config.json").write_text(json.dumps({"hidden_size": 24, "image_token_id": 77, "vision_start_token_id": 78, "vision_end_token_id": 79,
            "vision_config": {"hidden_size": 32, "depth": 2, "num_heads": 2, "intermediate_size": 48, "patch_size": 4, "spatial_merge_size": 2,
                              "hidden_act": "silu" if spec.mlp == "swiglu" else "gelu", "qk_norm": spec.qk_norm,
                              "num_position_embeddings": spec.pos_grid ** 2}}))
        got_spec, ids = vision_spec_from_snapshot(d)
        assert ids == {"pad": 77, "start": 78, "end": 79}
        want = (32, 2, 16, spec.mlp, spec.norm, spec.pos_grid, 24)
        assert (got_spec.hidden, got_spec.depth, got_spec.head_dim, got_spec.mlp, got_spec.norm, got_spec.pos_grid, got_spec.out_hidden) == want
        back = read_vision_masters(d, got_spec)
        g = torch.Generator().manual_seed(1)
        p = rgb_to_patches(torch.randint(0, 256, (8, 8, 3), generator=g, dtype=torch.uint8), spec)
        a = vision_forward(spec, w, p, 2, 2)
        b = vision_forward(got_spec.replace(qkv_bias=spec.qkv_bias), back, p, 2, 2)
        assert torch.allclose(a, b, atol=1e-5)


def test_audio_oracle_front_end_and_im2col_weight_order():
    """The convolution-as-GEMM layout the device uses (operand columns (tap, channel)) reproduces F.conv1d in the oracle's arithmetic,
    and the mel front end gives whole groups of four frames."""
    import torch.nn.functional as F

    from cuteafd_b200.ref.audio import AudioSpec, audio_forward, init_audio_weights, log_mel, mel_filters
    spec = AudioSpec(hidden=32, depth=1, n_heads=2, head_dim=16, intermediate=48, out_hidden=24, n_mels=16)
    fb = mel_filters(spec)
    assert fb.shape == (16, 201) and (fb >= 0).all() and (fb.sum(dim=1) > 0).all()
    frames = log_mel(torch.randn(16000, generator=torch.Generator().manual_seed(0)), spec)
    assert frames.shape == (100, 16)
    w = init_audio_weights(spec, 1)
    out = audio_forward(spec, w, frames)
    assert out.shape == (25, 24) and torch.isfinite(out).all()
    # im2col with zero rows at both ends, columns (tap, channel), against conv1d with padding 1 and stride 2
    x = torch.randn(10, 32)
    pad = torch.cat([torch.zeros(1, 32), x, torch.zeros(1, 32)])
    rows = torch.stack([torch.cat([pad[2 * t + k] for k in range(3)]) for t in range(5)])
    wg = w["conv2_w"].permute(0, 2, 1).reshape(32, -1)
    want = F.conv1d(x.T[None], w["conv2_w"], None, stride=2, padding=1)[0].T
    assert torch.allclose(rows @ wg.T, want, atol=1e-5)


def test_chat_with_an_audio_clip_and_an_image_in_one_request():
    import base64
    import io
    import wave

    import numpy as np
    import pytest
    pytest.importorskip("fastapi")
    from fastapi.testclient import TestClient

    from cuteafd_b200.engine.kv import PagePool
    from cuteafd_b200.parallel.health import Health
    from cuteafd_b200.ref.audio import AudioSpec
    from cuteafd_b200.ref.vision import VisionSpec
    from cuteafd_b200.serving.api import ServingLoop, build_app
    from cuteafd_b200.serving.runner import FakeRunner
    from cuteafd_b200.serving.scheduler import Scheduler
    from cuteafd_b200.serving.vision import VisionFrontEnd

    class FakeAudio:
        device = None
        spec = AudioSpec(out_hidden=8, n_mels=16)
        encodes = 0

        def encode(self, clips):
            self.encodes += 1
            return [torch.ones(c.shape[0] // 4, 8, dtype=torch.bfloat16) for c in clips]

    buf = io.BytesIO()
    with wave.open(buf, "wb") as wf:
        wf.setnchannels(1); wf.setsampwidth(2); wf.setframerate(8000)          # resampled to 16 kHz by the loader
        wf.writeframes((np.sin(np.arange(8000) * 0.05) * 12000).astype("<i2").tobytes())
    tower, audio = _FakeTower(VisionSpec(patch=16, merge=2, out_hidden=8, max_tokens=64)), FakeAudio()
    runner = FakeRunner(vocab=96)
    runner.next_token = lambda prefix: 32 + (sum(prefix[-3:]) % 60)
    seen = []
    real_run = runner.run
    runner.run = lambda rows: (seen.extend((r.state.req.embeds, list(r.tokens)) for r in rows), real_run(rows))[1]
    loop = ServingLoop(Scheduler(runner, PagePool(256)), Health()).start()
    try:
        c = TestClient(build_app(loop, vision=VisionFrontEnd(tower, pad_id=90, start_id=91, end_id=92, audio_tower=audio, audio_pad_id=93,
                                                             audio_start_id=94, audio_end_id=95)))
        url = "data:image/png;base64," + base64.b64encode(_png(64, 64)).decode()
        r = c.post("/v1/chat/completions", json={"model": "m", "max_tokens": 3, "messages": [{"role": "user", "content": [
            {"type": "input_audio", "input_audio": {"data": base64.b64encode(buf.getvalue()).decode(), "format": "wav"}},
            {"type": "text", "text": " and "}, {"type": "image_url", "image_url": {"url": url}}]}]})
        assert r.status_code == 200, r.text
        emb, toks = next(s for s in seen if s[0] is not None)
        assert toks.count(93) == 25 and toks.count(90) == 4                     # 1 s of audio = 100 frames = 25 tokens; 64 x 64 px = 4 tokens
        assert toks.index(94) < toks.index(93) < toks.index(95) < toks.index(91) < toks.index(90)
        rows = emb["rows"].float()
        assert rows.shape == (29, 8) and bool((rows[:25] == 1).all()) and bool((rows[25:] == 0).all())      # prompt order: audio rows, then image rows
        assert [toks[p] for p in emb["positions"]] == [93] * 25 + [90] * 4
    finally:
        loop.stop()
