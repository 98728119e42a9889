"""End-to-end: the tiny MoE decoder on the GPU engine vs the fp32 CPU oracle (prefill 2x64, 16 greedy tokens)."""
import pytest
import torch

from cuteafd_b200.config import tiny_spec, QuantSpec
from cuteafd_b200.engine.engine import Engine
from cuteafd_b200.engine.generate import BatchGenerator, generate
from cuteafd_b200.models.weights import DeviceWeights
from cuteafd_b200.ref.model import RefModel, RefCache, init_weights

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _prompts(spec, n, length, seed=7):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, spec.vocab, (length,), generator=g).tolist() for _ in range(n)]


@pytest.mark.parametrize("experts", ["bf16", "nvfp4", "mxfp4"])
def test_tiny_model_matches_oracle(experts):
    spec = tiny_spec().replace(quant=QuantSpec(experts=experts, dense="bf16"))
    masters = init_weights(spec, 0)
    dw = DeviceWeights.from_masters(spec, masters, DEV)
    eng = Engine(dw, n_pages=32, max_seqs=8, max_pages_per_seq=4)
    prompts = _prompts(spec, 2, 64)
    # logits of the prefill's last row vs the oracle evaluated on the weights the kernels really use
    ref = RefModel(spec, dw.dequantized_masters())
    gen = BatchGenerator(eng)
    first = gen.prefill(prompts)
    lane = eng.lane(128)
    torch.cuda.synchronize()
    eng.check_status()
    tol = 0.05 if experts == "bf16" else 0.2
    for i, p in enumerate(prompts):
        rl, _ = ref.forward(torch.tensor(p), 0, RefCache())
        got = lane.logits[i].float().cpu()
        err = float((got - rl[-1]).norm() / rl[-1].norm())
        assert err < tol, f"prompt {i}: logits rel err {err}"
    gen.release()
    if experts == "bf16":
        out = generate(eng, prompts, 16)
        for i, p in enumerate(prompts):
            want, rows = ref.generate_greedy(torch.tensor(p), 16)
            # greedy tokens agree wherever the oracle's top-2 margin exceeds bf16 noise
            for j, (a, b) in enumerate(zip(out[i], want)):
                top2 = rows[j].topk(2).values
                if a != b:
                    assert float(top2[0] - top2[1]) < 0.05, f"prompt {i} step {j}: {a} != {b}"
                    break


def test_decode_graph_replay_matches_eager():
    spec = tiny_spec()
    dw = DeviceWeights.from_masters(spec, init_weights(spec, 1), DEV)
    eng = Engine(dw, n_pages=32, max_seqs=8, max_pages_per_seq=4)
    prompts = _prompts(spec, 3, 20)
    a = generate(eng, prompts, 8, use_graph=False)
    b = generate(eng, prompts, 8, use_graph=True)
    assert a == b
    assert eng.graph_captures >= 1


@pytest.mark.parametrize("head_dim,heads,kv", [(32, 8, 2), (128, 4, 2)])
def test_hybrid_full_and_sliding_window_stack_matches_oracle(head_dim, heads, kv):
    """MiMo-V2-style stack: layers 0, 2 are full causal attention, layers 1, 3 slide a 16-token window with per-head sinks and
    their own RoPE base.  Prompts longer than the window, on both attention kernels (SIMT for 32-wide heads, tcgen05 for 128)."""
    import dataclasses
    base = tiny_spec()
    spec = base.replace(n_layers=4, attn=dataclasses.replace(base.attn, n_heads=heads, n_kv_heads=kv, head_dim=head_dim, window=16, sink=True,
                                                             full_every=2, swa_rope_theta=5000.0))
    assert [spec.layer_window(i) for i in range(5)] == [0, 16, 0, 16, 0] and [spec.layer_has_sink(i) for i in range(4)] == [False, True, False, True]
    masters = init_weights(spec, 3)
    assert "sink" not in masters["layers"][0] and "sink" in masters["layers"][1]
    dw = DeviceWeights.from_masters(spec, masters, DEV)
    eng = Engine(dw, n_pages=32, max_seqs=8, max_pages_per_seq=4)
    ref = RefModel(spec, dw.dequantized_masters())
    prompts = _prompts(spec, 2, 50)
    gen = BatchGenerator(eng)
    gen.prefill(prompts)
    lane = eng.lane(100)
    torch.cuda.synchronize()
    eng.check_status()
    for i, p in enumerate(prompts):
        rl, _ = ref.forward(torch.tensor(p), 0, RefCache())
        got = lane.logits[i].float().cpu()
        assert float((got - rl[-1]).norm() / rl[-1].norm()) < 0.05
    gen.release()
    out = generate(eng, prompts, 10)
    for i, p in enumerate(prompts):
        want, rows = ref.generate_greedy(torch.tensor(p), 10)
        for j, (a, b) in enumerate(zip(out[i], want)):
            if a != b:
                top2 = rows[j].topk(2).values
                assert float(top2[0] - top2[1]) < 0.05, f"prompt {i} step {j}: {a} != {b}"
                break


def test_engine_passes_golden_windows(tmp_path):
    """The GPU engine's teacher-forced logits against golden windows sealed from the fp32 oracle; an engine with other weights fails."""
    from cuteafd_b200.bench.golden import check_logits, engine_logits_fn, write_golden
    spec = tiny_spec()
    masters = init_weights(spec, 0)
    gold = write_golden(str(tmp_path / "g.json"), spec, masters, n=4, length=40, tail=12, topk=6)
    eng = Engine(DeviceWeights.from_masters(spec, masters, DEV), n_pages=16, max_seqs=4, max_pages_per_seq=4)
    rep = check_logits(engine_logits_fn(eng), gold, spec=spec, max_rel_l2=0.05)
    assert rep["pass"], rep
    other = Engine(DeviceWeights.from_masters(spec, init_weights(spec, 3), DEV), n_pages=16, max_seqs=4, max_pages_per_seq=4)
    assert not check_logits(engine_logits_fn(other), gold, spec=spec)["pass"]


@pytest.mark.parametrize("per_channel", [False, True])
def test_hybrid_linear_attention_stack_matches_oracle(per_channel):
    """Hybrid stack: layers 0, 2 are gated delta-rule layers (GDN: decay per head; KDA: per key channel), layers 1, 3 full GQA.  The
    prompts are ingested in chunks (the recurrent state and the convolution history cross the chunk boundary), then decoded."""
    import dataclasses
    base = tiny_spec()
    spec = base.replace(n_layers=4, attn=dataclasses.replace(base.attn, n_heads=4, n_kv_heads=2, head_dim=128, linear_every=2, linear_k_heads=1,
                                                             linear_v_heads=2, linear_per_channel=per_channel))
    assert [spec.layer_is_linear(i) for i in range(4)] == [True, False, True, False]
    masters = init_weights(spec, 5)
    dw = DeviceWeights.from_masters(spec, masters, DEV)
    eng = Engine(dw, n_pages=32, max_seqs=8, max_pages_per_seq=4)
    ref = RefModel(spec, dw.dequantized_masters())
    prompts = _prompts(spec, 3, 50)
    gen = BatchGenerator(eng, prefill_chunk=32)
    gen.prefill(prompts)
    torch.cuda.synchronize()
    eng.check_status()
    gen.release()
    gen = BatchGenerator(eng)            # whole prompts in one step: logits of every prompt's last row sit in one lane
    gen.prefill(prompts)
    lane = eng.lane(150)
    torch.cuda.synchronize()
    eng.check_status()
    for i, p in enumerate(prompts):
        rl, _ = ref.forward(torch.tensor(p), 0, RefCache())
        got = lane.logits[i].float().cpu()
        err = float((got - rl[-1]).norm() / rl[-1].norm())
        assert err < 0.05, f"prompt {i}: logits rel err {err}"
    gen.release()
    for chunk in (4096, 32):             # chunked prefill must reach the same tokens as whole-prompt prefill
        g = BatchGenerator(eng, prefill_chunk=chunk)
        g.prefill(prompts)
        out = [[t] for t in g.last]
        for _ in range(9):
            for o, t in zip(out, g.decode_step(use_graph=(chunk == 32))):
                o.append(t)
        g.release()
        for i, p in enumerate(prompts):
            want, rows = ref.generate_greedy(torch.tensor(p), 10)
            for j, (a, b) in enumerate(zip(out[i], want)):
                if a != b:
                    top2 = rows[j].topk(2).values
                    assert float(top2[0] - top2[1]) < 0.05, f"chunk {chunk} prompt {i} step {j}: {a} != {b}"
                    break


def test_mhc_boundary_kernel_matches_oracle():
    """One hyper-connection boundary: spread the embedding (init), open; then close with a sub-layer output and re-open; then the head's
    collapse.  Coefficients, streams and the normalised collapse against the fp32 oracle; a cluster per token, one and two rows per CTA."""
    from cuteafd_b200.ops import native
    from cuteafd_b200.ops.native import ptr
    from cuteafd_b200.ref import ops as rops
    g = torch.Generator().manual_seed(0)
    for T, H in ((5, 256), (300, 256), (600, 512), (3, 7168), (16, 4096)):
        W = 4 * H
        emb = (torch.randn(T, H, generator=g) * 0.5).to(torch.bfloat16)
        sub = (torch.randn(T, H, generator=g) * 0.3).to(torch.bfloat16)
        fns = [torch.randn(24, W, generator=g) * (2.0 / W ** 0.5) for _ in range(2)] + [torch.randn(4, W, generator=g) * (2.0 / W ** 0.5)]
        scale = torch.tensor([0.5, 0.7, 0.9])
        bases = [torch.randn(24, generator=g) * 0.5, torch.randn(24, generator=g) * 0.5, torch.randn(4, generator=g) * 0.5]
        nw = torch.rand(H, generator=g) + 0.5
        d = lambda t: t.to(DEV).contiguous()
        res, coef = torch.zeros(T, 4, H, dtype=torch.bfloat16, device=DEV), torch.zeros(T, 20, device=DEV)
        y_raw, y_norm = torch.zeros(T, H, dtype=torch.bfloat16, device=DEV), torch.zeros(T, H, dtype=torch.bfloat16, device=DEV)
        emb_d, sub_d, scale_d, nw_d = d(emb), d(sub), d(scale), d(nw)
        fn_d, base_d = [d(f) for f in fns], [d(b) for b in bases]
        b16 = lambda t: t.to(torch.bfloat16).float()

        def check(r_want, pre, post, comb, n_proj):
            y = (pre[:, :, None] * r_want).sum(1)
            want = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + 1e-5) * nw
            torch.cuda.synchronize()
            assert torch.equal(res.float().cpu(), r_want) or float((res.float().cpu() - r_want).abs().max()) < 0.02
            assert float((y_norm.float().cpu() - want).norm() / want.norm()) < 0.01
            if n_proj == 24:
                got = coef.cpu()
                assert float((got[:, :4] - post).abs().max()) < 2e-3 and float((got[:, 4:].reshape(T, 4, 4) - comb).abs().max()) < 2e-3

        # 1: init + open
        native.call("cuteafd_mhc_boundary", ptr(res), ptr(emb_d), None, ptr(fn_d[0]), ptr(scale_d), ptr(base_d[0]), ptr(nw_d), None, ptr(y_norm), ptr(coef),
                    T, H, 24, 1, 20, 1e-5, native.stream())
        r0 = emb.float()[:, None, :].expand(-1, 4, -1).contiguous()
        pre, post, comb = rops.mhc_mixes(r0, fns[0], scale, bases[0])
        check(r0, pre, post, comb, 24)
        # 2: close with `sub`, re-open
        native.call("cuteafd_mhc_boundary", ptr(res), ptr(sub_d), ptr(coef), ptr(fn_d[1]), ptr(scale_d), ptr(base_d[1]), ptr(nw_d), None, ptr(y_norm), ptr(coef),
                    T, H, 24, 0, 20, 1e-5, native.stream())
        r1 = b16(rops.mhc_close(r0, sub.float(), post, comb))
        pre, post, comb = rops.mhc_mixes(r1, fns[1], scale, bases[1])
        check(r1, pre, post, comb, 24)
        # 3: close, head collapse (4 projections), un-normalised rows too
        native.call("cuteafd_mhc_boundary", ptr(res), ptr(sub_d), ptr(coef), ptr(fn_d[2]), ptr(scale_d), ptr(base_d[2]), ptr(nw_d), ptr(y_raw), ptr(y_norm), None,
                    T, H, 4, 0, 20, 1e-5, native.stream())
        r2 = b16(rops.mhc_close(r1, sub.float(), post, comb))
        pre, _, _ = rops.mhc_mixes(r2, fns[2], scale, bases[2])
        check(r2, pre, None, None, 4)
        y = (pre[:, :, None] * r2).sum(1)
        assert float((y_raw.float().cpu() - y).norm() / y.norm()) < 0.01


def test_hyper_connection_stack_matches_oracle():
    """Tiny model with four residual streams (hyper-connections around every sub-layer): prefill logits and greedy decode vs the oracle."""
    spec = tiny_spec().replace(n_layers=3, hyper_streams=4)
    masters = init_weights(spec, 6)
    dw = DeviceWeights.from_masters(spec, masters, DEV)
    eng = Engine(dw, n_pages=32, max_seqs=8, max_pages_per_seq=4)
    ref = RefModel(spec, dw.dequantized_masters())
    prompts = _prompts(spec, 2, 40)
    gen = BatchGenerator(eng)
    gen.prefill(prompts)
    lane = eng.lane(80)
    torch.cuda.synchronize()
    eng.check_status()
    for i, p in enumerate(prompts):
        rl, _ = ref.forward(torch.tensor(p), 0, RefCache())
        got = lane.logits[i].float().cpu()
        err = float((got - rl[-1]).norm() / rl[-1].norm())
        assert err < 0.05, f"prompt {i}: logits rel err {err}"
    gen.release()
    out = generate(eng, prompts, 10)
    for i, p in enumerate(prompts):
        want, rows = ref.generate_greedy(torch.tensor(p), 10)
        for j, (a, b) in enumerate(zip(out[i], want)):
            if a != b:
                top2 = rows[j].topk(2).values
                assert float(top2[0] - top2[1]) < 0.05, f"prompt {i} step {j}: {a} != {b}"
                break


@pytest.mark.parametrize("variant", ["layernorm-gelu-pos", "rmsnorm-swiglu-qknorm"])
def test_vision_tower_matches_oracle(variant):
    """ViT encoder (bf16 tcgen05 GEMMs, bidirectional attention over heads padded to 128, fused glue) against the fp32 oracle:
    two images of different grids in one batch; patch width 14 exercises the padded patch rows."""
    from cuteafd_b200.models.vision import VisionTower
    from cuteafd_b200.ref.vision import VisionSpec, init_vision_weights, rgb_to_patches, vision_bf16_round, vision_forward
    if variant == "layernorm-gelu-pos":
        spec = VisionSpec(hidden=128, depth=2, n_heads=2, head_dim=64, intermediate=192, patch=14, out_hidden=256, pos_grid=6)
    else:
        spec = VisionSpec(hidden=192, depth=2, n_heads=4, head_dim=48, intermediate=256, patch=16, out_hidden=128, norm="rmsnorm", mlp="swiglu",
                          qk_norm=True, qkv_bias=False)
    w = vision_bf16_round(init_vision_weights(spec, 3))
    tower = VisionTower(spec, w, DEV, max_patches=1024, max_images=4)
    g = torch.Generator().manual_seed(5)
    P = spec.patch
    images = [torch.randint(0, 256, (gh * P, gw * P, 3), generator=g, dtype=torch.uint8) for gh, gw in ((12, 16), (6, 4))]
    outs = tower.encode(images)
    torch.cuda.synchronize()
    for im, got in zip(images, outs):
        gh, gw = im.shape[0] // P, im.shape[1] // P
        want = vision_forward(spec, w, rgb_to_patches(im, spec).bfloat16().float(), gh, gw)
        assert got.shape == want.shape
        err = float((got.float().cpu() - want).norm() / want.norm())
        assert err < 0.03, f"{variant}: {gh}x{gw} rel err {err}"
    # a second call reuses the buffers and the scratch store: same rows for the same image alone
    again = tower.encode([images[1]])[0]
    assert float((again.float() - outs[1].float()).abs().max()) < 2e-2


def test_audio_tower_matches_oracle():
    """Audio encoder (convolution front end as GEMMs over im2col rows, shared encoder blocks without rotation, two-frame mean folded
    into the projection GEMM) against the fp32 oracle: two clips of different lengths in one batch."""
    from cuteafd_b200.models.audio import AudioTower
    from cuteafd_b200.ref.audio import AudioSpec, audio_bf16_round, audio_forward, init_audio_weights, log_mel
    spec = AudioSpec(hidden=128, depth=2, n_heads=2, head_dim=64, intermediate=256, out_hidden=192, n_mels=64)
    w = audio_bf16_round(init_audio_weights(spec, 4))
    tower = AudioTower(spec, w, DEV, max_frames=2048, max_clips=4)
    g = torch.Generator().manual_seed(9)
    clips = [log_mel(torch.randn(n, generator=g) * 0.3, spec) for n in (16000 * 3, 16000)]
    outs = tower.encode(clips)
    torch.cuda.synchronize()
    for f, got in zip(clips, outs):
        want = audio_forward(spec, w, f.bfloat16().float())
        assert got.shape == want.shape == (f.shape[0] // 4, 192)
        err = float((got.float().cpu() - want).norm() / want.norm())
        assert err < 0.03, f"{f.shape[0]} frames: rel err {err}"
