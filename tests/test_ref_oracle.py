"""CPU oracle self-consistency (mirrors the reference's python/reference/tests: rmsnorm, rope, router,
moe, chunked == unchunked prefill, KV boundaries, MTP verify, nibble packing, NVFP4 fixtures)."""
import numpy as np
import pytest
import torch

from cuteafd_b200.config import tiny_spec, deepseek_v3_spec, AttentionSpec, MoESpec, ModelSpec
from cuteafd_b200.ref import ops, quant, sampler, exl3
from cuteafd_b200.ref.model import RefModel, RefCache, init_weights


def test_rmsnorm_matches_definition():
    x = torch.randn(5, 64)
    w = torch.randn(64)
    y = ops.rmsnorm(x, w, 1e-5)
    ref = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w
    assert torch.allclose(y, ref, atol=1e-6)


@pytest.mark.parametrize("interleaved", [True, False])
def test_rope_is_a_rotation_and_relative(interleaved):
    q = torch.randn(4, 2, 32)
    k = torch.randn(4, 2, 32)
    p = torch.tensor([3, 4, 10, 11])
    rq, rk = ops.apply_rope(q, p, interleaved=interleaved), ops.apply_rope(k, p, interleaved=interleaved)
    assert torch.allclose(rq.norm(dim=-1), q.norm(dim=-1), atol=1e-5)
    rq2, rk2 = ops.apply_rope(q, p + 7, interleaved=interleaved), ops.apply_rope(k, p + 7, interleaved=interleaved)
    assert torch.allclose((rq * rk).sum(-1), (rq2 * rk2).sum(-1), atol=1e-4)


def test_router_topk_normalised_and_bias_only_affects_choice():
    h = torch.randn(6, 32)
    w = torch.randn(16, 32)
    idx, wt = ops.route_topk(h, w, 4, "sigmoid", True)
    assert torch.allclose(wt.sum(-1), torch.ones(6), atol=1e-6)
    bias = torch.zeros(16)
    bias[5] = 100.0
    idx2, wt2 = ops.route_topk(h, w, 4, "sigmoid", False, bias=bias)
    assert (idx2[:, 0] == 5).all()
    assert torch.allclose(wt2[:, 0], torch.sigmoid(h @ w.T)[:, 5], atol=1e-6)


def test_group_limited_routing_stays_in_groups():
    h, w = torch.randn(8, 32), torch.randn(16, 32)
    idx, _ = ops.route_topk(h, w, 4, "sigmoid", True, n_group=4, topk_group=2)
    assert (torch.tensor([len(set((r // 4).tolist())) for r in idx]) <= 2).all()


def test_moe_forward_equals_per_row_loop():
    torch.manual_seed(0)
    x = torch.randn(5, 16)
    wg, wu, wd = torch.randn(4, 8, 16), torch.randn(4, 8, 16), torch.randn(4, 16, 8)
    idx, wt = ops.route_topk(x, torch.randn(4, 16), 2)
    y = ops.moe_forward(x, wg, wu, wd, idx, wt)
    ref = torch.zeros_like(x)
    for r in range(5):
        for s in range(2):
            e = int(idx[r, s])
            ref[r] += wt[r, s] * ops.expert_ffn(x[r:r + 1], wg[e], wu[e], wd[e])[0]
    assert torch.allclose(y, ref, atol=1e-5)


def test_chunked_prefill_equals_unchunked_and_decode_matches_full():
    spec = tiny_spec()
    m = RefModel(spec, init_weights(spec, 1))
    toks = torch.randint(0, spec.vocab, (24,), generator=torch.Generator().manual_seed(2))
    full, _ = m.forward(toks, 0, RefCache())
    chunked, _ = m.forward(toks, 0, RefCache(), chunk=7)
    assert torch.allclose(full, chunked, atol=1e-4)
    cache = RefCache()
    m.forward(toks[:20], 0, cache)
    for i in range(20, 24):
        step, _ = m.forward(toks[i:i + 1], i, cache)
        assert torch.allclose(step[0], full[i], atol=1e-4)


def test_mla_oracle_runs_and_is_causal():
    spec = ModelSpec(vocab=128, hidden=64, n_layers=2,
                     attn=AttentionSpec(kind="mla", n_heads=4, n_kv_heads=4, head_dim=24, q_lora_rank=32,
                                        kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16),
                     moe=MoESpec(n_experts=8, top_k=2, intermediate=32, first_dense=1, dense_intermediate=64),
                     mtp_layers=1)
    m = RefModel(spec, init_weights(spec, 3))
    toks = torch.randint(0, 128, (10,))
    a, _ = m.forward(toks, 0, RefCache())
    toks2 = toks.clone()
    toks2[7] = (toks2[7] + 1) % 128
    b, _ = m.forward(toks2, 0, RefCache())
    assert torch.allclose(a[:7], b[:7], atol=1e-5) and not torch.allclose(a[7:], b[7:], atol=1e-5)


def test_speculative_generation_is_lossless():
    spec = tiny_spec().replace(mtp_layers=1)
    m = RefModel(spec, init_weights(spec, 5))
    prompt = torch.randint(0, spec.vocab, (12,), generator=torch.Generator().manual_seed(9))
    greedy, _ = m.generate_greedy(prompt, 12)
    spec_out, acc = m.generate_speculative(prompt, 12, n_draft=3)
    assert spec_out == greedy
    assert all(0 <= a <= 3 for a in acc)


def test_greedy_verify_protocol():
    assert ops.greedy_verify([5, 6, 7, 8], [6, 7, 9, 1], None, 100) == (3, [6, 7, 9], False, False)
    assert ops.greedy_verify([5, 6], [6, 7], None, 100) == (2, [6, 7], False, False)
    assert ops.greedy_verify([5, 6, 7], [6, 2, 9], 2, 100)[2] is True
    assert ops.greedy_verify([5, 6, 7], [6, 7, 9], None, 2) == (3, [6, 7], False, True)


# ---- formats -------------------------------------------------------------
def test_e4m3_roundtrip_all_codes():
    codes = torch.tensor([c for c in range(256) if (c & 0x7F) != 0x7F], dtype=torch.uint8)
    vals = quant.e4m3_decode(codes)
    back = quant.e4m3_encode(vals)
    assert torch.equal(quant.e4m3_decode(back), vals)
    assert float(quant.e4m3_decode(quant.e4m3_encode(torch.tensor([1e6])))) == 448.0


def test_e2m1_encode_nearest_even_and_pack():
    x = torch.tensor([0.0, 0.24, 0.25, 0.26, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.75, -6.0])
    c = quant.e2m1_encode(x)
    assert quant.e2m1_decode(c).tolist() == [0.0, 0.0, 0.0, 0.5, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -1.0, -6.0]
    codes = torch.randint(0, 16, (3, 64), dtype=torch.uint8)
    assert torch.equal(quant.unpack_nibbles(quant.pack_nibbles(codes)), codes)


def test_mxfp4_and_nvfp4_quantisation_error_bounds():
    w = torch.randn(8, 256) * 0.02
    p, s = quant.mxfp4_quantize(w)
    assert p.shape == (8, 128) and s.shape == (8, 8)
    err = (quant.mxfp4_dequantize(p, s) - w).abs().max() / w.abs().max()
    assert err < 0.3
    p, s, g = quant.nvfp4_quantize(w)
    assert s.shape == (8, 16)
    rel = (quant.nvfp4_dequantize(p, s, g) - w).norm() / w.norm()
    assert rel < 0.12
    # exactly representable tensors survive
    exact = quant.nvfp4_dequantize(p, s, g)
    p2, s2, _ = quant.nvfp4_quantize(exact, g)
    assert torch.allclose(quant.nvfp4_dequantize(p2, s2, g), exact, rtol=1e-6, atol=0)


def test_fp8_block_and_wire_rows():
    w = torch.randn(130, 260)
    q, s = quant.fp8_block_quantize(w)
    assert s.shape == (2, 3)
    assert (quant.fp8_block_dequantize(q, s) - w).abs().max() < 0.07 * w.abs().max()
    x = torch.randn(4, 128)
    q, sb = quant.act_quant_fp8_ue8m0(x)
    deq = quant.act_dequant_fp8_ue8m0(q, sb)
    assert (deq - x).abs().max() < 0.07 * x.abs().max()
    assert (quant.e4m3_decode(q).abs() <= 448).all()


def test_sf_swizzle_roundtrip_and_known_offsets():
    sf = torch.arange(130 * 6, dtype=torch.int32).remainder(251).to(torch.uint8).reshape(130, 6)
    flat = quant.swizzle_sf_128x4(sf)
    assert flat.numel() == 2 * 2 * 512
    assert torch.equal(quant.unswizzle_sf_128x4(flat, 130, 6), sf)
    # row 33 (r%32=1, r//32=1), sf index 5 (chunk 1, s=1) of row-block 0
    assert int(flat[1 * 512 + 1 * 16 + 1 * 4 + 1]) == int(sf[33, 5])


# ---- sampler ---------------------------------------------------------------
def test_sampler_chain_and_determinism():
    torch.manual_seed(0)
    logits = torch.randn(1000)
    p = sampler.SamplingParams(temperature=0.8, top_p=0.9, top_k=50, min_p=0.01, seed=1234).validate()
    order, probs = sampler.candidate_set(logits, p)
    assert order.numel() <= 50 and abs(float(probs.sum()) - 1) < 1e-5
    assert int(order[0]) == int(logits.argmax())
    a = [sampler.sample(logits, p, pos) for pos in range(20)]
    b = [sampler.sample(logits, p, pos) for pos in range(20)]
    assert a == b and len(set(a)) > 1
    assert sampler.sample(logits, sampler.SamplingParams(), 0) == int(logits.argmax())
    mask = torch.zeros(1000, dtype=torch.bool)
    mask[[3, 7]] = True
    assert sampler.sample(logits, p, 5, mask) in (3, 7)
    with pytest.raises(ValueError):
        sampler.sample(logits, p, 5, torch.zeros(1000, dtype=torch.bool))


def test_uniform_is_uniform_enough():
    us = np.array([sampler.uniform_from(42, i) for i in range(4000)])
    assert 0.47 < us.mean() < 0.53 and us.max() <= sampler.MAX_UNIFORM and us.min() >= 0


# ---- EXL3 ------------------------------------------------------------------
@pytest.mark.parametrize("bits", [2, 3, 4, 5])
def test_exl3_pack_unpack_and_decode(bits):
    rng = np.random.default_rng(bits)
    sym = rng.integers(0, 1 << bits, size=(2, 3, 256)).astype(np.uint32)
    words = exl3.pack_symbols(sym, bits)
    assert words.shape == (2, 3, 16 * bits) and words.dtype == np.uint16
    assert np.array_equal(exl3.unpack_symbols(words, bits), sym)
    inner = exl3.decode_tiles(words)
    assert inner.shape == (32, 48) and np.isfinite(inner).all()


def test_exl3_greedy_encoder_tracks_target_and_hadamard_is_orthonormal():
    rng = np.random.default_rng(0)
    target = rng.standard_normal((128, 128)).astype(np.float32)
    tr = exl3.encode_tiles_greedy(target, 4)
    dec = exl3.decode_tiles(tr)
    assert np.corrcoef(dec.ravel(), target.ravel())[0, 1] > 0.9
    x = rng.standard_normal((3, 256))
    assert np.allclose(exl3.hadamard128(exl3.hadamard128(x)), x, atol=1e-10)
    w = exl3.dequantize(tr, np.ones(128), np.ones(128))
    assert w.shape == (128, 128)


def test_hybrid_layer_pattern_facts_and_config_detection():
    """Full / sliding-window layer pattern: per-layer window, sink and RoPE base, read from a MiMo-V2-style config."""
    import dataclasses
    from cuteafd_b200.config import from_hf_config, tiny_spec
    base = tiny_spec()
    spec = base.replace(n_layers=6, attn=dataclasses.replace(base.attn, window=8, sink=True, full_every=3, swa_rope_theta=777.0))
    assert [spec.layer_is_full(i) for i in range(7)] == [True, False, False, True, False, False, True]
    assert spec.layer_rope_theta(0) == base.attn.rope_theta and spec.layer_rope_theta(1) == 777.0
    cfg = {"architectures": ["MiMoV2FlashForCausalLM"], "hidden_size": 256, "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 32,
           "num_hidden_layers": 6, "vocab_size": 100, "hybrid_layer_pattern": [0, 1, 1, 0, 1, 1], "sliding_window_size": 128,
           "rope_theta": 5e6, "swa_rope_theta": 1e4, "n_routed_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 64,
           "scoring_func": "sigmoid"}
    s = from_hf_config(cfg)
    assert s.family == "mimo_v2" and s.attn.full_every == 3 and s.attn.window == 128 and s.attn.sink and s.attn.swa_rope_theta == 1e4
    import pytest
    with pytest.raises(ValueError):
        from_hf_config(dict(cfg, hybrid_layer_pattern=[0, 1, 0, 0, 1, 1]))
    # the window changes what the oracle computes beyond its length, and only in the sliding layers
    import torch
    from cuteafd_b200.ref.model import RefCache, RefModel, init_weights
    small = base.replace(n_layers=2, attn=dataclasses.replace(base.attn, window=4, sink=True, full_every=2))
    w = init_weights(small, 1)
    toks = torch.arange(12) % small.vocab
    a, _ = RefModel(small, w).forward(toks, 0, RefCache())
    full = small.replace(attn=dataclasses.replace(small.attn, window=0, full_every=0, sink=False))
    w2 = {**w, "layers": [{k: v for k, v in l.items() if k != "sink"} for l in w["layers"]]}
    b, _ = RefModel(full, w2).forward(toks, 0, RefCache())
    assert not torch.allclose(a[-1], b[-1], atol=1e-4)


def test_compressor_pooling_is_chunk_invariant_and_softmax_weighted():
    import torch

    from cuteafd_b200.ref.ops import compress_pool
    g = torch.Generator().manual_seed(0)
    kv, sc, w = torch.randn(23, 64, generator=g), torch.randn(23, 64, generator=g) * 2, 1 + 0.1 * torch.randn(64, generator=g)
    rows, state = compress_pool(kv, sc, 4, w, 1e-6)
    assert rows.shape == (5, 64) and state is not None                      # 23 = 5 blocks of 4 + 3 open positions
    # block 1, channel 7, by hand
    p = torch.softmax(sc[4:8, 7], 0)
    pooled = (p * kv[4:8, 7]).sum()
    full = torch.stack([(torch.softmax(sc[4:8, d], 0) * kv[4:8, d]).sum() for d in range(64)]).bfloat16().float()
    assert abs(float(full[7]) - float(pooled.bfloat16())) < 1e-6
    assert torch.allclose(rows[1], full * torch.rsqrt(full.pow(2).mean() + 1e-6) * w, atol=1e-5)
    # the same rows when the positions arrive as 6 + 1 + 1 + 15
    got, st, pos = [], None, 0
    for n in (6, 1, 1, 15):
        r, st = compress_pool(kv[pos:pos + n], sc[pos:pos + n], 4, w, 1e-6, pos0=pos, state=st)
        got.append(r)
        pos += n
    assert torch.allclose(torch.cat(got), rows, atol=1e-5) and torch.allclose(st, state, atol=1e-5)
