"""DeepSeek-V3-shape attention (MLA, absorbed, tcgen05 kernel) end to end against the fp32 oracle on a small model
with the real head geometry (nope 128, rope 64, v 128, latent 512)."""
import pytest
import torch

from cuteafd_b200.config import AttentionSpec, ModelSpec, MoESpec, QuantSpec
from cuteafd_b200.engine.generate import BatchGenerator, generate
from cuteafd_b200.engine.mla import MlaEngine, mla_weights_from_masters
from cuteafd_b200.ref.model import RefCache, RefModel, init_weights

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def small_mla_spec(n_heads=4, q_lora=64):
    return ModelSpec(name="mla-small", family="deepseek_v3", vocab=512, hidden=256, n_layers=2, rms_eps=1e-6,
                     attn=AttentionSpec(kind="mla", n_heads=n_heads, n_kv_heads=n_heads, head_dim=192, q_lora_rank=q_lora, kv_lora_rank=512,
                                        qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128),
                     moe=MoESpec(n_experts=8, top_k=2, intermediate=128, n_shared=1, scoring="sigmoid", use_bias=True, n_group=4, topk_group=2,
                                 route_scale=2.5, first_dense=1, dense_intermediate=256),
                     quant=QuantSpec(experts="bf16", dense="bf16"))


def bf16_round(tree):
    if isinstance(tree, torch.Tensor):
        return tree.to(torch.bfloat16).float() if tree.dim() >= 2 else tree
    if isinstance(tree, dict):
        return {k: bf16_round(v) for k, v in tree.items()}
    if isinstance(tree, list):
        return [bf16_round(v) for v in tree]
    return tree


@pytest.mark.parametrize("n_heads,q_lora", [(4, 64), (16, 0)])
def test_mla_engine_matches_oracle(n_heads, q_lora):
    spec = small_mla_spec(n_heads, q_lora)
    masters = bf16_round(init_weights(spec, 0))
    dw = mla_weights_from_masters(spec, masters, DEV)
    eng = MlaEngine(dw, n_pages=32, max_seqs=8, max_pages_per_seq=6)
    ref = RefModel(spec, masters)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, spec.vocab, (n,), generator=g).tolist() for n in (70, 33)]
    gen = BatchGenerator(eng)
    gen.prefill(prompts)
    torch.cuda.synchronize()
    eng.check_status()
    lane = eng.lane(sum(len(p) for p in prompts))
    for i, p in enumerate(prompts):
        rl, _ = ref.forward(torch.tensor(p), 0, RefCache())
        got = lane.logits[i].float().cpu()
        err = float((got - rl[-1]).norm() / rl[-1].norm())
        assert err < 0.06, f"prompt {i}: logits rel err {err}"
    # decode steps (split-KV path) keep tracking the oracle
    for _ in range(3):
        toks = gen.decode_step(use_graph=False)
    torch.cuda.synchronize()
    eng.check_status()
    gen.release()
    out = generate(eng, prompts, 6)
    for i, p in enumerate(prompts):
        want, rows = ref.generate_greedy(torch.tensor(p), 6)
        for j, (a_, b_) in enumerate(zip(out[i], want)):
            if a_ != b_:
                top2 = rows[j].topk(2).values
                assert float(top2[0] - top2[1]) < 0.05, f"prompt {i} step {j}: {a_} != {b_}"
                break


def test_mla_prefill_kernel_matches_fp32_reference():
    """The non-absorbed prefill kernel against a plain PyTorch fp32 causal attention of the same operands: two sequences with
    different chunk offsets (a cached prefix before the query chunk), a ragged last query tile and a ragged last key tile."""
    from cuteafd_b200.ops.native import call, ptr, stream
    torch.manual_seed(3)
    Hl = 3
    q_lens, kv_lens = [200, 77], [200 + 150, 77]
    T = sum(q_lens)
    starts, tot = [], 0
    for n in kv_lens:
        starts.append(tot)
        tot += -(-n // 64) * 64
    rows = tot + 64
    q_nope = (torch.randn(Hl, T, 128, device=DEV) * 0.5).to(torch.bfloat16)
    q_rope = (torch.randn(T, Hl, 64, device=DEV) * 0.5).to(torch.bfloat16)
    kvb = torch.randn(rows, Hl * 256, device=DEV).to(torch.bfloat16)
    lat = torch.randn(rows, 576, device=DEV).to(torch.bfloat16)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    q_start = [0, q_lens[0]]
    out = torch.zeros(T, Hl * 128, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    scale = 192 ** -0.5
    d_starts, d_kv, d_qs, d_ql = i32(starts), i32(kv_lens), i32(q_start), i32(q_lens)      # held: a temporary would be recycled by the allocator
    call("cuteafd_mla_prefill_attention", ptr(q_nope), ptr(q_rope), ptr(kvb), ptr(lat), rows, ptr(d_starts), ptr(d_kv), ptr(d_qs),
         ptr(d_ql), ptr(out), T, 2, max(q_lens), Hl, scale, ptr(status), stream())
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    for s in range(2):
        ql, kl, c0, t0 = q_lens[s], kv_lens[s], starts[s], q_start[s]
        k_rope = lat[c0:c0 + kl, 512:].float()
        pos_q = torch.arange(kl - ql, kl, device=DEV)
        mask = torch.arange(kl, device=DEV)[None, :] <= pos_q[:, None]
        for h in range(Hl):
            k = torch.cat([kvb[c0:c0 + kl, h * 256:h * 256 + 128].float(), k_rope], dim=1)
            v = kvb[c0:c0 + kl, h * 256 + 128:h * 256 + 256].float()
            q = torch.cat([q_nope[h, t0:t0 + ql].float(), q_rope[t0:t0 + ql, h].float()], dim=1)
            sc = (q @ k.T) * scale
            p = torch.softmax(sc.masked_fill(~mask, float("-inf")), dim=-1)
            want = p @ v
            got = out[t0:t0 + ql, h * 128:(h + 1) * 128].float()
            err = float((got - want).norm() / want.norm())
            assert err < 0.02, f"seq {s} head {h}: rel err {err}"


def test_mla_engine_prefill_path_matches_oracle():
    """A prompt long enough for the non-absorbed prefill path (chunked: the second chunk attends over a cached prefix), then
    decode steps through the absorbed kernel over the same cache."""
    spec = small_mla_spec(4, 64)
    masters = bf16_round(init_weights(spec, 0))
    dw = mla_weights_from_masters(spec, masters, DEV)
    eng = MlaEngine(dw, n_pages=32, max_seqs=4, max_pages_per_seq=8)
    ref = RefModel(spec, masters)
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, spec.vocab, (n,), generator=g).tolist() for n in (300, 140)]
    used = []
    orig = MlaEngine._prefill_attention

    def spy(self, *a, **k):
        used.append(1)
        return orig(self, *a, **k)
    MlaEngine._prefill_attention = spy
    try:
        gen = BatchGenerator(eng, prefill_chunk=160)          # steps of 160 rows, 140 + 20 rows (over a cached prefix), 120 rows (absorbed path)
        out = [[t] for t in gen.prefill(prompts)]
    finally:
        MlaEngine._prefill_attention = orig
    for _ in range(4):
        for o, t in zip(out, gen.decode_step(use_graph=False)):
            o.append(t)
    torch.cuda.synchronize()
    eng.check_status()
    gen.release()
    assert len(used) == 2 * spec.n_layers, "the prefill path runs for the two steps whose longest query run reaches 128 rows"
    for i, p in enumerate(prompts):
        want, rows = ref.generate_greedy(torch.tensor(p), 5)
        for j, (a_, b_) in enumerate(zip(out[i], want)):
            if a_ != b_:
                top2 = rows[j].topk(2).values
                assert float(top2[0] - top2[1]) < 0.05, f"prompt {i} step {j}: {a_} != {b_}"
                break


def test_mla_engine_with_hyper_connections_matches_oracle():
    """Latent attention under four residual streams (the V4 line's pairing): prefill logits and greedy decode against the oracle."""
    spec = small_mla_spec(4, 64).replace(hyper_streams=4)
    masters = bf16_round(init_weights(spec, 2))
    eng = MlaEngine(mla_weights_from_masters(spec, masters, DEV), n_pages=32, max_seqs=8, max_pages_per_seq=6)
    ref = RefModel(spec, masters)
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, spec.vocab, (n,), generator=g).tolist() for n in (40, 21)]
    gen = BatchGenerator(eng)
    gen.prefill(prompts)
    torch.cuda.synchronize()
    eng.check_status()
    lane = eng.lane(sum(len(p) for p in prompts))
    for i, p in enumerate(prompts):
        rl, _ = ref.forward(torch.tensor(p), 0, RefCache())
        got = lane.logits[i].float().cpu()
        err = float((got - rl[-1]).norm() / rl[-1].norm())
        assert err < 0.06, f"prompt {i}: logits rel err {err}"
    gen.release()
    out = generate(eng, prompts, 6)
    for i, p in enumerate(prompts):
        want, rows = ref.generate_greedy(torch.tensor(p), 6)
        for j, (a_, b_) in enumerate(zip(out[i], want)):
            if a_ != b_:
                top2 = rows[j].topk(2).values
                assert float(top2[0] - top2[1]) < 0.05, f"prompt {i} step {j}: {a_} != {b_}"
                break
