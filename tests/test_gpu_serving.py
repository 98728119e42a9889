"""The serving stack on the real engine: scheduler + EngineRunner + prefix cache + n-gram speculation must reproduce
plain greedy generation exactly (prefix-restore exactness and lossless speculation gates), and sampling is a pure
function of (seed, position)."""
import pytest
import torch

from cuteafd_b200.config import tiny_spec
from cuteafd_b200.engine.engine import Engine
from cuteafd_b200.engine.generate import generate
from cuteafd_b200.engine.kv import PagePool
from cuteafd_b200.models.weights import DeviceWeights
from cuteafd_b200.ref.model import init_weights
from cuteafd_b200.ref.sampler import SamplingParams
from cuteafd_b200.serving.prefix import PrefixCache
from cuteafd_b200.serving.runner import EngineRunner, attach_pool
from cuteafd_b200.serving.scheduler import NgramDrafter, Request, Scheduler

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def build(drafter=None, prefix=True, n_pages=64):
    spec = tiny_spec()
    eng = Engine(DeviceWeights.from_masters(spec, init_weights(spec, 2), DEV), n_pages=n_pages, max_seqs=8, max_pages_per_seq=8)
    pool = PagePool(n_pages)
    runner = attach_pool(EngineRunner(eng, max_rows=256), pool)
    cache = PrefixCache(pool, min_tokens=64) if prefix else None
    return spec, eng, Scheduler(runner, pool, max_seqs=4, prefill_chunk=96, prefix=cache, drafter=drafter), cache


def run_requests(sched, prompts, n_new, **kw):
    res = {}
    for i, p in enumerate(prompts):
        def cb(toks, done, reason, i=i):
            res.setdefault(i, []).extend(toks)
        sched.submit(Request(f"r{i}", p, max_tokens=n_new, on_token=cb, **kw))
    sched.run_until_idle()
    return [res[i] for i in range(len(prompts))]


def test_scheduler_on_engine_matches_plain_generation_with_prefix_reuse_and_speculation():
    spec, eng, sched, cache = build(drafter=NgramDrafter())
    g = torch.Generator().manual_seed(11)
    shared = torch.randint(0, spec.vocab, (130,), generator=g).tolist()
    prompts = [shared + torch.randint(0, spec.vocab, (n,), generator=g).tolist() for n in (5, 17, 9)]
    _, ref_eng, _, _ = build(prefix=False)
    want = generate(ref_eng, prompts, 12, use_graph=False)
    got_cold = run_requests(sched, prompts[:1], 12)
    got_warm = run_requests(sched, prompts[1:], 12)              # these restore the 128-token shared prefix from the cache
    assert got_cold + got_warm == want
    assert cache.stats["hits"] >= 2 and cache.stats["hit_tokens"] >= 256
    again = run_requests(sched, prompts[:1], 12)                 # whole prompt cached except its tail: still identical
    assert again == want[:1]


def test_sampling_depends_only_on_seed_and_position():
    spec, eng, sched, _ = build(prefix=False)
    p = torch.randint(0, spec.vocab, (20,), generator=torch.Generator().manual_seed(1)).tolist()
    sp = SamplingParams(temperature=0.9, top_p=0.95, top_k=40, seed=7)
    a = run_requests(sched, [p], 10, sampling=sp)
    b = run_requests(sched, [p, p[:10]], 10, sampling=sp)        # different batch layout, same request
    assert a[0] == b[0] and len(set(a[0])) > 1
    c = run_requests(sched, [p], 10, sampling=SamplingParams(temperature=0.9, top_p=0.95, top_k=40, seed=8))
    assert c[0] != a[0]


def test_sampled_requests_are_drafted_and_verified_losslessly():
    """Sampled verification: a sampling request with the n-gram drafter yields the token stream of the same request without drafts
    (verify rows are sampled with the (seed, position) generator; a draft is accepted when it equals its row's sample)."""
    sp = SamplingParams(temperature=0.4, top_p=0.95, top_k=40, seed=12)
    g = torch.Generator().manual_seed(3)
    spec = tiny_spec()
    base = torch.randint(0, spec.vocab, (12,), generator=g).tolist()
    prompts = [base * 4, base[:7] * 6]
    _, _, plain, _ = build(prefix=False)
    want = run_requests(plain, prompts, 24, sampling=sp)
    _, _, sched, _ = build(drafter=NgramDrafter(), prefix=False)
    got = run_requests(sched, prompts, 24, sampling=sp)
    assert got == want
    assert sched.stats["drafted"] > 0


def test_scheduler_with_mtp_drafter_is_lossless():
    """The model's own MTP module drafts inside the serving loop (chunked prefill, several sequences): the output must
    equal plain greedy generation, and drafts must have been proposed and verified."""
    from cuteafd_b200.serving.mtp_drafter import MtpDrafter
    spec = tiny_spec().replace(mtp_layers=1)
    masters = init_weights(spec, 4)
    n_pages = 64
    eng = Engine(DeviceWeights.from_masters(spec, masters, DEV), n_pages=n_pages, max_seqs=8, max_pages_per_seq=8)
    pool = PagePool(n_pages)
    runner = attach_pool(EngineRunner(eng, max_rows=256), pool)
    drafter = MtpDrafter(runner)
    sched = Scheduler(runner, pool, max_seqs=4, prefill_chunk=48, drafter=drafter)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, spec.vocab, (n,), generator=g).tolist() for n in (7, 70, 23)]
    ref_eng = Engine(DeviceWeights.from_masters(spec, masters, DEV), n_pages=n_pages, max_seqs=8, max_pages_per_seq=8)
    want = generate(ref_eng, prompts, 14, use_graph=False)
    got = run_requests(sched, prompts, 14)
    assert got == want
    assert drafter.proposed > 0 and sched.stats["drafted"] > 0


def test_host_tier_restores_an_evicted_prefix_exactly():
    """Pages written behind into pinned host memory and copied back give the same tokens as the device-resident prefix."""
    from cuteafd_b200.serving.hostcache import attach_host_tier
    spec, eng, sched, _ = build(prefix=False)
    pool = sched.pool
    host = attach_host_tier(eng, 0.05, min_tokens=128)
    cache = PrefixCache(pool, min_tokens=64, host=host)
    sched.prefix = cache
    g = torch.Generator().manual_seed(5)
    shared = torch.randint(0, spec.vocab, (200,), generator=g).tolist()
    p1, p2 = shared + [3, 4, 5], shared + [9, 8, 7, 6]
    ref = run_requests(build(prefix=False)[2], [p1, p2], 12)
    out1 = run_requests(sched, [p1], 12)[0]
    cache.evict(10 ** 6)                                               # the device tier forgets the chain
    assert cache.lookup(p2) == 0 and host.lookup(p2) == 3
    eng.kv.zero_()                                                     # whatever was on the device is gone for good
    out2 = run_requests(sched, [p2], 12)[0]
    eng.check_status()
    assert out1 == ref[0] and out2 == ref[1]
    assert cache.stats["host_hits"] == 1 and cache.stats["host_hit_tokens"] == 192 and host.copy.launches >= 2


def test_graph_census_follows_the_engine():
    spec, eng, sched, _ = build(prefix=False)
    g = torch.Generator().manual_seed(1)
    run_requests(sched, [torch.randint(0, spec.vocab, (40,), generator=g).tolist()], 6)
    snap = eng.census.snapshot()
    assert snap["captures"] == eng.graph_captures and snap["replays"] >= snap["captures"] > 0
    eng.census.seal()
    key = next(iter(eng.graphs))
    before = eng.graph_captures
    run_requests(sched, [torch.randint(0, spec.vocab, (40,), generator=g).tolist()], 6)       # same shapes: no new capture
    assert eng.graph_captures == before and eng.census.snapshot()["steady_state_captures"] == 0
    assert key in eng.census.shapes


def test_json_grammar_mask_steers_the_real_sampler_and_argmax():
    """A request with a grammar constraint goes through the masked argmax (greedy) and the masked sampler (top-k) kernels:
    whatever the tiny model prefers, the text stays a JSON object prefix and only ends after a complete object."""
    import json
    from cuteafd_b200.loader.tokenizer import ByteTokenizer
    from cuteafd_b200.serving.constraints import JsonConstraint, JsonPrefix
    spec, eng, sched, _ = build(prefix=False)
    tok = ByteTokenizer()
    prompt = tok.encode("answer in json:")
    for i, sampling in enumerate((SamplingParams(), SamplingParams(temperature=0.8, top_k=40, seed=7))):
        outs = []
        c = JsonConstraint(tok, spec.vocab, len(prompt), eos_id=257, top="object")
        sched.submit(Request(f"j{i}", list(prompt), max_tokens=48, sampling=sampling, eos_id=257, constraint=c,
                             on_token=lambda toks, done, reason, outs=outs: outs.extend(toks)))
        sched.run_until_idle()
        eng.check_status()
        text = tok.decode([t for t in outs if t != 257])
        assert all(t < 258 for t in outs) and text.lstrip().startswith("{") and JsonPrefix("object").feed_text(text), text
        if outs and outs[-1] == 257:
            assert isinstance(json.loads(text), dict)


def test_scheduler_serves_a_hybrid_linear_attention_model():
    """Continuous batching over a stack with gated delta-rule layers: every live sequence owns a recurrent-state slot of the engine
    (assigned at its first chunk, freed when it finishes, reused by later requests); chunked prefill, more requests than slots in
    flight at once, and the tokens of plain generation."""
    import dataclasses
    base = tiny_spec()
    spec = base.replace(n_layers=4, attn=dataclasses.replace(base.attn, n_heads=4, n_kv_heads=2, head_dim=128, linear_every=2, linear_k_heads=1,
                                                             linear_v_heads=2))
    masters = init_weights(spec, 9)
    n_pages = 64
    eng = Engine(DeviceWeights.from_masters(spec, masters, DEV), n_pages=n_pages, max_seqs=4, max_pages_per_seq=8)
    pool = PagePool(n_pages)
    runner = attach_pool(EngineRunner(eng, max_rows=256), pool)
    sched = Scheduler(runner, pool, max_seqs=3, prefill_chunk=40)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, spec.vocab, (n,), generator=g).tolist() for n in (9, 75, 30, 52, 18)]
    ref_eng = Engine(DeviceWeights.from_masters(spec, masters, DEV), n_pages=n_pages, max_seqs=8, max_pages_per_seq=8)
    want = generate(ref_eng, prompts, 10, use_graph=False)
    got = run_requests(sched, prompts, 10)
    assert got == want
    assert not runner._state_slot and sorted(runner._free_slots) == [0, 1, 2, 3]      # every slot came back
    again = run_requests(sched, prompts[:2], 6)                                         # reused slots start from a zero state
    assert again == [w[:6] for w in want[:2]]


@pytest.mark.parametrize("per_channel", [False, True])
def test_drafted_decoding_over_linear_attention_layers_is_lossless(per_channel):
    """Speculation on a hybrid stack: verify steps leave the recurrent state and the convolution history alone, the accepted rows are
    replayed into them (`Engine.commit_state`), so drafted greedy and sampled decoding reproduce the undrafted token streams -
    with drafts accepted (repetitive prompts) and rejected."""
    import dataclasses
    base = tiny_spec()
    spec = base.replace(n_layers=4, attn=dataclasses.replace(base.attn, n_heads=4, n_kv_heads=2, head_dim=128, linear_every=2, linear_k_heads=1,
                                                             linear_v_heads=2, linear_per_channel=per_channel))
    masters = init_weights(spec, 11)

    def make(drafter):
        eng = Engine(DeviceWeights.from_masters(spec, masters, DEV), n_pages=64, max_seqs=4, max_pages_per_seq=8)
        pool = PagePool(64)
        runner = attach_pool(EngineRunner(eng, max_rows=256), pool)
        return Scheduler(runner, pool, max_seqs=3, prefill_chunk=48, drafter=drafter), runner
    g = torch.Generator().manual_seed(2)
    rep = torch.randint(0, spec.vocab, (9,), generator=g).tolist()
    prompts = [rep * 5, torch.randint(0, spec.vocab, (33,), generator=g).tolist(), rep[:4] * 9]
    plain, _ = make(None)
    want = run_requests(plain, prompts, 20)
    spec_sched, runner = make(NgramDrafter())
    got = run_requests(spec_sched, prompts, 20)
    assert got == want
    assert spec_sched.stats["drafted"] > 0 and spec_sched.stats["drafted"] > spec_sched.stats["accepted"] >= 0
    assert runner._deferred is None
    sp = SamplingParams(temperature=0.5, top_p=0.9, top_k=30, seed=3)
    assert run_requests(make(NgramDrafter())[0], prompts, 16, sampling=sp) == run_requests(make(None)[0], prompts, 16, sampling=sp)


def test_image_rows_replace_placeholder_embeddings_exactly():
    """Rows handed in for placeholder positions (a vision tower's output) enter the model exactly like token embeddings: a prompt
    whose placeholders carry the embedding rows of other tokens generates what the prompt with those tokens generates - across
    prefill chunks, and in a short last chunk that would otherwise replay a captured graph."""
    spec, eng, sched, _ = build(prefix=False)
    g = torch.Generator().manual_seed(21)
    real = torch.randint(1, spec.vocab, (100,), generator=g).tolist()
    positions = list(range(10, 30)) + [60, 61] + [97, 98]
    holder = list(real)
    for p in positions:
        holder[p] = 0
    rows = eng.weights.embed[torch.tensor([real[p] for p in positions], device=DEV)].contiguous()
    want = run_requests(sched, [real], 10)
    got = run_requests(sched, [holder], 10, embeds={"positions": positions, "rows": rows}, use_cache=False)
    assert got == want
    assert run_requests(sched, [holder], 10) != want            # the placeholders alone are a different prompt
    # two requests in one round, one with image rows, one without
    res = {0: [], 1: []}
    sched.submit(Request("img", holder, max_tokens=6, on_token=lambda t, d, r: res[0].extend(t), use_cache=False,
                         embeds={"positions": positions, "rows": rows}))
    sched.submit(Request("txt", real[:40], max_tokens=6, on_token=lambda t, d, r: res[1].extend(t), use_cache=False))
    sched.run_until_idle()
    assert res[0] == want[0][:6] and res[1] == run_requests(sched, [real[:40]], 6)[0]
