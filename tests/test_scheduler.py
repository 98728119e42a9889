"""Scheduler / prefix cache / speculation on CPU with the deterministic fake runner (no GPU): mirrors the reference's
serve-loop unit tests and its prefix-cache exactness + lossless-speculation gates."""
import pytest

from cuteafd_b200.engine.kv import PAGE, OutOfPages, PagePool, SeqKV
from cuteafd_b200.serving.draft_policy import ResourcePricedPolicy, SimpleDraftPolicy
from cuteafd_b200.serving.prefix import PrefixCache
from cuteafd_b200.serving.runner import FakeRunner
from cuteafd_b200.serving.scheduler import NgramDrafter, Request, Scheduler


def collect(results, rid):
    def cb(toks, done, reason):
        r = results.setdefault(rid, {"tokens": [], "done": False, "reason": None})
        r["tokens"] += toks
        r["done"], r["reason"] = done, reason
    return cb


def direct(runner, prompt, n):
    toks = list(prompt)
    out = []
    for _ in range(n):
        t = runner.next_token(toks)
        out.append(t)
        toks.append(t)
    return out


def make(n_pages=64, **kw):
    pool = PagePool(n_pages)
    runner = FakeRunner()
    return Scheduler(runner, pool, **kw), runner, pool


def test_continuous_batching_matches_direct_generation_and_frees_pages():
    sched, runner, pool = make(max_seqs=3, prefill_chunk=50)
    free0 = pool.n_free
    res = {}
    prompts = {f"r{i}": list(range(i, i + 30 + 17 * i)) for i in range(5)}
    for rid, p in prompts.items():
        sched.submit(Request(rid, p, max_tokens=9, on_token=collect(res, rid)))
    sched.run_until_idle()
    for rid, p in prompts.items():
        assert res[rid]["done"] and res[rid]["reason"] == "length"
        assert res[rid]["tokens"] == direct(runner, p, 9)
    assert pool.n_free == free0 and sched.stats["finished"] == 5


def test_speculation_is_lossless_and_accepts_repetitive_text():
    base, r0, _ = make()
    spec, r1, _ = make(drafter=NgramDrafter(), policy=SimpleDraftPolicy(3))
    # a fake "model" that loops makes copy-continuation drafts hit
    r0.next_token = r1.next_token = lambda prefix: (prefix[-1] * 7 + 3) % 11
    a, b = {}, {}
    prompt = [1, 2, 3, 4, 5]
    base.submit(Request("x", prompt, max_tokens=40, on_token=collect(a, "x")))
    spec.submit(Request("x", prompt, max_tokens=40, on_token=collect(b, "x")))
    base.run_until_idle(), spec.run_until_idle()
    assert a["x"]["tokens"] == b["x"]["tokens"] and len(b["x"]["tokens"]) == 40
    assert spec.stats["accepted"] > 0 and spec.stats["steps"] < base.stats["steps"]


def test_sampling_requests_draft_too_and_keep_their_token_stream():
    """A sampling request is drafted and verified (a draft is accepted when it equals its row's sample), and so is a request with a
    grammar constraint."""
    from cuteafd_b200.ref.sampler import SamplingParams
    sp = SamplingParams(temperature=0.8, top_p=0.9, top_k=50, seed=4)
    base, r0, _ = make()
    spec, r1, _ = make(drafter=NgramDrafter(), policy=SimpleDraftPolicy(3))
    r0.next_token = r1.next_token = lambda prefix: (prefix[-1] * 7 + 3) % 11      # stands for "the sample at this position"
    a, b = {}, {}
    base.submit(Request("x", [1, 2, 3, 4, 5], max_tokens=30, on_token=collect(a, "x"), sampling=sp))
    spec.submit(Request("x", [1, 2, 3, 4, 5], max_tokens=30, on_token=collect(b, "x"), sampling=sp))
    base.run_until_idle(), spec.run_until_idle()
    assert a["x"]["tokens"] == b["x"]["tokens"] and spec.stats["accepted"] > 0

    # with a grammar constraint every verify row is masked by the state of ITS prefix: drafted and undrafted streams agree
    import torch

    class NoSixAfterEven:
        def mask(self, prefix):
            words = torch.full((1000 // 32 + 1,), -1, dtype=torch.int32)
            if prefix[-1] % 2 == 0:
                words[0] &= ~(1 << 6)
            return words
    c, d = {}, {}
    base2, r3, _ = make()
    spec2, r2, _ = make(drafter=NgramDrafter(), policy=SimpleDraftPolicy(3))
    r2.next_token = r3.next_token = r0.next_token
    base2.submit(Request("y", [1, 2, 3, 4, 5], max_tokens=30, on_token=collect(c, "y"), constraint=NoSixAfterEven()))
    spec2.submit(Request("y", [1, 2, 3, 4, 5], max_tokens=30, on_token=collect(d, "y"), constraint=NoSixAfterEven()))
    base2.run_until_idle(), spec2.run_until_idle()
    assert c["y"]["tokens"] == d["y"]["tokens"] and spec2.stats["drafted"] > 0
    assert all(not (a % 2 == 0 and b == 6) for a, b in zip(c["y"]["tokens"], c["y"]["tokens"][1:]))


def test_prefix_cache_restores_exactly_and_skips_recompute():
    pool = PagePool(64)
    runner = FakeRunner()
    cache = PrefixCache(pool, max_entries=8, min_tokens=64)
    sched = Scheduler(runner, pool, prefix=cache)
    shared = list(range(1000, 1000 + 3 * PAGE))
    res = {}
    sched.submit(Request("a", shared + [1, 2, 3], max_tokens=4, on_token=collect(res, "a")))
    sched.run_until_idle()
    rows_cold = runner.rows_seen
    sched.submit(Request("b", shared + [9, 8, 7, 6], max_tokens=4, on_token=collect(res, "b")))
    sched.run_until_idle()
    assert cache.stats["hits"] == 1 and cache.stats["hit_tokens"] == 3 * PAGE
    assert runner.rows_seen - rows_cold == 4 + 3                     # only the 4 new prompt tokens + 3 decode rows ran
    assert res["b"]["tokens"] == direct(runner, shared + [9, 8, 7, 6], 4)   # identical to a cold run
    # the very same physical pages back both sequences (byte-exact by construction)
    adm1, adm2 = cache.admit(shared + [5]), cache.admit(shared + [6])
    assert adm1.seq.pages[:3] == adm2.seq.pages[:3]
    cache.release(adm1.seq), cache.release(adm2.seq)


def test_prefix_cache_eviction_returns_pages():
    pool = PagePool(16)
    cache = PrefixCache(pool, max_entries=2, min_tokens=64)
    free0 = pool.n_free
    for i in range(4):
        toks = [i] * (2 * PAGE)
        adm = cache.admit(toks)
        adm.seq.length = len(toks)
        cache.capture(toks, adm.seq)
        cache.release(adm.seq)
    assert cache.snapshot()["entries"] <= 2 and cache.stats["evictions"] >= 2
    cache.evict(100)
    assert pool.n_free == free0
    with pytest.raises(OutOfPages):
        cache.admit(list(range(20 * PAGE)))


def test_kv_pressure_defers_then_admits():
    sched, runner, pool = make(n_pages=8, max_seqs=8)
    res = {}
    for i in range(4):
        sched.submit(Request(f"r{i}", list(range(100)), max_tokens=20, on_token=collect(res, f"r{i}")))
    sched.run_until_idle()
    assert all(res[f"r{i}"]["reason"] == "length" for i in range(4))
    assert sched.stats["deferred"] > 0


def test_failed_step_fails_only_its_requests_and_fatal_fans_out():
    sched, runner, pool = make()
    res = {}
    sched.submit(Request("a", [1, 2, 3], max_tokens=5, on_token=collect(res, "a")))
    runner.fail_next = "injected step failure"
    sched.run_until_idle()
    assert res["a"]["done"] and res["a"]["reason"].startswith("error")
    sched.submit(Request("b", [1, 2, 3], max_tokens=5, on_token=collect(res, "b")))
    sched.run_until_idle()
    assert res["b"]["reason"] == "length"
    sched.submit(Request("c", list(range(50)), max_tokens=50, on_token=collect(res, "c")))
    sched.submit(Request("d", [1], max_tokens=5, on_token=collect(res, "d")))
    sched.step()
    sched.fail_all("expert transport failed")
    assert res["c"]["reason"].startswith("error") and res["d"]["reason"].startswith("error")
    assert not sched.submit(Request("e", [1], on_token=collect(res, "e"))) and res["e"]["reason"].startswith("unavailable")
    assert pool.n_free == pool.n_pages - 1


def test_cancelled_prefill_is_parked_as_a_snapshot():
    pool = PagePool(64)
    cache = PrefixCache(pool, min_tokens=64)
    sched = Scheduler(FakeRunner(), pool, prefix=cache, prefill_chunk=PAGE)
    res = {}
    prompt = list(range(5 * PAGE + 7))
    sched.submit(Request("p", prompt, max_tokens=4, on_token=collect(res, "p")))
    sched.step(), sched.step()
    sched.cancel("p")
    sched.run_until_idle()
    assert res["p"]["reason"] == "cancelled" and cache.stats["parked"] == 1
    assert cache.lookup(prompt) >= 2 * PAGE


def test_stop_ids_eos_and_decode_share():
    sched, runner, _ = make(prefill_chunk=32, decode_share=0.5)
    runner.next_token = lambda prefix: 7 if len(prefix) % 5 == 0 else 3
    res = {}
    sched.submit(Request("s", [1, 2, 3], max_tokens=50, eos_id=7, on_token=collect(res, "s")))
    sched.submit(Request("long", list(range(300)), max_tokens=2, on_token=collect(res, "long")))
    sched.run_until_idle()
    assert res["s"]["reason"] == "stop" and res["s"]["tokens"][-1] == 7
    assert res["long"]["reason"] == "length"


def test_resource_priced_policy_prefers_width_when_acceptance_is_high():
    p = ResourcePricedPolicy(max_width=4, base_ms=30, row_ms=0.3, draft_ms=0.5, prior=0.5)
    for _ in range(50):
        p.observe("r", 4, 4)
    assert p.width("r", 64) == 4
    q = ResourcePricedPolicy(max_width=4, base_ms=1.0, row_ms=2.0, draft_ms=2.0, prior=0.5)
    for _ in range(50):
        q.observe("r", 4, 0)
    assert q.width("r", 64) == 0
    assert p.width("r", 1) == 0


def test_admission_wait_budget_answers_busy_instead_of_queueing_forever():
    import time as _t
    from cuteafd_b200.engine.kv import PagePool
    from cuteafd_b200.serving.runner import FakeRunner
    from cuteafd_b200.serving.scheduler import Request, Scheduler
    sched = Scheduler(FakeRunner(vocab=50), PagePool(64), max_seqs=1, queue_wait_s=0.05)
    got = {}
    for name, n in (("a", 400), ("b", 4)):
        sched.submit(Request(name, [1, 2, 3], max_tokens=n, on_token=lambda t, d, r, name=name: got.setdefault(name, []).append((len(t), d, r))))
    sched.step()                                   # "a" is admitted, "b" waits for a lane
    _t.sleep(0.08)
    sched.step()
    assert got["b"][-1][1] and got["b"][-1][2].startswith("busy") and sched.stats["rejected"] == 1
    sched.run_until_idle()
    assert got["a"][-1][2] == "length"
