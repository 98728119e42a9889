"""Baseline card runner on the CPU fake runner: sections, counters and quality gates."""
from cuteafd_b200.bench.card import run_card, synth_prompt
from cuteafd_b200.engine.kv import PagePool
from cuteafd_b200.serving.prefix import PrefixCache
from cuteafd_b200.serving.runner import FakeRunner
from cuteafd_b200.serving.scheduler import NgramDrafter, Scheduler


def make():
    pool = PagePool(4096)
    return Scheduler(FakeRunner(vocab=500), pool, max_seqs=16, prefill_chunk=512, prefix=PrefixCache(pool, min_tokens=64),
                     drafter=NgramDrafter())


def test_synthetic_prompts_have_the_requested_length_and_texture():
    for kind in ("code", "prose", "json"):
        p = synth_prompt(kind, 300, 500)
        assert len(p) == 300 and all(0 <= t < 500 for t in p)
        assert p == synth_prompt(kind, 300, 500)
    rep = lambda p: 1 - len(set(zip(p, p[1:], p[2:]))) / (len(p) - 2)          # share of repeated trigrams
    assert min(rep(synth_prompt("json", 600, 500)), rep(synth_prompt("code", 600, 500))) > rep(synth_prompt("prose", 600, 500)) + 0.1


def test_card_runs_every_section_and_the_quality_gates_hold():
    card = run_card(make, vocab=500, c1_tokens=40, wave_tokens=20, levels=(4, 8), prefill_tokens=1500, prompt_len=120)
    assert set(card["c1"]) == {"code", "prose", "json"}
    for kind, r in card["c1"].items():
        assert r["generated"] == 40 and r["tokens_per_s"] > 0 and r["ttft_s"] is not None
    assert card["aggregate"]["c4"]["admitted"] == 4 and card["aggregate"]["c8"]["admitted"] == 8
    assert card["aggregate"]["c8"]["tokens_per_s"] > 0
    assert card["prefill"]["prompt_tokens"] == 1500 and card["prefill"]["tokens_per_s"] > 0 and card["ttft_short_s"] is not None
    assert card["quality"] == {"prefix_cache_exact": True, "speculation_lossless": True, "c1_equals_c4": True}
