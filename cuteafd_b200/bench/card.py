"""Baseline card of a serving stack, measured through its own scheduler (the in-server benchmark of the reference:
cuteafd-bench/src/baseline.rs:19-75, profiles.rs:33-35, quality checks quick.rs):

  * C1 decode tokens/s on three prompt kinds ("code", "prose", "json": synthetic token streams with different amounts of
    self-repetition, which is what makes draft acceptance content dependent), 320 generated tokens, greedy;
  * aggregate tokens/s at C4 / C8 / C16: 160 tokens per stream, one untimed warm wave, then a timed wave;
  * cold prefill of one ~8k-token prompt: prompt tokens/s and TTFT; TTFT of a 55-token prompt;
  * quick quality gates that need no golden files: prefix-cache exactness (a repeated prompt reproduces its output),
    lossless speculation (drafts on == drafts off), C1 vs C4 agreement (batching does not change tokens).

`run_card(make_scheduler, vocab)` takes a factory returning a fresh scheduler (so cold numbers are cold); it runs on the GPU
engine (`cuteafd card`) and on the CPU fake runner (tests).
"""
from __future__ import annotations

import random
import time

from ..serving.scheduler import Request


def synth_prompt(kind: str, n: int, vocab: int, seed: int = 0) -> list[int]:
    """Token stream of a given 'texture': code repeats short spans often, json repeats a rigid skeleton, prose rarely repeats."""
    rng = random.Random(f"{kind}:{seed}")
    lo = min(16, vocab - 1)
    fresh = lambda: rng.randrange(lo, vocab)
    if kind == "prose":
        return [fresh() for _ in range(n)]
    out: list[int] = []
    if kind == "json":
        skeleton = [fresh() for _ in range(6)]
        while len(out) < n:
            out += skeleton[:3] + [fresh()] + skeleton[3:] + [fresh()]
        return out[:n]
    spans = [[fresh() for _ in range(rng.randrange(3, 9))] for _ in range(12)]
    while len(out) < n:
        out += rng.choice(spans) if rng.random() < 0.6 else [fresh() for _ in range(rng.randrange(1, 5))]
    return out[:n]


def _run_wave(sched, prompts, max_tokens, **req_kw):
    """Submits all prompts, runs to idle.  Returns (outputs, per-request ttft seconds, wall seconds)."""
    outs = {i: [] for i in range(len(prompts))}
    first: dict = {}
    t0 = time.perf_counter()
    for i, p in enumerate(prompts):
        def cb(toks, done, reason, i=i):
            if toks and i not in first:
                first[i] = time.perf_counter() - t0
            outs[i].extend(toks)
        sched.submit(Request(f"card-{i}-{time.perf_counter_ns()}", list(p), max_tokens=max_tokens, on_token=cb, **req_kw))
    sched.run_until_idle()
    wall = time.perf_counter() - t0
    return [outs[i] for i in range(len(prompts))], [first.get(i) for i in range(len(prompts))], wall


def run_card(make_scheduler, vocab: int, *, c1_tokens: int = 320, wave_tokens: int = 160, levels=(4, 8, 16), prefill_tokens: int = 8192,
             short_prompt: int = 55, prompt_len: int = 200) -> dict:
    card: dict = {"c1": {}, "aggregate": {}, "quality": {}}
    # ---- C1 decode on the three prompt kinds
    for kind in ("code", "prose", "json"):
        sched = make_scheduler()
        p = synth_prompt(kind, prompt_len, vocab)
        _run_wave(sched, [p], 8, use_cache=False)                                  # warm-up (graphs, allocations)
        outs, ttft, wall = _run_wave(sched, [p], c1_tokens, use_cache=False)
        dec = wall - (ttft[0] or 0.0)
        card["c1"][kind] = {"tokens_per_s": round((len(outs[0]) - 1) / dec, 2) if dec > 0 and len(outs[0]) > 1 else None,
                            "ttft_s": round(ttft[0], 6) if ttft[0] is not None else None, "generated": len(outs[0]),
                            "drafted": sched.stats.get("drafted", 0), "accepted": sched.stats.get("accepted", 0)}
    # ---- aggregate throughput
    for n in levels:
        sched = make_scheduler()
        prompts = [synth_prompt("code", prompt_len, vocab, seed=s) for s in range(n)]
        _run_wave(sched, prompts, 8, use_cache=False)
        outs, _, wall = _run_wave(sched, [synth_prompt("code", prompt_len, vocab, seed=100 + s) for s in range(n)], wave_tokens, use_cache=False)
        admitted = sum(1 for o in outs if o)
        card["aggregate"][f"c{n}"] = {"tokens_per_s": round(sum(len(o) for o in outs) / wall, 2), "admitted": admitted}
    # ---- prefill and TTFT
    sched = make_scheduler()
    _run_wave(sched, [synth_prompt("prose", 64, vocab, seed=7)], 2, use_cache=False)
    _, ttft, _ = _run_wave(sched, [synth_prompt("prose", prefill_tokens, vocab, seed=1)], 1, use_cache=False)
    card["prefill"] = {"prompt_tokens": prefill_tokens, "ttft_s": round(ttft[0], 6) if ttft[0] is not None else None,
                       "tokens_per_s": round(prefill_tokens / max(ttft[0], 1e-9), 1) if ttft[0] is not None else None}
    _, ttft, _ = _run_wave(sched, [synth_prompt("code", short_prompt, vocab, seed=2)], 1, use_cache=False)
    card["ttft_short_s"] = round(ttft[0], 6) if ttft[0] is not None else None
    # ---- quick quality gates
    p = synth_prompt("code", prompt_len, vocab, seed=9)
    sched = make_scheduler()
    a, _, _ = _run_wave(sched, [p], 48)
    b, _, _ = _run_wave(sched, [p], 48)                                            # second time: prefix restored from the cache
    card["quality"]["prefix_cache_exact"] = a == b
    nodraft, _, _ = _run_wave(make_scheduler(), [p], 48, allow_drafts=False, use_cache=False)
    card["quality"]["speculation_lossless"] = a == nodraft
    others = [synth_prompt("prose", prompt_len, vocab, seed=20 + s) for s in range(3)]
    batch, _, _ = _run_wave(make_scheduler(), [p] + others, 48, use_cache=False)
    card["quality"]["c1_equals_c4"] = batch[0] == a[0]
    return card
