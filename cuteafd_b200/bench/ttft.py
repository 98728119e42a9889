"""Long-prefill + exact prefix-cache workload: N sessions share a long prefix and append a unique tail.
Measures cold-prefill TTFT (first session), prefix-restore TTFT (later sessions reuse the cached pages of the shared
prefix and only compute their tail), then decodes a few tokens per session.  Runs through the serving scheduler
(admission, chunked prefill, prefix cache), i.e. the path an HTTP request takes minus HTTP.

    python -m cuteafd_b200.bench.ttft --model qwen3-235b --prompt 32768 --shared 28672 --sessions 4 --decode 32
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch


def measure_sessions(sched, vocab: int, *, prompt: int, shared: int, sessions: int, decode: int, after_session=None) -> dict:
    """Runs `sessions` requests one after the other through a scheduler: each prompt = a common prefix of `shared` tokens + its own
    tail up to `prompt` tokens, then `decode` generated tokens.  Returns per-session time to first token (host clock from submit to
    the first token, device synchronised) and decode rates.  The first session is the cold prefill; later ones restore the prefix."""
    from ..serving.scheduler import Request
    g = torch.Generator().manual_seed(0)
    common = torch.randint(0, vocab, (shared,), generator=g).tolist()
    ttfts, outs, decode_s = [], [], []
    for s in range(sessions):
        p = common + torch.randint(0, vocab, (prompt - shared,), generator=g).tolist()
        t_first, toks = [None], []
        t0 = time.perf_counter()

        def cb(new, done, reason):
            if new and t_first[0] is None:
                torch.cuda.synchronize()
                t_first[0] = time.perf_counter() - t0
            toks.extend(new)
        sched.submit(Request(f"s{s}", p, max_tokens=decode, on_token=cb))
        sched.run_until_idle()
        torch.cuda.synchronize()
        total = time.perf_counter() - t0
        ttfts.append(t_first[0])
        outs.append(len(toks))
        decode_s.append(total - (t_first[0] or 0.0))
        if after_session is not None:
            after_session(s)
    warm = sorted(ttfts[1:])
    dec_tokens = sum(max(0, n - 1) for n in outs)
    return {"prompt_tokens": prompt, "shared_prefix_tokens": shared, "sessions": sessions, "cold_ttft_s": round(ttfts[0], 4),
            "cold_prefill_tok_s": round(prompt / ttfts[0], 1), "restore_ttft_s_p50": round(warm[len(warm) // 2], 4) if warm else None,
            "restore_ttfts_s": [round(t, 4) for t in ttfts[1:]], "decoded_per_session": outs,
            "decode_tok_s_per_session": round(dec_tokens / max(sum(decode_s), 1e-9), 2)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-235b")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--prompt", type=int, default=32768)
    ap.add_argument("--shared", type=int, default=28672)
    ap.add_argument("--sessions", type=int, default=4)
    ap.add_argument("--decode", type=int, default=32)
    ap.add_argument("--chunk", type=int, default=4096)
    ap.add_argument("--host-tier-gib", type=float, default=0.0,
                    help="attach a pinned host tier of this size and empty the device prefix cache between sessions, so every warm "
                         "session restores its shared pages from host memory")
    a = ap.parse_args()
    from ..config import qwen3_235b_spec, tiny_spec
    from ..engine.engine import Engine
    from ..engine.kv import PagePool
    from ..models.weights import DeviceWeights
    from ..serving.prefix import PrefixCache
    from ..serving.runner import EngineRunner, attach_pool
    from ..serving.scheduler import Request, Scheduler
    torch.cuda.set_device(0)
    spec = qwen3_235b_spec(a.layers or 94) if a.model == "qwen3-235b" else tiny_spec()
    dw = DeviceWeights.random(spec, "cuda", seed=1)
    pages_per = -(-(a.prompt + a.decode + 8) // 64) + 1
    n_pages = pages_per * (a.sessions + 1) + 8
    eng = Engine(dw, n_pages=n_pages, max_seqs=4, max_pages_per_seq=pages_per)
    pool = PagePool(n_pages)
    runner = attach_pool(EngineRunner(eng, max_rows=a.chunk), pool)
    host = None
    if a.host_tier_gib > 0:
        from ..serving.hostcache import attach_host_tier
        host = attach_host_tier(eng, a.host_tier_gib)
    cache = PrefixCache(pool, max_entries=64, min_tokens=64, max_cached_pages=n_pages, host=host)
    sched = Scheduler(runner, pool, max_seqs=1, prefill_chunk=a.chunk, prefix=cache)
    res = measure_sessions(sched, spec.vocab, prompt=a.prompt, shared=a.shared, sessions=a.sessions, decode=a.decode,
                           after_session=(lambda s: cache.evict(n_pages)) if host is not None else None)   # host tier: the device tier forgets everything
    eng.check_status()
    print(json.dumps(dict(res, bench="ttft_prefix_restore", model=spec.name, layers=spec.n_layers, prefix_cache=cache.snapshot(),
                          host_tier=(dict(host.snapshot(), copy_launches=host.copy.launches) if host is not None else None),
                          data="synthetic tokens, random-init weights")))
    return 0


if __name__ == "__main__":
    sys.exit(main())
