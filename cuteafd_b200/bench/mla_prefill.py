"""Prefill of the DeepSeek-V3 shape on ONE GPU (all heads local, a few dense-FFN layers): one chunk of `--chunk` query rows
over a context of `--context` tokens, absorbed attention (the decode kernel, 1088 multiply-adds per key and head) against the
non-absorbed prefill path (gather + kv_b expansion + per-head kernel, 320 per key and head), with the per-kernel split of the
attention part of one layer measured by CUDA events on the kernels launched alone:

    python -m cuteafd_b200.bench.mla_prefill --context 32768 --chunk 2048 --layers 2
    python -m cuteafd_b200.bench.mla_prefill --context 4096 --chunk 512 --layers 1 --iters 1      # small case for a profiler

The latent cache is filled with random values for the part of the context that precedes the chunk.  FLOP counts are the causal
ones (keys a row cannot see are not counted).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..config import deepseek_v3_spec
from ..engine.engine import PAGE, StepShape
from ..engine.kv import PagePool, SeqKV
from ..engine.mla import DQK, MlaEngine, mla_weights_random
from ..ops.native import call, ptr, stream
from .. import ops


def _events(fn, iters: int) -> float:
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--context", type=int, default=32768, help="tokens in the cache after the chunk")
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--heads", type=int, default=128, help="local heads (64 = one rank of a TP2 attention group)")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--no-absorbed", action="store_true", help="skip the absorbed arm (slow at long contexts)")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    spec = deepseek_v3_spec(a.layers)
    dw = mla_weights_random(spec, dev, heads_local=a.heads, distinct_moe_layers=2, seed=1)
    pages = a.context // PAGE + 4
    eng = MlaEngine(dw, n_pages=pages, max_seqs=1, max_pages_per_seq=pages)
    pool = PagePool(pages)
    s = SeqKV()
    s.ensure(pool, a.context + 1)
    eng.kv.normal_(0, 1)
    off = a.context - a.chunk
    toks = torch.randint(0, spec.vocab, (a.chunk,)).tolist()
    eng.set_inputs(toks, list(range(off, a.context)), [s.slot(p) for p in range(off, a.context)], [a.chunk - 1], [a.context], [0], [a.chunk], [s.pages])
    sh = StepShape(T=a.chunk, n_seq=1, max_q_len=a.chunk, n_logits=1, attn_splits=1)
    Hl = a.heads
    keys_seen = a.chunk * off + a.chunk * (a.chunk + 1) // 2            # causal (query, key) pairs
    res = {"bench": "mla_prefill", "context": a.context, "chunk": a.chunk, "layers": a.layers, "heads_local": Hl}
    for name, min_q in (("non_absorbed", 128), ("absorbed", 0)):
        if name == "absorbed" and a.no_absorbed:
            continue
        MlaEngine.PREFILL_MIN_Q = min_q
        ms = _events(lambda: eng.run(sh, use_graph=False), a.iters)
        eng.check_status()
        res[name] = {"ms_per_chunk_all_layers": round(ms, 3), "ms_per_layer": round(ms / a.layers, 3),
                     "chunk_tokens_per_s": round(a.chunk / (ms / 1e3) * (1.0 / a.layers), 1)}
    MlaEngine.PREFILL_MIN_Q = 128
    # per-kernel split of the attention part of one layer (kernels launched alone on the state the step left behind)
    w = dw.layers[0].mla
    b = eng._mla_buf(eng.lane(a.chunk))
    q_nope = b["q_nope"][:Hl * a.chunk]
    md, st = eng.md, ptr(eng.status)
    rows = eng._pf_plan[1]
    scale = 192 ** -0.5
    parts = {
        "gather_ctx": lambda: call("cuteafd_mla_gather_ctx", ptr(eng.kv[0]), ptr(md["page_table"]), ptr(eng._pf_starts), ptr(md["kv_len"]), ptr(eng._pf_lat), 1,
                                   a.context, md["page_table"].shape[1], eng.kv.shape[1], eng._pf_cap, st, stream()),
        "kv_b_expand_gemm": lambda: ops.tc_linear(w.ensure_kvb(), eng._pf_act, eng._pf_kvb, rows=rows, status=eng.status),
        "mla_prefill_kernel": lambda: call("cuteafd_mla_prefill_attention", ptr(q_nope), ptr(b["q_rope"]), ptr(eng._pf_kvb), ptr(eng._pf_lat), eng._pf_cap,
                                           ptr(eng._pf_starts), ptr(md["kv_len"]), ptr(md["q_start"]), ptr(md["q_len"]), ptr(b["o_tok"]), a.chunk, 1,
                                           a.chunk, Hl, scale, st, stream()),
    }
    flops = {"gather_ctx": 0.0, "kv_b_expand_gemm": 2.0 * rows * 512 * Hl * 256, "mla_prefill_kernel": 2.0 * keys_seen * Hl * (192 + 128)}
    peaks = {}
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        peaks = json.load(open(path))
    peak = float(peaks.get("bf16_tflops", 1590.0))
    split = {}
    for name, fn in parts.items():
        ms = _events(fn, a.iters)
        tf = flops[name] / (ms / 1e3) / 1e12
        split[name] = {"ms": round(ms, 3), "tflops": round(tf, 1), "of_bf16_peak": round(tf / peak, 3)}
    eng.check_status()
    res["attention_part_of_one_layer"] = split
    res["bf16_peak_tflops_used"] = peak
    res["peak_source"] = "measured" if peaks else "fallback"
    print(json.dumps(res))


if __name__ == "__main__":
    main()
