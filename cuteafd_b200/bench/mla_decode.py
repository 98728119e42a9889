"""Decode step of the DeepSeek-V3 shape on ONE GPU (all heads local, a few layers), timed as CUDA-graph replays with CUDA
events: the micro-benchmark behind the absorbed-MLA attention numbers.

    python -m cuteafd_b200.bench.mla_decode --batch 64 --context 8192 --layers 7
    python -m cuteafd_b200.bench.mla_decode --batch 16 --layers 2 --steps 2        # small case for a profiler
    python -m cuteafd_b200.bench.mla_decode --batch 16 --context 32768 --layers 7 --index-topk 2048   # sparse attention (indexer + top-k)

The latent cache is filled with random values instead of running a prefill; with `--layers` <= 3 every layer is a dense-FFN
layer of the shape (no routed experts), which keeps the resident weights to a few GB.
"""
from __future__ import annotations

import argparse
import json

import torch

from ..config import deepseek_v3_spec
from ..engine.engine import PAGE, StepShape
from ..engine.generate import BatchGenerator
from ..engine.kv import PagePool, SeqKV
from ..engine.mla import MlaEngine, mla_weights_random


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=7)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--index-topk", type=int, default=0, help="sparse attention: the indexer keeps this many positions per query (0 = dense)")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    spec = deepseek_v3_spec(a.layers)
    if a.index_topk:
        import dataclasses
        spec = spec.replace(attn=dataclasses.replace(spec.attn, index_topk=a.index_topk, index_heads=32, index_dim=128))
    dw = mla_weights_random(spec, dev, distinct_moe_layers=2, seed=1)
    pages = a.batch * (a.context // PAGE + 2) + 2
    eng = MlaEngine(dw, n_pages=pages, max_seqs=a.batch, max_pages_per_seq=a.context // PAGE + 4)
    gen = BatchGenerator(eng, PagePool(pages))
    gen.seqs = []
    for _ in range(a.batch):
        s = SeqKV()
        s.ensure(gen.pool, a.context + 8)
        s.length = a.context
        gen.seqs.append(s)
    eng.kv.normal_(0, 1)
    if a.index_topk:
        eng.idx_kv.normal_(0, 1)
    gen.last = torch.randint(0, spec.vocab, (a.batch,)).tolist()
    for _ in range(a.warmup):
        gen.decode_step()                                   # fills the step metadata, captures the graph
    torch.cuda.synchronize()
    eng.check_status()
    sh = StepShape(T=a.batch, n_seq=a.batch, max_q_len=1, n_logits=a.batch, attn_splits=eng.attn_splits_for(a.batch, 1, a.context + 1), uniform=True)
    for _ in range(a.warmup):
        eng.run(sh)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        eng.run(sh)
    e1.record()
    torch.cuda.synchronize()
    eng.check_status()
    latent_mb = a.batch * a.context * 576 * 2 / 1e6
    print(json.dumps({"bench": "mla_decode", "batch": a.batch, "context": a.context, "layers": a.layers, "ms_per_step": round(e0.elapsed_time(e1) / a.steps, 3),
                      "launches_per_step": eng.launches_per_step, "attn_splits": sh.attn_splits, "latent_mb_per_layer": round(latent_mb, 1),
                      "index_topk": a.index_topk}))


if __name__ == "__main__":
    main()
