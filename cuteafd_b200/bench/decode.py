"""Decode-throughput benchmark of a MoE decoder (the `bench.py` flagship).

Measures K decode steps of `batch_per_gpu * n_gpus` sequences at a fixed context length:
  * device arm: K CUDA-graph replays of the step, timed with CUDA events on the launching stream between a
    barrier + synchronize on both sides, max over ranks;
  * end-to-end arm: the same K steps through `BatchGenerator.decode_step()` (the public generation API), each
    step copying its inputs host-to-device from pinned memory and reading the chosen tokens back.
Weights are far larger than L2 (hundreds of GB streamed per second), so no explicit L2 flush is needed.
"""
from __future__ import annotations

import time

import torch

from ..config import deepseek_v3_spec, qwen3_235b_spec, default_deployment
from ..engine.engine import Engine, StepShape, PAGE
from ..engine.generate import BatchGenerator
from ..engine.kv import PagePool, SeqKV
from ..models.weights import DeviceWeights


def _fill_context(gen: BatchGenerator, eng: Engine, batch: int, context: int, vocab: int, seed: int):
    """Synthetic context: allocate pages for `context` tokens per sequence and fill their KV with random values
    (equivalent, for decode timing, to having prefetched `context` random tokens)."""
    g = torch.Generator(device=eng.device).manual_seed(seed)
    gen.seqs = []
    for _ in range(batch):
        s = SeqKV()
        s.ensure(gen.pool, context + 1)
        s.length = context
        gen.seqs.append(s)
    for li in range(eng.kv.shape[0]):
        eng.kv[li].normal_(0, 1, generator=g)
    gen.last = torch.randint(0, vocab, (batch,), generator=torch.Generator().manual_seed(seed)).tolist()


def run_decode_bench(args, rank: int, world: int, local: int, clocks) -> dict:
    dev = torch.device("cuda", local)
    if args.config.startswith("deepseek-v3"):
        spec = deepseek_v3_spec(args.layers or 61)
        if world == 1:
            raise SystemExit("the DeepSeek-V3 shape needs the attention/expert split (run with --gpus 4 or 8)")
    elif args.config.startswith("hybrid-"):
        from ..config import hybrid_gdn_spec
        spec = hybrid_gdn_spec(args.layers or 48, per_channel=args.config.startswith("hybrid-kda"))
    else:
        spec = qwen3_235b_spec(args.layers or 94)
    if getattr(args, "hyper_streams", 0):          # the same shape with four residual streams (hyper-connections), single GPU
        spec = spec.replace(hyper_streams=args.hyper_streams, name=spec.name + f"+mhc{args.hyper_streams}")
    batch = getattr(args, "batch_total", 0) or args.batch_per_gpu * world
    if world > 1:
        from ..parallel.runner import run_decode_bench_distributed
        return run_decode_bench_distributed(args, spec, rank, world, local, clocks)

    t0 = time.time()
    dw = DeviceWeights.random(spec, dev, seed=1)
    pages = batch * (-(-(args.context + args.steps + args.warmup + 8) // PAGE) + 1) + 2
    eng = Engine(dw, n_pages=pages, max_seqs=batch, max_pages_per_seq=-(-(args.context + 256) // PAGE))
    gen = BatchGenerator(eng, PagePool(pages))
    if args.real_prefill:
        g = torch.Generator().manual_seed(0)
        gen.prefill([torch.randint(0, spec.vocab, (args.context,), generator=g).tolist() for _ in range(batch)])
    else:
        _fill_context(gen, eng, batch, args.context, spec.vocab, 0)
    torch.cuda.synchronize()
    setup_s = time.time() - t0

    # ---- end-to-end arm (public API; H2D inputs + D2H tokens every step)
    for _ in range(args.warmup):
        gen.decode_step()
    torch.cuda.synchronize()
    gen.h2d_bytes = gen.d2h_bytes = 0
    t1 = time.perf_counter()
    for _ in range(args.steps):
        gen.decode_step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t1
    h2d, d2h = gen.h2d_bytes // args.steps, gen.d2h_bytes // args.steps

    # ---- device arm: graph replays timed with CUDA events
    kv_len = [s.length + 1 for s in gen.seqs]
    sh = StepShape(T=batch, n_seq=batch, max_q_len=1, n_logits=batch, attn_splits=eng.attn_splits_for(batch, 1, max(kv_len)), uniform=True)
    for _ in range(args.warmup):
        eng.run(sh)
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    clocks.start()
    time.sleep(0.3)
    torch.cuda.synchronize()
    ev0.record()
    for _ in range(args.steps):
        eng.run(sh)
    ev1.record()
    torch.cuda.synchronize()
    dev_ms = ev0.elapsed_time(ev1)
    time.sleep(0.2)
    clk = clocks.stop()
    eng.check_status()

    ms_per_step = dev_ms / args.steps
    wbytes = dw.nbytes()
    res = {
        "metric": "decode_tokens_per_s", "value": round(batch * args.steps / (dev_ms / 1e3), 2), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 activations, NVFP4 (W4A4) GEMMs",
        "data": "synthetic token ids, random-init weights" + ("" if args.real_prefill else ", context KV random-filled"),
        "config": {"model": spec.name + (f" (DEBUG {args.layers} layers: INVALID)" if args.layers else ""),
                   "global_batch": batch, "seq_len": args.context, "parallelism": "single" if world == 1 else f"afd-tp2-ep{world - 2}",
                   "layers": spec.n_layers, "weights_gb": round(wbytes / 1e9, 1),
                   "l2": "inputs (weights + KV) far larger than L2; no flush needed",
                   "setup_s": round(setup_s, 1)},
        "clocks": clk,
        "e2e": {"value": round(batch * args.steps / e2e_s, 2), "unit": "tokens/s", "ms_per_step": round(e2e_s * 1e3 / args.steps, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": eng.launches_per_step * args.steps,
        "graph_captures": eng.graph_captures,
    }
    return res
