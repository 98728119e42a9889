"""Where a decode step's time goes INSIDE its replayed CUDA graph (one GPU, the Qwen3-235B-A22B or DeepSeek-V3 shape, a few layers).

A launch list taken under a profiler times every kernel cold and alone; what a kernel costs inside the step is different (weights
prefetched under the previous kernel, L2 contents, exposed tails).  Three views, all of the same replayed graph:

    python -m cuteafd_b200.bench.step_timeline --mode kernels          # per-kernel start / duration / exposed time (activity records)
    python -m cuteafd_b200.bench.step_timeline --mode ablate           # step time with one kernel family's launches left out
    python -m cuteafd_b200.bench.step_timeline --mode cluster-trace    # device stamps inside the cluster split-K GEMM (wo, wqkv)
    python -m cuteafd_b200.bench.step_timeline --model deepseek-v3 --batch 1 --context 8192 --layers 7 --mode kernels

`kernels` uses the torch profiler's CUDA activity records around three replays (diagnosis: its durations are not bench values);
"exposed" is the part of a kernel's span after every earlier kernel has ended (kernels launched with programmatic dependent launch
start early and wait).  `ablate` replays the graph with the launches of one family skipped (consumers read the previous replay's
buffers, so the data stays valid) and reports the step-time difference per layer.  `cluster-trace` turns on the global-timer stamps
of `tc_linear_cluster_kernel` for one output width and prints min / median / max over the CTAs of the step's last such launch.
"""
from __future__ import annotations

import argparse
import collections
import json

import torch

from .. import ops
from ..config import deepseek_v3_spec, qwen3_235b_spec
from ..engine.engine import PAGE, Engine, StepShape
from ..engine.generate import BatchGenerator
from ..engine.kv import PagePool, SeqKV
from ..models.weights import DeviceWeights
from ..ops import native


def build(a):
    dev = torch.device("cuda", 0)
    if a.model == "deepseek-v3":
        from ..engine.mla import MlaEngine, mla_weights_random
        spec = deepseek_v3_spec(a.layers)
        dw = mla_weights_random(spec, dev, distinct_moe_layers=2, seed=1)
        pages = a.batch * (a.context // PAGE + 2) + 2
        eng = MlaEngine(dw, n_pages=pages, max_seqs=a.batch, max_pages_per_seq=a.context // PAGE + 4)
    else:
        spec = qwen3_235b_spec(a.layers)
        dw = DeviceWeights.random(spec, dev, seed=1)
        pages = a.batch * (-(-(a.context + 64) // PAGE) + 1) + 2
        eng = Engine(dw, n_pages=pages, max_seqs=a.batch, max_pages_per_seq=-(-(a.context + 256) // PAGE))
    gen = BatchGenerator(eng, PagePool(pages))
    gen.seqs = []
    for _ in range(a.batch):
        s = SeqKV()
        s.ensure(gen.pool, a.context + 16)
        s.length = a.context
        gen.seqs.append(s)
    eng.kv.normal_(0, 1)
    gen.last = torch.randint(0, spec.vocab, (a.batch,)).tolist()
    for _ in range(3):
        gen.decode_step()
    sh = StepShape(T=a.batch, n_seq=a.batch, max_q_len=1, n_logits=a.batch, attn_splits=eng.attn_splits_for(a.batch, 1, a.context + 1), uniform=True)
    for _ in range(3):
        eng.run(sh)
    torch.cuda.synchronize()
    eng.check_status()
    return eng, sh


def timed(eng, sh, n: int = 30) -> float:
    eng.graphs.clear()
    for _ in range(3):
        eng.run(sh)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        eng.run(sh)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n


def kernels(eng, sh, a):
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            eng.run(sh)
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and "Memcpy" not in e.name and "Memset" not in e.name]
    ev.sort(key=lambda e: e.time_range.start)
    n = len(ev) // 3
    last = ev[2 * n:]                                     # the third replay
    span = last[-1].time_range.end - last[0].time_range.start
    per, prev_end, rows = collections.OrderedDict(), None, []
    for e in last:
        d = e.time_range.end - e.time_range.start
        exposed = d if prev_end is None else max(0.0, e.time_range.end - max(prev_end, e.time_range.start))
        acc = per.setdefault(e.name[:72], [0, 0.0, 0.0])
        acc[0] += 1
        acc[1] += d
        acc[2] += exposed
        rows.append((e.time_range.start - last[0].time_range.start, d, exposed, e.name[:72]))
        prev_end = max(prev_end or 0, e.time_range.end)
    print(f"step span {span:.1f} us, {n} kernels, {a.layers} layers")
    print(f"{'kernel':72s} {'n':>4s} {'dur us':>8s} {'exposed':>8s} {'exposed total':>14s}")
    for k, (c, d, v) in sorted(per.items(), key=lambda kv: -kv[1][2]):
        print(f"{k:72s} {c:4d} {d / c:8.2f} {v / c:8.2f} {v:14.1f}")
    i0 = len(rows) // 2
    print("--- a stretch of the timeline (start us, duration, exposed)")
    for s, d, v, name in rows[i0:i0 + a.stretch]:
        print(f"{s:10.2f} +{d:7.2f} exposed {v:7.2f}  {name}")


def ablate(eng, sh, a):
    real_call, state = native.call, {"skip": None}
    seen = collections.Counter()

    def family(name, args):
        if name == "cuteafd_tc_linear":
            if args[1]:
                return "grouped / dense GEMM with SwiGLU"
            if args[12] is not None:
                return "grouped GEMM"
            return f"dense GEMM N={args[19]} K={args[20]}"
        return name.replace("cuteafd_", "")

    def patched(name, *args):
        f = family(name, args)
        seen[f] += 1
        if f == state["skip"]:
            return None
        return real_call(name, *args)

    native.call = ops.call = patched
    try:
        base = timed(eng, sh)
        print(f"baseline {base:.4f} ms per step = {base * 1e3 / a.layers:.1f} us per layer")
        for f in sorted(seen):
            state["skip"] = f
            t = timed(eng, sh)
            state["skip"] = None
            print(f"{f:44s} {(base - t) * 1e3 / a.layers:8.2f} us per layer")
    finally:
        native.call = ops.call = real_call
        eng.graphs.clear()


def cluster_trace(eng, sh, a):
    import numpy as np
    labels = ["entry", "-", "released by the previous kernel", "first stage landed", "last MMA committed", "accumulator complete",
              "cluster barrier passed", "epilogue done"]
    for n_out in a.widths:
        buf = torch.zeros(512, 8, dtype=torch.int64, device=eng.device)
        ops.tc_trace(buf, -n_out)
        eng.graphs.clear()
        for _ in range(6):
            eng.run(sh)
        torch.cuda.synchronize()
        ops.tc_trace(None)
        eng.graphs.clear()
        t = buf.cpu().numpy()
        t = t[t[:, 0] != 0].astype(np.float64)
        if not len(t):
            print(f"N = {n_out}: no cluster split-K launch of this width in the step")
            continue
        t0 = t[:, 0].min()
        print(f"== N = {n_out}: {len(t)} CTAs; us from the first CTA's entry (min / median / max over CTAs)")
        for i, lab in enumerate(labels):
            col = t[:, i][t[:, i] != 0]
            if i != 1 and len(col):
                col = (col - t0) / 1e3
                print(f"  {lab:34s} {col.min():8.2f} {np.median(col):8.2f} {col.max():8.2f}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="kernels", choices=["kernels", "ablate", "cluster-trace"])
    ap.add_argument("--model", default="qwen3-235b", choices=["qwen3-235b", "deepseek-v3"])
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--stretch", type=int, default=30, help="kernels: rows of the timeline printed in order")
    ap.add_argument("--widths", type=int, nargs="*", default=[4096, 9216], help="cluster-trace: output widths N to stamp (wo, wqkv of the Qwen shape)")
    a = ap.parse_args()
    eng, sh = build(a)
    {"kernels": kernels, "ablate": ablate, "cluster-trace": cluster_trace}[a.mode](eng, sh, a)
    eng.check_status()
    print(json.dumps({"bench": "step_timeline", "mode": a.mode, "model": a.model, "layers": a.layers, "batch": a.batch, "context": a.context}))


if __name__ == "__main__":
    main()
