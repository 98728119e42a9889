"""A multi-GPU layout's decode step run as ONE process on ONE GPU (`parallel.local.LocalWorld`: every rank's real kernels and
flag protocol, "peers" in local memory), full-size layer shapes and a few layers.  The ranks' kernels run one after the other on
the one GPU, so the step time is NOT a throughput number; the point is a single-process target whose launch list (a profiler's
`gpu__time_duration.sum` per launch, or `--events`) shows what every kernel of a layer costs without NVLink:

    python -m cuteafd_b200.bench.local_layout --model qwen3-235b --layers 3 --ranks 4 --layout colocated --batch 16 --context 4096
    python -m cuteafd_b200.bench.local_layout --model deepseek-v3 --layers 4 --ranks 4 --layout split --batch 32 --context 2048

`--batch` is sequences per attention group.  Prints the eager step time, the launches per step and per rank, and the status words.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from ..config import deepseek_v3_spec, deployment_by_name, qwen3_235b_spec
from ..engine.engine import PAGE
from ..engine.generate import BatchGenerator
from ..engine.kv import PagePool, SeqKV
from ..parallel.afd import LanePlan
from ..parallel.local import LocalWorld


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-235b", choices=["qwen3-235b", "deepseek-v3"])
    ap.add_argument("--layers", type=int, default=3)
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--layout", default="colocated", choices=["colocated", "split"])
    ap.add_argument("--attn-groups", type=int, default=1)
    ap.add_argument("--n-micro", type=int, default=1)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    spec = qwen3_235b_spec(a.layers) if a.model == "qwen3-235b" else deepseek_v3_spec(a.layers)
    dep = deployment_by_name(a.layout, a.ranks, a.attn_groups)
    plan = LanePlan(dep, t_cap=max(16, -(-a.batch // a.n_micro)), n_micro=a.n_micro, merged=dep.colocated)
    plan.check()
    pages_per_seq = a.context // PAGE + 2
    world = LocalWorld(spec, plan, dev, n_pages=a.batch * pages_per_seq + 2, max_seqs=a.batch, max_pages_per_seq=pages_per_seq)
    gens = {}
    for r, eng in world.engines.items():
        g = BatchGenerator(eng, PagePool(eng.n_pages))
        g.seqs = []
        for _ in range(a.batch):
            s = SeqKV()
            s.ensure(g.pool, a.context + a.steps + a.warmup + 4)
            s.length = a.context
            g.seqs.append(s)
        g.last = torch.randint(0, spec.vocab, (a.batch,)).tolist()
        eng.kv.normal_(0, 1)
        gens[r] = g

    def step():
        shapes = {r: g.plan_decode() for r, g in gens.items()}
        lanes = world.step(shapes)
        for r, g in gens.items():
            g.commit_decode(lanes[r])

    for _ in range(a.warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    world.check()
    launches = {f"attn{r}": e.launches_per_step for r, e in world.engines.items()}
    launches.update({f"exp{r}": w.launches_per_step for r, w in world.workers.items()})
    print(json.dumps({"bench": "local_layout", "model": spec.name, "layers": a.layers, "layout": dep.describe(), "ranks": a.ranks, "n_micro": a.n_micro,
                      "batch_per_group": a.batch, "context": a.context, "ms_per_step_all_ranks_serialised": round(e0.elapsed_time(e1) / a.steps, 3),
                      "launches_per_step": launches, "note": "all ranks share one GPU: not a throughput number"}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
