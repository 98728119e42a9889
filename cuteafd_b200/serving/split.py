"""Serving on a multi-GPU layout: the scheduler, prefix cache, host tier, drafters and HTTP API of the single-GPU server run
on ONE rank (the attention leader) over the engine of the attention/expert split; every other rank follows.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m cuteafd_b200.cli serve --model deepseek-v3 ...

  * leader (first attention rank): `Scheduler` + `EngineRunner` over its `AttnRankEngine`; each executed step is announced in
    the step mailbox, and with a tensor-parallel attention group the packed input block of every step goes there too;
  * other attention ranks of the group: `AfdRunner.follow_loop` - load the leader's inputs, execute the same step (their half
    of the heads; the residual stream stays bit-identical through the rank-ordered exchange);
  * expert ranks: `AfdRunner.serve_loop` - replay the expert step graph per announced step.

Prefix restore is exact for the same reason as on one GPU (restored pages ARE the pages a prefill wrote; every attention rank
holds the same page numbers because followers receive the leader's page tables).  Weights come from a snapshot directory
(decoded once to masters, cut per rank, stored in the kernels' formats) or, for a named synthetic shape, are random.
Reference: run_serve / serve_loop of the generic engine, families/deepseek_v4/serve.rs:74-200; the coordinator is the only
process that talks HTTP there too.
"""
from __future__ import annotations

import atexit
import os

import torch


def build_split_serving(a, world: int):
    """Returns (spec, scheduler) on the leader; runs the follower / expert loop to completion and returns None elsewhere."""
    import torch.distributed as dist
    from ..config import NAMED_SPECS, spec_by_name, spec_from_snapshot
    from ..engine.kv import PagePool
    from ..parallel.runner import AfdRunner, OP_STOP, default_layout
    from .prefix import PrefixCache
    from .runner import EngineRunner, attach_pool
    from .scheduler import NgramDrafter, Scheduler
    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    spec = spec_by_name(a.model) if a.model in NAMED_SPECS else spec_from_snapshot(a.model)
    if getattr(a, "layers", 0):
        spec = spec.replace(n_layers=a.layers)
    masters = None
    if os.path.isdir(a.model):
        from ..loader.checkpoint import read_masters
        masters = read_masters(a.model, spec)
    elif spec.name == "tiny":
        from ..ref.model import init_weights
        masters = init_weights(spec, 0)
    lay = default_layout(spec, world, "p2p")
    lay["layout"], lay["attn_groups"] = "split", 1           # one scheduler drives one attention group
    lay["n_micro"] = 2 if spec.attn.kind == "mla" and world >= 4 else 1
    if getattr(a, "n_micro", 0):
        lay["n_micro"] = a.n_micro
    n_pages = a.pool_tokens // 64 if a.pool_tokens else 4096
    run = AfdRunner(spec, rank, world, local, t_cap=max(16, a.prefill_batch_tokens), n_pages=n_pages, max_seqs=a.max_sequences,
                    max_pages_per_seq=min(n_pages, a.max_context // 64 + 1), layout="split", attn_groups=1, n_micro=lay["n_micro"], masters=masters)
    if rank != run.root:
        if run.is_attn:
            run.follow_loop()
        else:
            run.serve_loop(timeout_s=float("inf"))
        run.check()
        run.close()
        return None
    eng = run.engine
    if run.dep.tp > 1:
        run.mirror_inputs(True)
    def shutdown():
        """Releases the follower and expert ranks (they leave their loops on OP_STOP); safe to call more than once."""
        if not getattr(run, "_stopped", False):
            run._stopped = True
            run.control(OP_STOP)
            run.close()
    run.shutdown = shutdown
    atexit.register(shutdown)
    pool = PagePool(n_pages)
    runner = attach_pool(EngineRunner(eng, max_rows=a.prefill_batch_tokens), pool)
    host = None
    if getattr(a, "host_cache_gib", 0) > 0 and run.dep.tp == 1:
        from .hostcache import attach_host_tier
        host = attach_host_tier(eng, max(0.0, a.host_cache_gib - a.host_cache_headroom_gib), min_tokens=a.host_cache_min_tokens)
    prefix = PrefixCache(pool, max_entries=a.prefix_cache_entries, min_tokens=a.prefix_cache_min_tokens, host=host)
    drafter = None
    if a.draft == "ngram":
        drafter = NgramDrafter()
    elif a.draft == "mtp":
        if run.dep.tp > 1:
            raise SystemExit("unsupported: the MTP drafter of the server needs an attention group of one rank (its hidden-state "
                             "bookkeeping is not mirrored to a tensor-parallel partner); use --draft ngram, or a layout with attention TP1")
        from .mtp_drafter import MtpDrafter
        drafter = MtpDrafter(runner)
    sched = Scheduler(runner, pool, max_seqs=a.max_sequences, prefill_chunk=a.prefill_batch_tokens, decode_share=a.decode_share,
                      prefix=prefix, drafter=drafter, max_draft=a.draft_limit, queue_limit=getattr(a, "http_queue", 64),
                      queue_wait_s=getattr(a, "queue_wait_s", 0) or None)
    sched.afd_runner = run
    return spec, sched
