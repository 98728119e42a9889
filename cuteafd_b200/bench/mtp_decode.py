"""Decode with the model's own MTP drafter on a multi-GPU layout (DeepSeek-V3-shape headline configuration: attention
TP2 + experts on the other GPUs, a one-layer MTP module proposing `n_draft` tokens per round).

One ROUND per sequence batch = `n_draft` draft steps of the MTP module (its routed experts run on the expert ranks as an extra
layer) + ONE verify step of 1 + n_draft rows per sequence through the full model + acceptance on the device.  Every round
emits between 1 and 1 + n_draft tokens per sequence.  Reported separately, because random-init weights accept almost no draft:

  * rounds per second and tokens per second as measured (with the measured acceptance);
  * accepted drafts per round as measured;
  * the plain one-token-per-step decode of the same model, batch and context (no drafter);
  * tokens per second the measured round time WOULD give at stated acceptance levels (arithmetic, labelled as such).

Timing: K rounds (or steps) between device synchronisations, through the public `MtpSpeculator` / `BatchGenerator` API,
every step copying its inputs host-to-device from pinned memory and reading tokens back - an end-to-end number; the slowest
rank counts.  Reference: speculative_step, families/deepseek_v4/serve.rs:389-537.
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist

from ..config import ModelSpec
from ..engine.engine import PAGE
from ..engine.generate import BatchGenerator
from ..engine.kv import PagePool, SeqKV
from ..engine.mtp import MtpSpeculator, _Seq
from ..parallel.runner import AfdRunner, OP_STOP, default_layout


def run_mtp_decode_bench(args, spec: ModelSpec, rank: int, world: int, local: int, clocks, *, batch: int, context: int, n_draft: int = 3,
                         rounds: int = 10, warmup: int = 3, runner: AfdRunner | None = None) -> dict | None:
    """Returns the result dict on rank 0 (None elsewhere).  `runner`: reuse an already built model (several batch sizes on the
    same weights); otherwise one is built with the model's default layout."""
    comm = getattr(args, "comm", "p2p")
    lay = default_layout(spec, world, comm)
    if getattr(args, "layout", None):
        lay["layout"] = args.layout
        lay["attn_groups"] = world if args.layout == "colocated" else 1
        if args.layout == "colocated":
            lay["n_micro"] = 1
    if getattr(args, "attn_groups", 0) and lay["layout"] == "split":
        lay["attn_groups"] = args.attn_groups
    if lay["layout"] == "split" and spec.attn.kind == "mla" and world >= 4 and comm == "p2p":
        lay["n_micro"] = 2
    if getattr(args, "n_micro", 0):
        lay["n_micro"] = args.n_micro
    width = n_draft + 1
    ctx_pages = -(-(context + width * (rounds + warmup + 2) * 2 + 64) // PAGE)
    own = runner is None
    if own:
        from ..config import deployment_by_name
        groups = deployment_by_name(lay["layout"], world, lay["attn_groups"]).attn_groups
        if batch < groups:          # fewer sequences than attention groups (batch 1): one group on the split serves them
            lay = dict(default_layout(spec, world, comm), attn_groups=1)
            if lay["layout"] != "split":
                lay["layout"], lay["n_micro"] = "split", 1
            groups = 1
        per_group = -(-batch // groups)
        t_cap = max(16, -(-per_group * width // lay["n_micro"]))
        runner = AfdRunner(spec, rank, world, local, t_cap=t_cap, n_pages=per_group * (ctx_pages + 1) + 2, max_seqs=max(per_group, 1),
                           max_pages_per_seq=ctx_pages + 1, comm=comm, layout=lay["layout"], attn_groups=lay["attn_groups"], n_micro=lay["n_micro"],
                           expert_tp=bool(getattr(args, "expert_tp", False)))
    run = runner
    res = None
    stats = [0.0] * 6
    total_batch = batch
    if run.is_attn:
        # this rank's share of the sequences: its group's slice (every rank of a tensor-parallel group holds the same ones)
        g_all, my_g = run.dep.attn_groups, run.dep.group_of(rank)
        base, extra = divmod(total_batch, g_all)
        batch = base + (1 if my_g < extra else 0)
        leader = run.dep.group_ranks(my_g)[0] == rank
    if run.is_attn:
        eng = run.engine
        pool = PagePool(eng.n_pages)
        gk = torch.Generator(device=eng.device).manual_seed(7)
        for li in range(eng.kv.shape[0]):
            eng.kv[li].normal_(0, 1, generator=gk)
        g = torch.Generator().manual_seed(11 + my_g)
        first = torch.randint(0, spec.vocab, (batch,), generator=g).tolist()
        hid = torch.empty(batch, spec.hidden, dtype=torch.bfloat16, device=eng.device).normal_(0, 1, generator=gk)

        # ---- speculative rounds
        spec_dec = MtpSpeculator(eng, pool, n_draft=n_draft, use_graph=comm == "p2p")
        for i in range(batch):
            s = _Seq(kv=SeqKV())
            s.kv.ensure(pool, context + width + 2)
            s.length, s.anchor, s.out = context, first[i], [first[i]]
            s.pending = [(first[i], context, hid[i])]
            spec_dec.seqs.append(s)
        for _ in range(warmup):
            spec_dec.round()
        torch.cuda.synchronize()
        spec_dec.seconds_drafting = spec_dec.seconds_verifying = 0.0
        n0 = sum(len(s.out) for s in spec_dec.seqs)
        a0 = sum(sum(s.accepted) for s in spec_dec.seqs)
        if rank == 0:
            clocks.start()
        t0 = time.perf_counter()
        for _ in range(rounds):
            spec_dec.round()
        torch.cuda.synchronize()
        dt_spec = time.perf_counter() - t0
        clk = clocks.stop() if rank == 0 else None
        emitted = sum(len(s.out) for s in spec_dec.seqs) - n0
        accepted = sum(sum(s.accepted) for s in spec_dec.seqs) - a0
        end_len = max(s.length for s in spec_dec.seqs)

        # ---- plain decode of the same sequences (one token per step, no drafter)
        gen = BatchGenerator(eng, pool)
        gen.seqs = [s.kv for s in spec_dec.seqs]
        for kv, s in zip(gen.seqs, spec_dec.seqs):
            kv.length = s.length
        gen.last = [s.anchor for s in spec_dec.seqs]
        for _ in range(warmup):
            gen.decode_step(comm == "p2p")
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        for _ in range(rounds):
            gen.decode_step(comm == "p2p")
        torch.cuda.synchronize()
        dt_plain = time.perf_counter() - t1
        eng.check_status()
        # times: the slowest rank counts; tokens: summed over the groups' leaders
        stats = [dt_spec, dt_plain, float(emitted) if leader else 0.0, float(accepted) if leader else 0.0, float(end_len), spec_dec.seconds_drafting]
        if own:
            run.control(OP_STOP)
            run.check()
    elif own:
        run.serve_loop()
        run.check()
    if own:
        t = torch.tensor(stats, dtype=torch.float64, device=run.dev)
        tmax = t.clone(); dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone(); dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        stats = [float(tmax[0]), float(tmax[1]), float(tsum[2]), float(tsum[3]), float(tmax[4]), float(tmax[5])]
    batch = total_batch
    if rank == 0:
        dt_spec, dt_plain, emitted, accepted = stats[0], stats[1], stats[2], stats[3]
        round_ms = dt_spec * 1e3 / rounds
        res = {"batch": batch, "context": context, "n_draft": n_draft, "rounds": rounds, "warmup": warmup,
               "round_ms": round(round_ms, 3), "draft_steps_ms_per_round": round(stats[5] * 1e3 / rounds, 3),
               "verify_step_ms_per_round": round(round_ms - stats[5] * 1e3 / rounds, 3), "tokens_per_s_measured": round(emitted / dt_spec, 2),
               "accepted_drafts_per_round_per_seq": round(accepted / (rounds * max(batch, 1)), 3),
               "tokens_per_round_per_seq": round(emitted / (rounds * max(batch, 1)), 3),
               "plain_decode": {"ms_per_step": round(dt_plain * 1e3 / rounds, 3), "tokens_per_s": round(batch * rounds / dt_plain, 2)},
               "projected_tokens_per_s_at_acceptance": {f"{a:.1f}": round(batch * (1 + a) / (round_ms / 1e3), 1) for a in (0.0, 1.0, 2.0, 3.0) if a <= n_draft},
               "projection_note": "round time as measured x (1 + accepted drafts per round); random-init weights accept ~0 drafts",
               "parallelism": f"{run.dep.describe()}, {run.plan.n_micro} micro-batch(es) ({comm})", "clocks": clk if run.is_attn else None}
    if own:
        run.close()
    return res
