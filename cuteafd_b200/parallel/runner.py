"""Multi-rank driver for the attention/expert split: process groups, the control channel that tells expert ranks
which step to run, and the distributed decode benchmark.

Control protocol (CPU, gloo): before every step that really executes, attention rank 0 broadcasts (op, T).
Expert ranks sit in `serve_loop`, run one step of T token rows per message (eagerly the first time a size is
seen, from a captured CUDA graph afterwards) and leave on OP_STOP.  The data path itself never touches the host:
rows, routing tables and flags move through peer memory.  (Reference: worker selection + per-wave requests,
cuteafd-transport/src/worker_selection.rs, expert.rs:201-376; here the "request" shrinks to two integers.)
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist

from ..config import ModelSpec, default_deployment
from ..engine.engine import PAGE, StepShape
from ..engine.generate import BatchGenerator
from ..engine.kv import PagePool, SeqKV
from ..ops import KIND_BY_NAME
from .afd import AttnRankEngine, ExpertRankWorker, MlaAttnRankEngine, capture_expert_graph, make_block

OP_STOP, OP_STEP, OP_TIMER_START, OP_TIMER_STOP = 0, 1, 2, 3


class AfdRunner:
    def __init__(self, spec: ModelSpec, rank: int, world: int, local: int, *, t_max: int, n_pages: int, max_seqs: int,
                 max_pages_per_seq: int, comm: str = "p2p", seed: int = 1, attn_groups: int = 1):
        self.spec, self.rank, self.world = spec, rank, world
        self.dev = torch.device("cuda", local)
        self.dep = default_deployment(world, attn_groups)
        self.comm = comm
        self.ctrl = dist.new_group(backend="gloo")
        self.tp_group = dist.new_group(list(self.dep.attn_ranks))
        self.is_attn = rank in self.dep.attn_ranks
        self.root = self.dep.attn_ranks[0]
        kind = KIND_BY_NAME[spec.quant.experts]
        self.block = make_block(spec, self.dep, t_max, kind, rank, self.dev, None) if comm == "p2p" else None
        self.engine = self.worker = None
        if self.is_attn:
            cls = MlaAttnRankEngine if spec.attn.kind == "mla" else AttnRankEngine
            self.engine = cls(spec, self.dep, rank, self.dev, t_max=t_max, n_pages=n_pages, max_seqs=max_seqs,
                                         max_pages_per_seq=max_pages_per_seq, comm=comm, block=self.block, expert_kind=kind, seed=seed)
            self.engine.tp_group = self.tp_group
            self.engine.on_real_step = self._announce
        else:
            self.worker = ExpertRankWorker(spec, self.dep, rank, self.dev, t_max=t_max, comm=comm, block=self.block, seed=seed)
        self.graphs: dict = {}
        self.timer_ms = 0.0
        dist.barrier()

    # ---- control channel
    def _send(self, op: int, T: int = 0):
        msg = torch.tensor([op, T], dtype=torch.int64)
        dist.broadcast(msg, src=self.root, group=self.ctrl)
        return msg

    def _announce(self, sh: StepShape):
        self._send(OP_STEP, sh.T)

    def control(self, op: int):
        """Attention ranks: forward a timer/stop op to the expert ranks (all attention ranks must call it)."""
        self._send(op)

    def serve_loop(self):
        """Expert ranks: run steps until told to stop.  Returns device milliseconds between the timer marks."""
        w = self.worker
        ev0 = ev1 = None
        while True:
            msg = self._send(0)
            op, T = int(msg[0]), int(msg[1])
            if op == OP_STOP:
                break
            if op == OP_TIMER_START:
                torch.cuda.synchronize()
                ev0 = torch.cuda.Event(enable_timing=True)
                ev0.record()
                continue
            if op == OP_TIMER_STOP:
                ev1 = torch.cuda.Event(enable_timing=True)
                ev1.record()
                torch.cuda.synchronize()
                self.timer_ms = ev0.elapsed_time(ev1)
                continue
            if self.comm != "p2p":
                w.step(T)
            elif T not in self.graphs:
                w.step(T)                                   # first step of this size: eager, then capture for later
                torch.cuda.synchronize()
                self.graphs[T] = capture_expert_graph(w, T)
            else:
                self.graphs[T].replay()
        torch.cuda.synchronize()
        return self.timer_ms

    def check(self):
        st = self.engine.status if self.engine is not None else self.worker.status
        word = int(st[0])
        if word:
            from ..ops.native import decode_status
            raise RuntimeError(f"rank {self.rank}: device status {decode_status(word)}")

    def close(self):
        if self.block is not None:
            self.block.close()


def run_decode_bench_distributed(args, spec: ModelSpec, rank: int, world: int, local: int, clocks) -> dict:
    comm = getattr(args, "comm", "p2p")
    batch_total = getattr(args, "batch_total", 0) or args.batch_per_gpu * world
    # Data-parallel attention groups: by default two once there are four GPUs (GQA models over the peer-memory path);
    # MLA configs keep the single TP2 group their published layout names.
    groups = getattr(args, "attn_groups", 0) or (2 if (world >= 4 and comm == "p2p" and spec.attn.kind == "gqa" and batch_total % 2 == 0) else 1)
    if batch_total % groups:
        raise SystemExit(f"batch {batch_total} does not split over {groups} attention groups")
    batch = batch_total // groups                     # sequences served by each attention group
    ctx_pages = -(-(args.context + 4 * (args.steps + args.warmup) + 64) // PAGE)
    pages = batch * (ctx_pages + 1) + 2
    t0 = time.time()
    run = AfdRunner(spec, rank, world, local, t_max=max(16, batch), n_pages=pages, max_seqs=batch, max_pages_per_seq=ctx_pages + 1, comm=comm,
                    attn_groups=groups)
    use_graph = comm == "p2p"
    res = None
    if run.is_attn:
        eng = run.engine
        gen = BatchGenerator(eng, PagePool(pages))
        g = torch.Generator(device=eng.device).manual_seed(0)
        gen.seqs = []
        for _ in range(batch):
            s = SeqKV(); s.ensure(gen.pool, args.context + 1); s.length = args.context
            gen.seqs.append(s)
        for li in range(eng.kv.shape[0]):
            eng.kv[li].normal_(0, 1, generator=g)
        gen.last = torch.randint(0, spec.vocab, (batch,), generator=torch.Generator().manual_seed(0)).tolist()
        torch.cuda.synchronize()
        setup_s = time.time() - t0
        # end-to-end arm
        for _ in range(args.warmup):
            gen.decode_step(use_graph)
        torch.cuda.synchronize()
        gen.h2d_bytes = gen.d2h_bytes = 0
        t1 = time.perf_counter()
        for _ in range(args.steps):
            gen.decode_step(use_graph)
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t1
        # device arm
        kv_len = [s.length + 1 for s in gen.seqs]
        sh = StepShape(T=batch, n_seq=batch, max_q_len=1, n_logits=batch, attn_splits=eng.attn_splits_for(batch, 1, max(kv_len)))
        for _ in range(args.warmup):
            eng.run(sh, use_graph)
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clocks.start()
        time.sleep(0.2)
        torch.cuda.synchronize()
        run.control(OP_TIMER_START)          # expert ranks start their own device timers right before the first timed step
        ev0.record()
        for _ in range(args.steps):
            eng.run(sh, use_graph)
        ev1.record()
        torch.cuda.synchronize()
        dev_ms = ev0.elapsed_time(ev1)
        run.control(OP_TIMER_STOP)
        clk = clocks.stop()
        run.control(OP_STOP)
        run.check()
        launches = eng.launches_per_step
        h2d, d2h = gen.h2d_bytes // args.steps, gen.d2h_bytes // args.steps
    else:
        dev_ms = run.serve_loop()
        run.check()
        setup_s, e2e_s, clk, launches, h2d, d2h = 0.0, 0.0, None, run.worker.launches_per_step, 0, 0
    # max over ranks of the device time; launches summed over ranks
    t = torch.tensor([dev_ms, float(launches)], dtype=torch.float64, device=run.dev)
    tmax = t.clone(); dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    tsum = t.clone(); dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
    if rank == 0:
        ms = float(tmax[0])
        dep = run.dep
        res = {
            "metric": "decode_tokens_per_s", "value": round(batch_total * args.steps / (ms / 1e3), 2), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4),
            "higher_is_better": True, "scaling": "weak" if not getattr(args, "batch_total", 0) else "strong", "vs_baseline": None,
            "dtype": f"bf16 activations, {spec.quant.experts} experts / {spec.quant.dense} dense (dense runs as bf16 when the format has no kernel yet)",
            "data": "synthetic token ids, random-init weights, context KV random-filled",
            "config": {"model": spec.name + (f" (DEBUG {args.layers} layers: INVALID)" if args.layers else ""), "global_batch": batch_total,
                       "seq_len": args.context, "parallelism": f"afd {dep.describe()} ({comm})", "layers": spec.n_layers,
                       "l2": "inputs (weights + KV) far larger than L2; no flush needed", "setup_s": round(setup_s, 1)},
            "clocks": clk,
            "e2e": {"value": round(batch_total * args.steps / e2e_s, 2), "unit": "tokens/s", "ms_per_step": round(e2e_s * 1e3 / args.steps, 4),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(float(tsum[1])) * args.steps,
        }
    run.close()
    return res
