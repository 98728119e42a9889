"""Multi-rank driver for the attention/expert layouts: roles, the step mailbox that tells expert ranks what to run, and the
distributed decode benchmark.

Split layouts (disjoint attention / expert ranks): before every step that really executes, the attention leader posts
(op, argument) into a shared-memory mailbox (`parallel.mailbox`); expert ranks sit in `serve_loop`, replay their captured
step graph per message (the step's shape travels on the device: each lane's token count is written next to its rows, so ONE
graph serves every step size) and leave on OP_STOP.  Colocated layout: every rank runs its own experts inside its own step,
there is nobody to tell.  The data path never touches the host: rows, routing tables and flags move through peer memory.
(Reference: worker selection + per-wave requests, cuteafd-transport/src/worker_selection.rs, expert.rs:201-376; here the
"request" shrinks to two integers in shared memory.)
"""
from __future__ import annotations

import os
import time

import torch
import torch.distributed as dist

from ..config import ModelSpec, deployment_by_name
from ..engine.engine import PAGE, StepShape
from ..engine.generate import BatchGenerator
from ..engine.kv import PagePool, SeqKV
from ..ops import KIND_BY_NAME
from .afd import AttnRankEngine, ExpertRankWorker, LanePlan, MlaAttnRankEngine, capture_expert_graph, make_block
from .mailbox import Mailbox

OP_STOP, OP_STEP, OP_TIMER_START, OP_TIMER_STOP, OP_MTP, OP_INPUTS = 0, 1, 2, 3, 4, 5


class AfdRunner:
    def __init__(self, spec: ModelSpec, rank: int, world: int, local: int, *, t_cap: int, n_pages: int, max_seqs: int,
                 max_pages_per_seq: int, comm: str = "p2p", seed: int = 1, layout: str = "split", attn_groups: int = 1, n_micro: int = 1,
                 merged: bool | None = None, masters: dict | None = None, expert_tp: bool = False):
        self.spec, self.rank, self.world = spec, rank, world
        self.dev = torch.device("cuda", local)
        self.dep = dep = deployment_by_name(layout, world, attn_groups)
        if comm == "nccl" and (dep.colocated or n_micro > 1):
            raise ValueError("the NCCL-only baseline runs the split layout with one micro-batch")
        self.plan = LanePlan(dep, t_cap=t_cap, n_micro=n_micro, merged=dep.colocated if merged is None else merged, expert_tp=expert_tp)
        self.comm = comm
        self.tp_group = dist.new_group(list(dep.attn_ranks)) if comm == "nccl" else None
        self.is_attn, self.is_expert = rank in dep.attn_ranks, rank in dep.expert_ranks
        self.root = dep.attn_ranks[0]
        kind = KIND_BY_NAME[spec.quant.experts]
        self.block = make_block(spec, self.plan, kind, rank, self.dev, None) if comm == "p2p" else None
        # step mailbox (split layouts only)
        self.mail = None
        if not dep.colocated:
            name = [f"cuteafd_{os.getpid()}_{int(time.time() * 1e3) & 0xFFFFFF}" if rank == self.root else None]
            dist.broadcast_object_list(name, src=self.root)
            if rank == self.root:
                self.mail = Mailbox(name[0], create=True, slots=32, payload_bytes=1 << 20)
            dist.barrier()
            if rank != self.root:
                self.mail = Mailbox(name[0], create=False, slots=32, payload_bytes=1 << 20)
        self.engine = self.worker = None
        if self.is_attn:
            cls = MlaAttnRankEngine if spec.attn.kind == "mla" else AttnRankEngine
            self.engine = cls(spec, self.plan, rank, self.dev, n_pages=n_pages, max_seqs=max_seqs, max_pages_per_seq=max_pages_per_seq, comm=comm,
                              block=self.block, expert_kind=kind, seed=seed, masters=masters)
            self.engine.tp_group = self.tp_group
            if not dep.colocated:
                self.engine.on_real_step = self._announce
                self.engine.on_mtp_step = self._announce_mtp
        if self.is_expert:
            self.worker = ExpertRankWorker(spec, self.plan, rank, self.dev, comm=comm, block=self.block, seed=seed, masters=masters)
            if dep.colocated:
                self.engine.local_worker = self.worker
        self.graphs: dict = {}
        self.timer_ms = 0.0
        dist.barrier()

    # ---- control channel (split layouts)
    def _post(self, op: int, a: int = 0, b: int = 0):
        if self.mail is not None and self.rank == self.root:
            self.mail.post(op, a, b)

    def _announce(self, sh: StepShape, replay: bool = False):
        if self.mail is not None and self.rank == self.root:
            import numpy as np
            self.mail.post(OP_STEP, sh.T, 1 if replay else 0,
                           np.array([sh.T, sh.n_seq, sh.max_q_len, sh.n_logits, sh.attn_splits, int(sh.uniform)], dtype=np.int64))

    def mirror_inputs(self, on: bool = True):
        """Leader of a serving deployment: forward every step's packed input block to the attention ranks that mirror it (its
        tensor-parallel partner).  Benchmarks and self-tests run the same host code on every attention rank and need none."""
        if self.engine is not None and self.rank == self.root:
            self.engine.on_inputs = (lambda block: self.mail.post(OP_INPUTS, block.numel(), 0, block.numpy())) if on else None

    def follow_loop(self, timeout_s: float = 3600.0):
        """Attention ranks other than the leader, serving: mirror the leader's steps one execution at a time."""
        import numpy as np
        eng = self.engine
        while True:
            op, a, b, payload = self.mail.read(timeout_s)
            if op == OP_STOP:
                break
            if op == OP_INPUTS:
                eng.load_inputs(torch.from_numpy(np.frombuffer(payload, dtype=np.int32).copy()))
            elif op == OP_STEP:
                f = np.frombuffer(payload, dtype=np.int64)
                sh = StepShape(T=int(f[0]), n_seq=int(f[1]), max_q_len=int(f[2]), n_logits=int(f[3]), attn_splits=int(f[4]), uniform=bool(f[5]))
                eng.execute(sh, bool(b))
        torch.cuda.synchronize()

    def _announce_mtp(self, depth: int, sh: StepShape):
        self._post(OP_MTP, sh.T, depth)

    def control(self, op: int):
        """Attention leader: forward a timer / stop op to the expert ranks (a no-op on other ranks and in the colocated layout)."""
        self._post(op)

    def serve_loop(self, timeout_s: float = 600.0):
        """Expert ranks of a split layout: run steps until told to stop.  Returns device milliseconds between the timer marks."""
        w = self.worker
        ev0 = ev1 = None
        while True:
            op, a, b, _ = self.mail.read(timeout_s)
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
            if op == OP_INPUTS:
                continue                                    # step inputs concern the attention ranks only
            layers = None if op == OP_STEP else [self.spec.n_layers + b]
            if self.comm != "p2p":
                w.step_nccl(a, layers)
                continue
            key = "main" if op == OP_STEP else ("mtp", b)
            if key not in self.graphs:
                w.step(layers)                              # first step of this kind: eager, then captured for later
                torch.cuda.synchronize()
                self.graphs[key] = capture_expert_graph(w, layers)
            else:
                self.graphs[key].replay()
        torch.cuda.synchronize()
        return self.timer_ms

    def check(self):
        from ..ops.native import decode_status
        for who in (self.engine, self.worker):
            if who is not None and int(who.status[0]):
                raise RuntimeError(f"rank {self.rank}: device status {decode_status(int(who.status[0]))}")

    def close(self):
        if self.block is not None:
            self.block.close()
        if self.mail is not None:
            self.mail.close()


def default_layout(spec: ModelSpec, world: int, comm: str) -> dict:
    """Layout a benchmark uses when none is named: colocated (data-parallel attention + expert-parallel FFN on every GPU: nothing
    idles, every expert's weights stream once per layer for the whole batch, and attention splits its KV range over the SMs the
    small per-GPU batch leaves free).  Measured on 4 GPUs with the DeepSeek-V3 shape at batch 64 @ 8k (16 layers): 9.8 ms per
    step colocated against 25.0 ms on attention TP2 + EP2 with two micro-batches.  An MLA model on fewer than four GPUs keeps the
    split (its weights do not fit twice).  The NCCL-only arm always runs the split."""
    if comm == "nccl":
        return {"layout": "split", "attn_groups": 1, "n_micro": 1}
    if spec.attn.kind == "mla" and world < 4:
        return {"layout": "split", "attn_groups": 1, "n_micro": 1}
    return {"layout": "colocated", "attn_groups": world, "n_micro": 1}


def run_decode_bench_distributed(args, spec: ModelSpec, rank: int, world: int, local: int, clocks) -> dict:
    comm = getattr(args, "comm", "p2p")
    lay = default_layout(spec, world, comm)
    if getattr(args, "layout", None):
        lay["layout"] = args.layout
        if args.layout == "split":
            lay["attn_groups"] = 1
            if spec.attn.kind == "mla" and world >= 4 and comm == "p2p":
                lay["n_micro"] = 2         # the named split hides the expert round trip behind a second micro-batch
    if getattr(args, "attn_groups", 0) and lay["layout"] == "split":
        lay["attn_groups"] = args.attn_groups
    if getattr(args, "n_micro", 0):
        lay["n_micro"] = args.n_micro
    dep = deployment_by_name(lay["layout"], world, lay["attn_groups"])
    groups = dep.attn_groups
    batch_total = getattr(args, "batch_total", 0) or args.batch_per_gpu * world
    if batch_total < groups:
        groups_used = batch_total            # fewer sequences than groups (batch 1): the other groups idle
    else:
        groups_used = groups
    base, extra = divmod(batch_total, groups_used)
    ctx_pages = -(-(args.context + 4 * (args.steps + args.warmup) + 64) // PAGE)
    my_group = dep.group_of(rank) if rank in dep.attn_ranks else -1
    batch = (base + (1 if my_group < extra else 0)) if 0 <= my_group < groups_used else 0
    max_batch = base + (1 if extra else 0)
    pages = max(batch, 1) * (ctx_pages + 1) + 2
    t_cap = max(16, -(-max_batch // lay["n_micro"]))
    t0 = time.time()
    run = AfdRunner(spec, rank, world, local, t_cap=t_cap, n_pages=pages, max_seqs=max(max_batch, 1), max_pages_per_seq=ctx_pages + 1, comm=comm,
                    layout=lay["layout"], attn_groups=lay["attn_groups"], n_micro=lay["n_micro"], expert_tp=bool(getattr(args, "expert_tp", False)))
    use_graph = comm == "p2p"
    res = None
    dev_ms, setup_s, e2e_s, clk, launches, h2d, d2h = 0.0, 0.0, 0.0, None, 0, 0, 0
    if run.is_attn:
        eng = run.engine
        gen = BatchGenerator(eng, PagePool(pages))
        g = torch.Generator(device=eng.device).manual_seed(rank)
        gen.seqs = []
        for _ in range(batch):
            s = SeqKV(); s.ensure(gen.pool, args.context + 1); s.length = args.context
            gen.seqs.append(s)
        for li in range(eng.kv.shape[0]):
            eng.kv[li].normal_(0, 1, generator=g)
        gen.last = torch.randint(0, spec.vocab, (max(batch, 1),), generator=torch.Generator().manual_seed(my_group)).tolist()[:batch]
        torch.cuda.synchronize()
        setup_s = time.time() - t0
        idle = StepShape(0, 0, 1, 0, 1)
        # colocated ranks line up on the host before each phase; in a split layout the expert ranks are already serving (they
        # cannot join a host barrier) and the attention ranks meet through them every layer anyway
        sync = dist.barrier if dep.colocated else (lambda: None)

        def e2e_step():
            if batch:
                gen.decode_step(use_graph)
            else:
                eng._ensure_meta(16)
                eng.run(idle, use_graph)
        # end-to-end arm
        sync()
        for _ in range(args.warmup):
            e2e_step()
        torch.cuda.synchronize()
        sync()
        gen.h2d_bytes = gen.d2h_bytes = 0
        t1 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t1
        # device arm
        if batch:
            kv_len = [s.length + 1 for s in gen.seqs]
            sh = StepShape(T=batch, n_seq=batch, max_q_len=1, n_logits=batch, attn_splits=eng.attn_splits_for(batch, 1, max(kv_len)), uniform=True)
        else:
            sh = idle
        for _ in range(args.warmup):
            eng.run(sh, use_graph)
        torch.cuda.synchronize()
        sync()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if rank == 0:
            clocks.start()
        time.sleep(0.2)
        torch.cuda.synchronize()
        sync()
        run.control(OP_TIMER_START)          # expert ranks start their own device timers right before the first timed step
        ev0.record()
        for _ in range(args.steps):
            eng.run(sh, use_graph)
        ev1.record()
        torch.cuda.synchronize()
        dev_ms = ev0.elapsed_time(ev1)
        run.control(OP_TIMER_STOP)
        if rank == 0:
            clk = clocks.stop()
        run.control(OP_STOP)
        run.check()
        launches = eng.launches_per_step + (run.worker.launches_per_step if run.worker is not None else 0)
        h2d, d2h = gen.h2d_bytes // args.steps, gen.d2h_bytes // args.steps
    else:
        dev_ms = run.serve_loop()
        run.check()
        launches = run.worker.launches_per_step
    # max over ranks of the device and wall times; launches and copied bytes summed over ranks
    t = torch.tensor([dev_ms, e2e_s, float(launches), float(h2d), float(d2h)], dtype=torch.float64, device=run.dev)
    tmax = t.clone(); dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    tsum = t.clone(); dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
    if rank == 0:
        ms, e2e = float(tmax[0]), float(tmax[1])
        res = {
            "metric": "decode_tokens_per_s", "value": round(batch_total * args.steps / (ms / 1e3), 2), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4),
            "higher_is_better": True, "scaling": "weak" if not getattr(args, "batch_total", 0) else "strong", "vs_baseline": None,
            "dtype": f"bf16 activations, {spec.quant.experts} experts / {spec.quant.dense} dense",
            "data": "synthetic token ids, random-init weights, context KV random-filled",
            "config": {"model": spec.name + (f" (DEBUG {args.layers} layers: INVALID)" if args.layers else ""), "global_batch": batch_total,
                       "seq_len": args.context, "parallelism": f"{dep.describe()}, {lay['n_micro']} micro-batch(es){', expert TP' if run.plan.expert_tp else ''} ({comm})", "layers": spec.n_layers,
                       "l2": "inputs (weights + KV) far larger than L2; no flush needed", "setup_s": round(setup_s, 1)},
            "clocks": clk,
            "e2e": {"value": round(batch_total * args.steps / e2e, 2), "unit": "tokens/s", "ms_per_step": round(e2e * 1e3 / args.steps, 4),
                    "h2d_bytes_per_step": int(float(tsum[3])), "d2h_bytes_per_step": int(float(tsum[4]))},
            "gpu_launches": int(float(tsum[2])) * args.steps,
        }
    run.close()
    return res
