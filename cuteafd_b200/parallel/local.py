"""Several ranks of a multi-GPU layout run as ONE process on ONE GPU.

Kernels that wait on one another must never run as separate launches that depend on each other's progress on one GPU.
`LocalWorld` therefore never lets a waiting kernel into the stream before its producers: every rank's step is a program
(generator) that yields the peer flag addresses it is about to wait for, and the scheduler resumes a program only when all
those flags were published by launches that are already in the stream (`peer_ops.PUBLISHED`).  In-order execution then
guarantees every wait is satisfied the moment its kernel starts.  If no program can be resumed the protocol itself is
wrong (a wait without a matching push) and the scheduler raises instead of launching anything that could spin.

"Peer memory" is ordinary device memory of the same GPU: every rank gets its own block with the layout of
`SymmetricBlock`, and peer pointers are plain addresses of the other ranks' blocks.  What runs is the real kernels and
the real flag protocol of `parallel.afd`; only NVLink is missing.

Reference: host-side order fixtures of the peer exchange, shared/peer_split/order/{fixtures,host}.rs (push-before-wait
proven on the host); here the same property is enforced while real kernels run.
"""
from __future__ import annotations

import torch

from ..config import Deployment, ModelSpec
from ..engine.engine import Lane, StepShape
from ..ops import KIND_BY_NAME
from . import peer_ops
from .afd import AttnRankEngine, ExpertRankWorker, LanePlan, MlaAttnRankEngine, block_regions
from .symm import Region


class LocalBlocks:
    """`world` blocks with the layout of a SymmetricBlock, all on one device; `view(rank)` is rank's SymmetricBlock stand-in."""

    def __init__(self, regions: dict, device, world: int):
        self.regions, off = {}, 0
        for name, nbytes in regions.items():
            self.regions[name] = Region(off, nbytes)
            off += -(-nbytes // 256) * 256
        self.nbytes = max(off, 256)
        self.bufs = [torch.zeros(self.nbytes, dtype=torch.uint8, device=device) for _ in range(world)]
        self.base = [b.data_ptr() for b in self.bufs]
        self.world = world

    def view(self, rank: int) -> "LocalBlockView":
        return LocalBlockView(self, rank)


class LocalBlockView:
    def __init__(self, blocks: LocalBlocks, rank: int):
        self.blocks, self.rank, self.world, self.regions, self.base = blocks, rank, blocks.world, blocks.regions, blocks.base

    def local(self, name: str, dtype=torch.uint8, shape=None) -> torch.Tensor:
        r = self.regions[name]
        t = self.blocks.bufs[self.rank][r.offset:r.offset + r.nbytes].view(dtype)
        return t.view(*shape) if shape is not None else t

    def peer_ptr(self, rank: int, name: str, byte_offset: int = 0) -> int:
        return self.base[rank] + self.regions[name].offset + byte_offset

    def close(self):
        pass


class Deadlock(RuntimeError):
    pass


def run_programs(programs: dict) -> dict:
    """Runs {name: generator} to completion under the publish-before-wait rule.  Returns {name: last Lane yielded}."""
    peer_ops.PUBLISHED = set()
    try:
        waiting = {}                    # name -> flag addresses it needs before it may continue
        results, live = {}, dict(programs)
        for name in live:
            waiting[name] = []
        while live:
            progressed = False
            for name in list(live):
                if any(a not in peer_ops.PUBLISHED for a in waiting[name]):
                    continue
                progressed = True
                try:
                    item = next(live[name])
                except StopIteration:
                    del live[name]
                    continue
                if isinstance(item, Lane):
                    results[name] = item
                    waiting[name] = []
                else:
                    waiting[name] = list(item)
            if not progressed:
                missing = {n: [hex(a) for a in w if a not in peer_ops.PUBLISHED][:4] for n, w in waiting.items() if n in live}
                raise Deadlock(f"no rank can continue: every live program waits for a flag nobody has published: {missing}")
        return results
    finally:
        peer_ops.PUBLISHED = None


class LocalWorld:
    """All ranks of a deployment on one device.  `engines[r]` is rank r's attention engine (None for a pure expert rank),
    `workers[r]` its expert worker (None for a pure attention rank)."""

    def __init__(self, spec: ModelSpec, plan: LanePlan, device, *, n_pages: int, max_seqs: int, max_pages_per_seq: int, masters: dict | None = None,
                 seed: int = 1, act_gs: float = 1.0 / 64):
        dep: Deployment = plan.dep
        self.spec, self.plan, self.dep = spec, plan, dep
        kind = KIND_BY_NAME[spec.quant.experts]
        self.blocks = LocalBlocks(block_regions(spec, plan, kind), device, dep.world)
        self.engines, self.workers = {}, {}
        cls = MlaAttnRankEngine if spec.attn.kind == "mla" else AttnRankEngine
        for r in range(dep.world):
            blk = self.blocks.view(r)
            if r in dep.attn_ranks:
                self.engines[r] = cls(spec, plan, r, device, n_pages=n_pages, max_seqs=max_seqs, max_pages_per_seq=max_pages_per_seq, comm="p2p",
                                      block=blk, expert_kind=kind, seed=seed, masters=masters, act_gs=act_gs)
            if r in dep.expert_ranks:
                self.workers[r] = ExpertRankWorker(spec, plan, r, device, comm="p2p", block=blk, seed=seed, masters=masters, act_gs=act_gs)
            if dep.colocated:
                self.engines[r].local_worker = self.workers[r]

    def step(self, shapes: dict) -> dict:
        """One main-model step: `shapes[r]` is the StepShape of attention rank r (its inputs already set with `set_inputs`)."""
        progs = {("attn", r): e.program(shapes[r]) for r, e in self.engines.items()}
        if not self.dep.colocated:
            progs.update({("exp", r): w.step_program() for r, w in self.workers.items()})
        out = run_programs(progs)
        return {r: out[("attn", r)] for r in self.engines}

    def mtp_step(self, depth: int, shapes: dict, prev_hidden: dict) -> dict:
        progs = {("attn", r): e.mtp_program(depth, shapes[r], prev_hidden[r]) for r, e in self.engines.items()}
        if not self.dep.colocated:
            li = self.spec.n_layers + depth
            progs.update({("exp", r): w.step_program([li]) for r, w in self.workers.items()})
        out = run_programs(progs)
        return {r: out[("attn", r)] for r in self.engines}

    def check(self):
        from ..ops.native import decode_status
        for r, e in self.engines.items():
            if int(e.status[0]):
                raise RuntimeError(f"attention rank {r}: device status {decode_status(int(e.status[0]))}")
        for r, w in self.workers.items():
            if int(w.status[0]):
                raise RuntimeError(f"expert rank {r}: device status {decode_status(int(w.status[0]))}")


def generate_local(world: LocalWorld, prompts_by_group: list, n_new: int) -> list:
    """Greedy generation on a LocalWorld: group g serves `prompts_by_group[g]` (an empty list = an idle group, which still
    takes part in every step).  Returns the new tokens per group and prompt."""
    from ..engine.generate import BatchGenerator
    from ..engine.kv import PagePool
    dep = world.dep
    gens = {r: BatchGenerator(e, PagePool(e.n_pages)) for r, e in world.engines.items()}
    idle = StepShape(0, 0, 1, 0, 1)
    out = [[[] for _ in prompts_by_group[g]] for g in range(dep.attn_groups)]

    def run(plan, commit):
        shapes = {}
        for r, g in gens.items():
            grp = dep.group_of(r)
            if prompts_by_group[grp]:
                shapes[r] = plan(g, grp)
            else:
                g.eng._ensure_meta(16)
                shapes[r] = idle
        lanes = world.step(shapes)
        for r, g in gens.items():
            grp = dep.group_of(r)
            if prompts_by_group[grp]:
                toks = commit(g, lanes[r])
                if r == dep.group_ranks(grp)[0]:
                    for o, t in zip(out[grp], toks):
                        o.append(t)

    run(lambda g, grp: g.plan_prefill_all(prompts_by_group[grp]), lambda g, lane: g.commit_prefill_all(lane))
    for _ in range(n_new - 1):
        run(lambda g, grp: g.plan_decode(), lambda g, lane: g.commit_decode(lane))
    world.check()
    return out
