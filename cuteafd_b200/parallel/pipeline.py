"""Layer-range split: the decoder stack cut into consecutive stages, one per GPU, with the residual rows hopping from stage to stage
over peer memory.

Each stage is an ordinary engine over its slice of the layers (its own paged KV cache for those layers only), so everything the
single-GPU engine does - graphs, split-KV attention, fused MoE kernels - runs unchanged inside a stage.  The first stage embeds the
tokens, the last one runs the head and selects tokens.  A hop is one `push_bytes` of the step's rows into the next stage's landing
buffer with a release flag carrying the step number; the receiving stage's first kernel waits for that flag (bounded: a missing
flag becomes a status word) and copies the rows into its residual stream in the same launch (`wait_add` with a zero addend).
Every stage stages the same step inputs (tokens, positions, page tables for ITS cache), so only hidden rows cross the link:
T x hidden x 2 bytes per hop.

One step is in flight at a time: the selected tokens come from the last stage, and the drivers exchange them (a broadcast through
`torch.distributed`, or directly in the single-process form) before any stage starts the next step; that ordering is also what
makes a single landing buffer per stage sufficient.  The split exists to fit a model on GPUs whose memory one engine would
exceed; it does not overlap the stages of one step (the attention / expert layouts of `parallel/afd.py` are the throughput path).

Reference: rust/crates/cuteafd-loader/src/placement/residual.rs (layer ranges per device), rust/crates/cuteafd-daemon/src/shared/peer_split
(hidden-state hops between the two coordinator GPUs, `hops.rs`), families/deepseek_v4/engine.rs (`layer_device`, hop at the boundary).
"""
from __future__ import annotations

import torch

from ..config import ModelSpec
from ..engine.engine import Engine, StepShape
from ..engine.kv import PagePool, SeqKV
from ..models.weights import DeviceWeights
from . import peer_ops
from .symm import SymmetricBlock


def stage_ranges(n_layers: int, n_stages: int, period: int = 1) -> list[tuple[int, int]]:
    """Consecutive layer ranges, as even as the layer period allows (hybrid stacks repeat every `period` layers: cuts sit on multiples)."""
    units = n_layers // period
    if n_stages < 1 or units < n_stages:
        raise ValueError(f"{n_layers} layers (period {period}) cannot be cut into {n_stages} stages")
    cuts = [round(i * units / n_stages) * period for i in range(n_stages)] + [n_layers]
    return [(cuts[i], cuts[i + 1]) for i in range(n_stages)]


def stage_spec(spec: ModelSpec, lo: int, hi: int) -> ModelSpec:
    """The spec of layers [lo, hi) as a stack of its own: per-layer programs that depend on the layer index keep their meaning."""
    a = spec.attn
    period = max(a.full_every or 1, a.linear_every or 1)
    if lo % period:
        raise ValueError(f"stage boundary {lo} inside a period of {period} layers")
    if spec.hyper_streams or spec.mtp_layers or spec.engram_layers:
        raise NotImplementedError("layer-range split: single-stream stacks without MTP module or n-gram memory")
    import dataclasses
    moe = dataclasses.replace(spec.moe, first_dense=max(0, min(spec.moe.first_dense - lo, hi - lo)))
    return spec.replace(n_layers=hi - lo, moe=moe, name=f"{spec.name}[{lo}:{hi}]")


def stage_masters(masters: dict, lo: int, hi: int) -> dict:
    out = {k: v for k, v in masters.items() if k not in ("layers", "mtp")}
    out["layers"] = masters["layers"][lo:hi]
    return out


def hop_regions(spec: ModelSpec, t_cap: int) -> dict:
    return {"hop": t_cap * spec.hidden * 2, "flags": 256}


class StageLink:
    """What the engine calls at its ends (`Engine.stage`)."""

    def __init__(self, block, rank: int, n_stages: int, spec: ModelSpec, t_cap: int, device):
        self.block, self.rank, self.first, self.last = block, rank, rank == 0, rank == n_stages - 1
        self.H, self.t_cap = spec.hidden, t_cap
        self.ctl = torch.zeros(4, dtype=torch.int32, device=device)
        self.done = torch.zeros(4, dtype=torch.int32, device=device)
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.zero = torch.zeros(t_cap, spec.hidden, dtype=torch.bfloat16, device=device)
        self.landing = block.local("hop", torch.bfloat16, (t_cap, spec.hidden))
        self.hop_bytes = 0

    def begin(self):
        peer_ops.step_begin(self.ctl)

    def receive(self, x: torch.Tensor, T: int) -> int:
        flag = self.block.peer_ptr(self.rank, "flags", 0)
        peer_ops.wait_add(self.zero, self.landing, None, x, T * self.H, 0, flag, self.ctl, 0, self.status)
        return 1

    def send(self, x: torch.Tensor, T: int) -> int:
        if T > self.t_cap:
            raise ValueError(f"layer-range split: {T} rows in a step (hop buffers hold {self.t_cap})")
        nxt = self.rank + 1
        flag = self.block.peer_ptr(nxt, "flags", 0)
        peer_ops.push_bytes(x, self.block.peer_ptr(nxt, "hop", 0), T * self.H * 2, flag, self.ctl, 0, self.done[0:1])
        peer_ops.note_published([flag])
        self.hop_bytes += T * self.H * 2
        return 1


class StageEngine(Engine):
    """Engine over layers [lo, hi) of a model; `program` opens every step with the step counter the hop flags carry."""

    def __init__(self, spec: ModelSpec, lo: int, hi: int, link: StageLink, device, *, masters: dict | None = None, seed: int = 1, **kw):
        local = stage_spec(spec, lo, hi)
        dw = (DeviceWeights.from_masters(local, stage_masters(masters, lo, hi), device) if masters is not None
              else DeviceWeights.random(local, device, seed=seed + lo))
        super().__init__(dw, device=device, **kw)
        self.full_spec, self.lo, self.hi, self.stage = spec, lo, hi, link

    def _forward_single(self, sh: StepShape):
        self.stage.begin()
        lane = super()._forward_single(sh)
        self.launches_per_step += 1
        return lane

    def check_status(self):
        super().check_status()
        word = int(self.stage.status[0])
        if word:
            from ..ops.native import decode_status
            raise RuntimeError(f"stage {self.stage.rank}: hop status {decode_status(word)}")


class PipelineRank:
    """One process of a layer-range split (one stage per GPU).  Every rank drives the same sequence of steps with the same inputs;
    the tokens the last stage selects are broadcast to all ranks after each step."""

    def __init__(self, spec: ModelSpec, rank: int, world: int, device, *, n_pages: int, max_seqs: int, max_pages_per_seq: int, t_cap: int = 4096,
                 masters: dict | None = None, group=None, block=None):
        a = spec.attn
        self.spec, self.rank, self.world, self.device = spec, rank, world, torch.device(device)
        self.ranges = stage_ranges(spec.n_layers, world, max(a.full_every or 1, a.linear_every or 1))
        self.block = block if block is not None else SymmetricBlock(hop_regions(spec, t_cap), device, group, rank, world)
        self.link = StageLink(self.block, rank, world, spec, t_cap, device)
        lo, hi = self.ranges[rank]
        self.engine = StageEngine(spec, lo, hi, self.link, device, masters=masters, n_pages=n_pages, max_seqs=max_seqs,
                                  max_pages_per_seq=max_pages_per_seq)
        self.group = group

    def exchange_tokens(self, toks: list[int], n: int) -> list[int]:
        """The last stage's selection, on every rank."""
        if self.world == 1:
            return toks
        import torch.distributed as dist
        t = torch.tensor(toks if self.link.last else [0] * n, dtype=torch.int32, device=self.device)
        dist.broadcast(t, src=self.world - 1, group=self.group)
        return t.tolist()


def generate_pipeline(ranks: list, prompts: list[list[int]], n_new: int, use_graph: bool = True) -> list[list[int]]:
    """Greedy generation over a layer-range split.  `ranks`: the `PipelineRank` objects this process drives - all of them in the
    single-process form (stages run one after the other in one stream: the tests' form on one GPU), or the process's own rank in
    a multi-process run, where the token exchange is the broadcast."""
    from ..engine.generate import BatchGenerator
    gens = [BatchGenerator(r.engine, PagePool(r.engine.n_pages)) for r in ranks]
    multi = len(ranks) == 1 and ranks[0].world > 1
    outs = [[] for _ in prompts]

    def readback(lane_tokens: list[list[int]]) -> list[int]:
        toks = lane_tokens[-1]
        return ranks[0].exchange_tokens(toks, len(prompts)) if multi else toks

    # prefill: every stage stages the same whole-prompt step (its own page tables), stage by stage
    shs = [g.plan_prefill_all(prompts) for g in gens]
    lanes = [r.engine.run(sh, use_graph=False) for r, sh in zip(ranks, shs)]
    last = readback([g._readback(l, len(prompts)) for g, l in zip(gens, lanes)])
    for g in gens:
        for s, n in zip(g.seqs, g._prompt_lens):
            s.length = n
        g.last = list(last)
    for i, t in enumerate(last):
        outs[i].append(t)
    for _ in range(n_new - 1):
        shs = [g.plan_decode() for g in gens]
        lanes = [r.engine.run(sh, use_graph=use_graph) for r, sh in zip(ranks, shs)]
        toks = readback([g._readback(l, len(prompts)) for g, l in zip(gens, lanes)])
        for g in gens:
            for s in g.seqs:
                s.length += 1
            g.last = list(toks)
        for i, t in enumerate(toks):
            outs[i].append(t)
    for r in ranks:
        r.engine.check_status()
    for g in gens:
        g.release()
    return outs
