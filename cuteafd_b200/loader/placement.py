"""Placement solver for one NVSwitch node: which rank holds which weights, how big the KV pool can be.

Order of decisions (same as the reference: pool first, then graphs/workspaces, then expert placement;
cuteafd-loader/src/placement/mod.rs:7-10, placement/solve.rs): every rank reserves headroom and workspaces;
attention ranks take the dense backbone (attention / shared experts / dense FFN split over TP, embeddings + head,
router) and give what is left to the KV pool; expert ranks take an equal share of routed experts; a layout that
does not fit is reported with the shortfall per rank instead of raising.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..config import Deployment, ModelSpec, default_deployment

GIB = 1 << 30


@dataclass
class RankPlan:
    rank: int
    role: str
    weights: dict = field(default_factory=dict)     # category -> bytes
    workspace: int = 0
    reserve: int = 0
    kv_pool: int = 0
    shortfall: int = 0

    @property
    def weight_bytes(self) -> int:
        return int(sum(self.weights.values()))

    @property
    def total(self) -> int:
        return self.weight_bytes + self.workspace + self.reserve + self.kv_pool


@dataclass
class Layout:
    deployment: Deployment
    ranks: list
    pool_tokens: int
    max_context: int
    fits: bool
    notes: list = field(default_factory=list)

    def table(self) -> str:
        lines = [f"{'rank':>4} {'role':<14} {'weights GiB':>12} {'kv GiB':>8} {'work GiB':>9} {'total GiB':>10} {'short GiB':>10}"]
        for r in self.ranks:
            lines.append(f"{r.rank:>4} {r.role:<14} {r.weight_bytes / GIB:>12.1f} {r.kv_pool / GIB:>8.1f} {r.workspace / GIB:>9.1f} "
                         f"{r.total / GIB:>10.1f} {r.shortfall / GIB:>10.1f}")
        lines.append(f"pool tokens: {self.pool_tokens}   fits: {self.fits}")
        lines += [f"note: {n}" for n in self.notes]
        return "\n".join(lines)


def solve(spec: ModelSpec, world: int = 8, gpu_bytes: int = 180 * GIB, reserve_bytes: int = 6 * GIB, workspace_bytes: int = 4 * GIB,
          pool_tokens: int = 0, max_batch_rows: int = 4096, deployment: Deployment | None = None) -> Layout:
    dep = deployment or default_deployment(world)
    wb = spec.weight_bytes()
    plans, notes = [], []
    attn_share = (wb["attention"] + wb["shared_experts"] + wb["dense_ffn"]) / dep.tp
    replicated = wb["router"] + wb["embed_head"]
    routed_share = wb["routed_experts"] * (-(-spec.moe.n_experts // max(1, dep.ep))) / max(1, spec.moe.n_experts)   # largest range
    act = max_batch_rows * spec.hidden * 2 * 24 + max_batch_rows * spec.vocab * 4      # activations + logits rows
    for r in range(dep.world):
        is_attn, is_exp = r in dep.attn_ranks, r in dep.expert_ranks
        p = RankPlan(r, "attention" if is_attn and not is_exp else ("experts" if is_exp and not is_attn else "both"),
                     workspace=workspace_bytes + (act if is_attn else max_batch_rows * spec.moe.top_k * spec.hidden * 6), reserve=reserve_bytes)
        if is_attn:
            p.weights["dense_backbone"] = int(attn_share)
            p.weights["router_embed_head"] = int(replicated)
        if is_exp:
            p.weights["routed_experts"] = int(routed_share)
        plans.append(p)
    kv_tok_rank = spec.kv_bytes_per_token() / (dep.tp if spec.attn.kind == "gqa" else 1)    # MLA latent is replicated over TP
    tokens_fit = []
    for p in plans:
        free = gpu_bytes - p.weight_bytes - p.workspace - p.reserve
        if free < 0:
            p.shortfall = -free
        elif p.role != "experts":
            tokens_fit.append(int(free // kv_tok_rank))
    fits = all(p.shortfall == 0 for p in plans)
    auto_tokens = min(tokens_fit) if tokens_fit else 0
    tokens = auto_tokens if pool_tokens <= 0 else pool_tokens
    if pool_tokens > auto_tokens:
        fits = False
        notes.append(f"requested pool of {pool_tokens} tokens exceeds the {auto_tokens} that fit")
    tokens -= tokens % 64
    for p in plans:
        if p.role != "experts":
            p.kv_pool = int(tokens * kv_tok_rank)
    if not fits:
        for p in plans:
            if p.shortfall:
                notes.append(f"rank {p.rank} ({p.role}) is short {p.shortfall / GIB:.1f} GiB")
    if dep.ep and spec.moe.n_experts % dep.ep:
        notes.append(f"{spec.moe.n_experts} experts over {dep.ep} expert ranks: uneven ranges of "
                     f"{spec.moe.n_experts // dep.ep} or {spec.moe.n_experts // dep.ep + 1} experts")
    return Layout(dep, plans, max(tokens, 0), min(spec.max_context, max(tokens, 0)), fits, notes)


def solve_stages(spec: ModelSpec, n_stages: int, gpu_bytes: int = 180 * GIB, reserve_bytes: int = 6 * GIB, workspace_bytes: int = 4 * GIB,
                 pool_tokens: int = 0, max_batch_rows: int = 4096) -> Layout:
    """Layer-range split (`parallel/pipeline.py`): consecutive layer ranges, one per GPU; every stage holds all weights of its layers
    and the KV cache of those layers only; the first stage adds the embedding, the last one the head.  The pool is what the tightest
    stage can hold.  (Reference: cuteafd-loader/src/placement/residual.rs: layer ranges per device.)"""
    from ..parallel.pipeline import stage_ranges
    a = spec.attn
    ranges = stage_ranges(spec.n_layers, n_stages, max(a.full_every or 1, a.linear_every or 1))
    wb = spec.weight_bytes()
    per_layer = (wb["attention"] + wb["shared_experts"] + wb["dense_ffn"] + wb["routed_experts"] + wb["router"]) / spec.n_layers
    embed = wb["embed_head"] / (1 if spec.tie_embeddings else 2)
    kv_layer = spec.kv_bytes_per_token() / spec.n_layers
    act = max_batch_rows * spec.hidden * 2 * 24
    plans, tokens_fit = [], []
    for r, (lo, hi) in enumerate(ranges):
        p = RankPlan(r, f"layers {lo}-{hi - 1}", workspace=workspace_bytes + act + (max_batch_rows * spec.vocab * 4 if r == n_stages - 1 else 0),
                     reserve=reserve_bytes)
        p.weights["layers"] = int(per_layer * (hi - lo))
        if r == 0:
            p.weights["embedding"] = int(embed)
        if r == n_stages - 1:
            p.weights["head"] = int(embed)
        free = gpu_bytes - p.weight_bytes - p.workspace - p.reserve
        if free < 0:
            p.shortfall = -free
        else:
            tokens_fit.append(int(free // (kv_layer * (hi - lo))))
        plans.append(p)
    fits = all(p.shortfall == 0 for p in plans)
    auto = min(tokens_fit) if len(tokens_fit) == n_stages else 0
    tokens = auto if pool_tokens <= 0 else pool_tokens
    notes = [f"layer-range split over {n_stages} GPUs: one step in flight, hidden rows of {spec.hidden * 2} bytes per token cross each boundary"]
    if pool_tokens > auto:
        fits = False
        notes.append(f"requested pool of {pool_tokens} tokens exceeds the {auto} that fit")
    tokens -= tokens % 64
    for p, (lo, hi) in zip(plans, ranges):
        p.kv_pool = int(max(tokens, 0) * kv_layer * (hi - lo))
        if p.shortfall:
            notes.append(f"stage {p.rank} ({p.role}) is short {p.shortfall / GIB:.1f} GiB")
    dep = Deployment(world=n_stages, attn_ranks=tuple(range(n_stages)), expert_ranks=tuple(range(n_stages)), colocated=True, attn_groups=1)
    return Layout(dep, plans, max(tokens, 0), min(spec.max_context, max(tokens, 0)), fits, notes)
