"""Owner scheduling for replicated expert groups (TP x EP): when several groups of expert ranks each hold a copy of every routed
expert, every ACTIVE expert of a layer step is executed by exactly one group, chosen so that the groups finish together.

Policy: whole experts, largest predicted cost first, each to the group with the smallest load so far (LPT greedy).  An expert's cost is
    weight_cost + ceil(routed_rows / tile_rows) * tile_cost
- its weights are streamed once whoever runs it (the dominant term at decode sizes), plus the padded row tiles.  Whole-expert
assignment keeps that reuse; a single dominant expert is therefore never split, and bounds the step from below.  The plan is a pure
function of (config, route counts, tie seed): no clock, no global state, so every rank that plans from the same routes gets the same
owners without exchanging them.  Ties between equal costs are broken by a hash of (tie seed, expert), so successive layers do not
all favour the low expert ids.

`apply_owner_plan` turns a plan into what an expert group sees: routes to experts another group owns keep their slot but carry the
UNASSIGNED id and weight 0 (the combine adds nothing for them), which is the encoding of the wire protocol (`parallel/protocol.py`).

Reference: rust/crates/cuteafd-core/src/replicated_expert_schedule.rs:1-145 (policy, cost model, determinism),
rust/crates/cuteafd-transport/src/expert.rs:47-56, 162-198 (owner bits in route words, unassigned id with zero weight).
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass

import numpy as np

INACTIVE = 255
MAX_GROUPS = 8


@dataclass(frozen=True)
class OwnerCostModel:
    weight_cost: int = 1000          # streaming one expert's weights, in abstract cost units
    tile_cost: int = 10              # one padded tile of routed rows
    tile_rows: int = 16

    def cost(self, routed_rows: int) -> int:
        return self.weight_cost + -(-routed_rows // self.tile_rows) * self.tile_cost if routed_rows > 0 else 0


@dataclass
class OwnerPlan:
    owner: np.ndarray                # uint8 [n_experts]: group that runs the expert, INACTIVE for experts without rows
    load: list                       # predicted cost per group
    active: int

    @property
    def makespan(self) -> int:
        return max(self.load) if self.load else 0

    @property
    def imbalance(self) -> float:
        """Largest group load over the mean load (1.0 = perfectly even)."""
        mean = sum(self.load) / len(self.load) if self.load else 0
        return self.makespan / mean if mean else 1.0


def _tie_key(seed: int, expert: int) -> int:
    return int.from_bytes(hashlib.blake2b(f"{seed}:{expert}".encode(), digest_size=8).digest(), "little")


class ReplicatedExpertScheduler:
    def __init__(self, n_groups: int, model: OwnerCostModel | None = None):
        if not 1 <= n_groups <= MAX_GROUPS:
            raise ValueError(f"1..{MAX_GROUPS} replicated expert groups")
        self.n_groups, self.model = n_groups, model or OwnerCostModel()

    def plan(self, route_counts, tie_seed: int = 0) -> OwnerPlan:
        """route_counts[e]: rows routed to expert e in this layer step (all attention ranks together)."""
        counts = np.asarray(route_counts, dtype=np.int64)
        if counts.ndim != 1 or (counts < 0).any():
            raise ValueError("route counts are a non-negative vector over the experts")
        owner = np.full(counts.shape[0], INACTIVE, dtype=np.uint8)
        active = [int(e) for e in np.nonzero(counts)[0]]
        order = sorted(active, key=lambda e: (-self.model.cost(int(counts[e])), _tie_key(tie_seed, e)))
        load = [0] * self.n_groups
        for e in order:
            g = min(range(self.n_groups), key=lambda i: (load[i], i))
            owner[e] = g
            load[g] += self.model.cost(int(counts[e]))
        return OwnerPlan(owner, load, len(active))

    def plan_routes(self, expert_ids, n_experts: int, tie_seed: int = 0) -> OwnerPlan:
        """From the routed expert ids of a step ([tokens, top_k], negative = no route)."""
        ids = np.asarray(expert_ids).reshape(-1)
        return self.plan(np.bincount(ids[ids >= 0], minlength=n_experts), tie_seed)


def apply_owner_plan(routes: np.ndarray, plan: OwnerPlan, group: int) -> np.ndarray:
    """The routes as group `group` executes them: entries of experts owned elsewhere become UNASSIGNED with gate 0."""
    from .protocol import UNASSIGNED
    out = routes.copy()
    exp = out["expert"].astype(np.int64)
    valid = (exp >= 0) & (exp < plan.owner.shape[0])
    mine = np.zeros(exp.shape, dtype=bool)
    mine[valid] = plan.owner[exp[valid]] == group
    out["expert"][~mine] = UNASSIGNED
    out["gate"][~mine] = 0.0
    return out


def static_range_plan(route_counts, n_groups: int, model: OwnerCostModel | None = None) -> OwnerPlan:
    """The baseline the scheduler is compared with: group g owns the contiguous expert range g (what plain expert parallelism does)."""
    model = model or OwnerCostModel()
    counts = np.asarray(route_counts, dtype=np.int64)
    n = counts.shape[0]
    owner = np.full(n, INACTIVE, dtype=np.uint8)
    load = [0] * n_groups
    for e in np.nonzero(counts)[0]:
        g = min(n_groups - 1, int(e) * n_groups // n)
        owner[e] = g
        load[g] += model.cost(int(counts[e]))
    return OwnerPlan(owner, load, int((counts > 0).sum()))
