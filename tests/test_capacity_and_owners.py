"""Start-up capacity policy and the owner scheduler of replicated expert groups (pure CPU planners)."""
import numpy as np
import pytest

from cuteafd_b200.parallel.owner_schedule import (INACTIVE, OwnerCostModel, ReplicatedExpertScheduler, apply_owner_plan, static_range_plan)
from cuteafd_b200.serving.capacity import (DEFAULT_POOL_TOKENS, CapacityError, CapacityPolicy, admission_ceiling, default_concurrency,
                                           plan_capacity)

GIB = 2 ** 30


def test_admission_ceiling_and_default_concurrency():
    assert admission_ceiling(180 * GIB, 92, 2 * GIB) == 180 * GIB * 92 // 100
    assert admission_ceiling(32 * GIB, 100, 3 * GIB) == 29 * GIB            # the absolute floor binds on a small card
    with pytest.raises(CapacityError):
        admission_ceiling(GIB, 0)
    assert default_concurrency(32 * GIB) == 8 and default_concurrency(180 * GIB) == 16


def test_default_pool_is_sized_to_the_device_and_explicit_requests_must_fit():
    kv = 94 * 4 * 128 * 2 * 2.0                          # Qwen3-235B shape: 94 layers, 4 KV heads of 128, K and V, bf16
    base = dict(total_bytes=180 * GIB, free_bytes=178 * GIB, weight_bytes=134 * GIB, kv_bytes_per_token=kv, model_max_context=131072)
    plan = plan_capacity(CapacityPolicy(), **base)
    budget = 180 * GIB * 92 // 100 - 2 * GIB - 4 * GIB - 134 * GIB
    assert plan.pool_tokens == int(budget // kv) // 64 * 64 < DEFAULT_POOL_TOKENS
    assert plan.pool_pages * 64 == plan.pool_tokens and plan.concurrency == 16 and 0 <= plan.headroom_bytes < 64 * kv
    assert plan.max_context == min(131072, plan.pool_tokens) and "KV pool" in plan.describe()
    small = plan_capacity(CapacityPolicy(), **{**base, "weight_bytes": GIB, "kv_bytes_per_token": 1024.0})
    assert small.pool_tokens == DEFAULT_POOL_TOKENS        # room to spare: the default logical pool, not everything that fits
    with pytest.raises(CapacityError, match="fit under the ceiling"):
        plan_capacity(CapacityPolicy(target_pool_tokens=1 << 20), **base)          # asked for, does not fit: an error, not a smaller pool
    ok = plan_capacity(CapacityPolicy(target_pool_tokens=60000, concurrency=4, max_context=32768), **base)
    assert ok.pool_tokens == 60032 and ok.concurrency == 4 and ok.max_context == 32768
    with pytest.raises(CapacityError, match="model's limit"):
        plan_capacity(CapacityPolicy(max_context=1 << 20), **base)
    with pytest.raises(CapacityError, match="does not fit a pool"):
        plan_capacity(CapacityPolicy(target_pool_tokens=8192, max_context=16384), **base)
    with pytest.raises(CapacityError, match="no room"):
        plan_capacity(CapacityPolicy(), **{**base, "free_bytes": 120 * GIB})
    loaded = plan_capacity(CapacityPolicy(), **{**base, "free_bytes": 44 * GIB, "weights_loaded": True})
    assert loaded.pool_tokens == plan.pool_tokens          # the same device seen after the weights were loaded


def test_owner_plan_is_deterministic_balanced_and_keeps_whole_experts():
    rng = np.random.default_rng(0)
    counts = np.zeros(128, dtype=np.int64)
    hot = rng.choice(128, 40, replace=False)
    counts[hot] = rng.integers(1, 30, 40)
    sched = ReplicatedExpertScheduler(3, OwnerCostModel(weight_cost=1000, tile_cost=10, tile_rows=16))
    plan = sched.plan(counts, tie_seed=7)
    assert plan.active == 40 and (plan.owner[counts == 0] == INACTIVE).all() and (plan.owner[counts > 0] < 3).all()
    assert sum(plan.load) == sum(sched.model.cost(int(c)) for c in counts if c) and plan.imbalance < 1.05
    again = sched.plan(counts, tie_seed=7)
    assert (again.owner == plan.owner).all()
    other = sched.plan(counts, tie_seed=8)
    assert (other.owner != plan.owner).any() and abs(other.makespan - plan.makespan) <= 1020       # ties fall differently, the balance holds
    # contiguous expert ranges (plain expert parallelism) are at the mercy of where the hot experts sit
    skew = np.zeros(128, dtype=np.int64)
    skew[:30] = 4
    assert static_range_plan(skew, 3).imbalance > 2.5 and sched.plan(skew).imbalance < 1.05
    # one dominant expert is not split: it bounds the step
    one = np.zeros(16, dtype=np.int64)
    one[5], one[9] = 4000, 3
    p = ReplicatedExpertScheduler(2).plan(one)
    assert p.owner[5] != p.owner[9] and p.makespan == OwnerCostModel().cost(4000)
    with pytest.raises(ValueError):
        ReplicatedExpertScheduler(0)


def test_owner_plan_applied_to_wire_routes():
    from cuteafd_b200.parallel.protocol import UNASSIGNED
    routes = np.zeros((3, 2), dtype=[("expert", "<u4"), ("gate", "<f4")])
    routes["expert"] = [[1, 5], [5, 9], [1, 9]]
    routes["gate"] = 0.5
    sched = ReplicatedExpertScheduler(2)
    plan = sched.plan_routes(routes["expert"].astype(np.int64), 16, tie_seed=3)
    seen = np.zeros((3, 2), dtype=int)
    for g in range(2):
        mine = apply_owner_plan(routes, plan, g)
        kept = mine["expert"] != UNASSIGNED
        assert (mine["gate"][~kept] == 0).all() and (mine["gate"][kept] == 0.5).all()
        assert (plan.owner[mine["expert"][kept].astype(np.int64)] == g).all()
        seen += kept
    assert (seen == 1).all()                                # every route is executed by exactly one group
    assert (routes["gate"] == 0.5).all()                    # the caller's routes are not modified


def test_layer_range_placement_and_plan_flag():
    from cuteafd_b200.config import spec_by_name
    from cuteafd_b200.loader import placement
    from cuteafd_b200.loader.plan import plan
    spec = spec_by_name("qwen3-235b")
    lay = placement.solve_stages(spec, 2)
    assert lay.fits and [r.role for r in lay.ranks] == ["layers 0-46", "layers 47-93"]
    assert "embedding" in lay.ranks[0].weights and "head" in lay.ranks[1].weights and "head" not in lay.ranks[0].weights
    assert all(r.total <= 180 * placement.GIB for r in lay.ranks) and lay.pool_tokens % 64 == 0 and lay.pool_tokens > 0
    one = placement.solve_stages(spec, 1, gpu_bytes=80 * placement.GIB)
    assert not one.fits and any("short" in n for n in one.notes)                     # 134 GB of weights on an 80 GB device
    assert placement.solve_stages(spec, 2, gpu_bytes=80 * placement.GIB).fits         # the split is what makes it fit
    rep = plan("qwen3-235b", stages=2)
    assert rep.supported and rep.layout.deployment.world == 2 and "layers 0-46" in rep.layout.table()
    bad = plan("qwen3-235b", stages=200)
    assert not bad.supported and any("layer-range split" in p for p in bad.problems)
