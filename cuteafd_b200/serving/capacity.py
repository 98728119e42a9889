"""Start-up capacity policy: how many KV pool tokens (and which context limit) a server gets on the memory it measured.

Pure arithmetic, no device work: the caller supplies the device's total and free bytes (measured before the server's own
allocations) and what the model costs; the policy answers with the pool size or says why the request does not fit.  Explicit
requests beyond what fits are rejected, never clipped silently: a pool that was asked for and cannot be had is an error, only the
default pool is sized down to what the device offers.

    ceiling  = min(total * occupancy%, total - minimum_free)          bytes this process may hold in all
    budget   = ceiling - already_used - weights - workspace           bytes left for the KV pool
    tokens   = min(target_pool_tokens, budget / kv_bytes_per_token)   rounded down to whole pages of 64 tokens

Reference: rust/crates/cuteafd-core/src/serving_capacity.rs (admission ceiling, default concurrency by card size, logical pool shared
by every device, explicit requests rejected instead of clipped).
"""
from __future__ import annotations

from dataclasses import dataclass

PAGE = 64
DEFAULT_POOL_TOKENS = 2 << 20          # the logical pool every family starts from; larger pools are explicit
SMALL_CARD_BYTES = 32 << 30


class CapacityError(ValueError):
    pass


def default_concurrency(gpu_bytes: int) -> int:
    """Sequences decoded together unless the operator says otherwise: 8 on cards of up to 32 GiB, 16 above."""
    return 8 if gpu_bytes <= SMALL_CARD_BYTES else 16


def admission_ceiling(total_bytes: int, occupancy_percent: int, minimum_free_bytes: int = 0) -> int:
    if not 1 <= occupancy_percent <= 100:
        raise CapacityError("GPU occupancy percent must be in 1..=100")
    return min(total_bytes * occupancy_percent // 100, max(0, total_bytes - minimum_free_bytes))


@dataclass(frozen=True)
class CapacityPolicy:
    concurrency: int = 0                    # 0: by card size
    target_pool_tokens: int = 0             # 0: DEFAULT_POOL_TOKENS, sized down to the device; > 0: explicit, must fit
    gpu_occupancy_percent: int = 92
    minimum_free_bytes: int = 2 << 30
    max_context: int = 0                    # 0: the model's own limit; explicit values beyond it are rejected


@dataclass(frozen=True)
class CapacityPlan:
    concurrency: int
    pool_tokens: int
    pool_pages: int
    pool_bytes: int
    max_context: int
    ceiling_bytes: int
    headroom_bytes: int                     # what stays free under the ceiling after weights, workspace and the pool

    def describe(self) -> str:
        gib = 2 ** 30
        return (f"{self.concurrency} sequences, KV pool {self.pool_tokens} tokens ({self.pool_bytes / gib:.1f} GiB, {self.pool_pages} pages), "
                f"context up to {self.max_context}, {self.headroom_bytes / gib:.1f} GiB under the {self.ceiling_bytes / gib:.1f} GiB ceiling left")


def plan_capacity(policy: CapacityPolicy, *, total_bytes: int, free_bytes: int, weight_bytes: int, kv_bytes_per_token: float,
                  model_max_context: int, workspace_bytes: int = 4 << 30, weights_loaded: bool = False) -> CapacityPlan:
    """`free_bytes`: free device memory measured now; with `weights_loaded` the weights are already part of what is used."""
    if kv_bytes_per_token <= 0 or total_bytes <= 0 or free_bytes < 0 or free_bytes > total_bytes:
        raise CapacityError("capacity inputs out of range")
    ceiling = admission_ceiling(total_bytes, policy.gpu_occupancy_percent, policy.minimum_free_bytes)
    used = total_bytes - free_bytes
    budget = ceiling - used - workspace_bytes - (0 if weights_loaded else weight_bytes)
    if budget < PAGE * kv_bytes_per_token:
        raise CapacityError(f"no room for a KV pool: ceiling {ceiling} bytes, in use {used}, weights {weight_bytes}, workspace {workspace_bytes}")
    fit_tokens = int(budget // kv_bytes_per_token) // PAGE * PAGE
    if policy.target_pool_tokens > 0:
        tokens = -(-policy.target_pool_tokens // PAGE) * PAGE
        if tokens > fit_tokens:
            raise CapacityError(f"a KV pool of {policy.target_pool_tokens} tokens needs {int(tokens * kv_bytes_per_token)} bytes; {int(budget)} fit under the ceiling")
    else:
        tokens = min(DEFAULT_POOL_TOKENS, fit_tokens)
    if policy.max_context > model_max_context:
        raise CapacityError(f"context {policy.max_context} exceeds the model's limit of {model_max_context}")
    context = policy.max_context or model_max_context
    if policy.max_context and policy.max_context > tokens:
        raise CapacityError(f"a context of {policy.max_context} tokens does not fit a pool of {tokens}")
    context = min(context, tokens)
    concurrency = policy.concurrency or default_concurrency(total_bytes)
    if concurrency < 1:
        raise CapacityError("concurrency must be positive")
    pool_bytes = int(tokens * kv_bytes_per_token)
    return CapacityPlan(concurrency, tokens, tokens // PAGE, pool_bytes, context, ceiling, int(budget) - pool_bytes)
