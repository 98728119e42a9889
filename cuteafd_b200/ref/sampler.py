"""Exact full-vocabulary sampler oracle.

Filter order (reference: rust/crates/cuteafd-core/src/target_sampling.rs:1-38):
  1. allowed-token mask (grammar),  2. temperature, 3. min_p (keep scaled logit >= max + ln(min_p)),
  4. top_k (exactly k survivors; lowest token id wins a boundary tie), 5. top_p (smallest descending
  prefix whose mass reaches top_p), then one categorical draw whose uniform is a pure function of
  (seed, position) - never of the batch row - so batching and speculative layouts cannot change a token.
Temperature below 1e-5 is greedy (lowest id wins ties).  An all-masked row is an error, never a fallback.

The GPU sampler (`csrc/sampling.cu`) implements the same chain and the same counter-based RNG and is
tested for token equality against this module.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

GREEDY_EPS = 1e-5
MAX_UNIFORM = 0.99999994
MASK32 = 0xFFFFFFFF


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0          # 0 = disabled
    min_p: float = 0.0
    seed: int = 0

    def validate(self):
        if not (0.0 <= self.temperature <= 2.0):
            raise ValueError("temperature must be in [0, 2]")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError("min_p must be in [0, 1]")
        return self

    @property
    def greedy(self) -> bool:
        return self.temperature < GREEDY_EPS


def _mix32(x: int) -> int:
    """32-bit finaliser (lowbias32-style); all arithmetic modulo 2**32 so CUDA matches bit for bit."""
    x &= MASK32
    x ^= x >> 16
    x = (x * 0x7FEB352D) & MASK32
    x ^= x >> 15
    x = (x * 0x846CA68B) & MASK32
    x ^= x >> 16
    return x


def uniform_from(seed: int, position: int) -> float:
    """Counter-based uniform in [0, MAX_UNIFORM]: hash of (seed lo, seed hi, position lo, position hi)."""
    s_lo, s_hi = seed & MASK32, (seed >> 32) & MASK32
    p_lo, p_hi = position & MASK32, (position >> 32) & MASK32
    h = _mix32(s_lo ^ 0x9E3779B9)
    h = _mix32(h ^ s_hi ^ 0x85EBCA6B)
    h = _mix32(h ^ p_lo ^ 0xC2B2AE35)
    h = _mix32(h ^ p_hi ^ 0x27D4EB2F)
    u = (h >> 8) * (1.0 / 16777216.0)      # 24 bits: exactly representable in fp32
    return min(u, MAX_UNIFORM)


def candidate_set(logits: torch.Tensor, params: SamplingParams, mask: torch.Tensor | None = None):
    """Applies the filter chain.  Returns (token ids sorted by descending scaled logit then ascending id,
    their fp32 probabilities renormalised over the survivors)."""
    x = logits.float().clone()
    V = x.numel()
    if not torch.isfinite(x).all():
        raise ValueError("non-finite logit")
    allowed = torch.ones(V, dtype=torch.bool) if mask is None else mask.bool()
    if mask is not None and mask.numel() != V:
        raise ValueError("mask width does not match vocabulary")
    if not allowed.any():
        raise ValueError("grammar allows no target token")
    x = x / max(params.temperature, GREEDY_EPS)
    x[~allowed] = float("-inf")
    if params.min_p > 0.0:
        x[x < x.max() + math.log(params.min_p)] = float("-inf")
    order = torch.sort(x, descending=True, stable=True).indices
    n_alive = int(torch.isfinite(x).sum())
    order = order[:n_alive]
    if params.top_k and params.top_k < n_alive:
        order = order[:params.top_k]
    xs = x[order]
    p = torch.exp(xs - xs[0])
    p = p / p.sum()
    if params.top_p < 1.0:
        cum = torch.cumsum(p, 0)
        keep = int((cum < params.top_p).sum()) + 1
        order, p = order[:keep], p[:keep]
        p = p / p.sum()
    return order, p


def sample(logits: torch.Tensor, params: SamplingParams, position: int, mask: torch.Tensor | None = None) -> int:
    if params.greedy:
        x = logits.float().clone()
        if mask is not None:
            if not mask.any():
                raise ValueError("grammar allows no target token")
            x[~mask.bool()] = float("-inf")
        return int(torch.argmax(x))          # torch.argmax returns the first (lowest-id) maximum
    order, p = candidate_set(logits, params, mask)
    u = uniform_from(params.seed, position)
    cum = torch.cumsum(p, 0)
    pick = int((cum <= u * float(cum[-1])).sum())
    return int(order[min(pick, order.numel() - 1)])


def logprob_of(logits: torch.Tensor, token: int) -> float:
    return float(torch.log_softmax(logits.float(), -1)[token])
