"""Cutting one model's fp32 masters into the shares of the ranks of a deployment.

An attention rank of a tensor-parallel group of size `tp` keeps every `tp`-th block of query heads (and, for GQA, of KV
heads), the matching columns of the output projection, the router, the shared expert / dense FFN, norms, embeddings and
the head; it holds no routed experts.  An expert rank keeps a contiguous range of routed experts and nothing else.
Shards are cut BEFORE quantisation, so a quantised shard is exactly what a loader would produce from a role-sliced
checkpoint, and a layout with bf16 projections reproduces the single-GPU model bit for bit.

Reference: role-sliced checkpoints (docs/sliced-checkpoints.md:1-47), output-channel / head shards of the two-GPU split
(families/deepseek_v41/v41_projection_tp2.rs, families/deepseek_v4/engine.rs:97-119).
"""
from __future__ import annotations

import dataclasses

import torch

from ..config import ModelSpec

EXPERT_KEYS = ("w_gate", "w_up", "w_down")


def local_attention_spec(spec: ModelSpec, tp: int) -> ModelSpec:
    a = spec.attn
    if a.n_heads % tp or (a.kind == "gqa" and a.n_kv_heads % tp):
        raise ValueError(f"heads ({a.n_heads}/{a.n_kv_heads}) do not split over tp={tp}")
    kv = a.n_kv_heads // tp if a.kind == "gqa" else a.n_heads // tp
    return spec.replace(attn=dataclasses.replace(a, n_heads=a.n_heads // tp, n_kv_heads=kv))


def _attn_layer_shard(spec: ModelSpec, lw: dict, tp: int, r: int) -> dict:
    a = spec.attn
    out = {k: v for k, v in lw.items() if k not in EXPERT_KEYS}
    if tp == 1:
        return out
    if a.kind == "gqa":
        hq, hkv, D = a.n_heads // tp, a.n_kv_heads // tp, a.head_dim
        out["wq"] = lw["wq"][r * hq * D:(r + 1) * hq * D].contiguous()
        out["wk"] = lw["wk"][r * hkv * D:(r + 1) * hkv * D].contiguous()
        out["wv"] = lw["wv"][r * hkv * D:(r + 1) * hkv * D].contiguous()
        out["wo"] = lw["wo"][:, r * hq * D:(r + 1) * hq * D].contiguous()
        if "sink" in lw:
            out["sink"] = lw["sink"][r * hq:(r + 1) * hq].contiguous()
        return out
    Hl = a.n_heads // tp
    qk, dv, nope = a.qk_nope_head_dim + a.qk_rope_head_dim, a.v_head_dim, a.qk_nope_head_dim
    qkey = "wq_b" if "wq_b" in lw else "wq"
    out[qkey] = lw[qkey][r * Hl * qk:(r + 1) * Hl * qk].contiguous()
    out["wkv_b"] = lw["wkv_b"].reshape(a.n_heads, nope + dv, a.kv_lora_rank)[r * Hl:(r + 1) * Hl].reshape(Hl * (nope + dv), a.kv_lora_rank).contiguous()
    out["wo"] = lw["wo"][:, r * Hl * dv:(r + 1) * Hl * dv].contiguous()
    return out


def attention_masters(spec: ModelSpec, masters: dict, tp: int = 1, tp_rank: int = 0) -> dict:
    """Masters of one attention rank (no routed experts; heads cut for `tp` > 1).  Goes with `local_attention_spec`."""
    out = {k: v for k, v in masters.items() if k not in ("layers", "mtp")}
    out["layers"] = [_attn_layer_shard(spec, lw, tp, tp_rank) for lw in masters["layers"]]
    if masters.get("mtp"):
        out["mtp"] = [dict(mw, layer=_attn_layer_shard(spec, mw["layer"], tp, tp_rank)) for mw in masters["mtp"]]
    return out


def expert_masters(spec: ModelSpec, masters: dict, e_lo: int, e_hi: int) -> list:
    """Per layer (main layers, then MTP draft layers): {"w_gate", "w_up", "w_down"} of experts [e_lo, e_hi), or None for a
    layer without routed experts."""
    layers = list(masters["layers"]) + [mw["layer"] for mw in masters.get("mtp", [])]
    out = []
    for lw in layers:
        out.append({k: lw[k][e_lo:e_hi].contiguous() for k in EXPERT_KEYS} if "w_gate" in lw else None)
    return out


def expert_tp_slice(intermediate: int, n_ranks: int, granule: int = 32) -> int:
    """Rows of the intermediate dimension each rank of an expert-TP group holds: equal slices rounded up to `granule`; the
    padding beyond the true intermediate size is zero weights (reference: zero-pad of the intermediate dimension to the tile
    size, native/shared/cuda/expert_pack.cu:9)."""
    per = -(-intermediate // n_ranks)
    return -(-per // granule) * granule


def expert_tp_masters(spec: ModelSpec, masters: dict, rank: int, n_ranks: int, granule: int = 32) -> list:
    """Per layer (main layers, then MTP draft layers): rank `rank`'s intermediate-dimension slice of EVERY routed expert -
    rows [rank * s, (rank + 1) * s) of gate / up and the matching columns of down, zero-padded past the true size - or None.
    Every rank then returns, per route, a partial sum over its slice; the attention rank adds the ranks in fixed order
    (reference: expert TP, native/shared/include/cuteafd_experts.h:13-23; cuteafd-transport/src/expert.rs:162-198)."""
    I = spec.moe.intermediate
    sl = expert_tp_slice(I, n_ranks, granule)
    lo, hi = rank * sl, (rank + 1) * sl
    layers = list(masters["layers"]) + [mw["layer"] for mw in masters.get("mtp", [])]
    out = []
    for lw in layers:
        if "w_gate" not in lw:
            out.append(None)
            continue
        E, _, H = lw["w_gate"].shape

        def rows(w):
            part = torch.zeros(E, sl, H, dtype=w.dtype)
            a, b = min(lo, I), min(hi, I)
            part[:, :b - a] = w[:, a:b]
            return part
        down = torch.zeros(E, H, sl, dtype=lw["w_down"].dtype)
        a, b = min(lo, I), min(hi, I)
        down[:, :, :b - a] = lw["w_down"][:, :, a:b]
        out.append({"w_gate": rows(lw["w_gate"]), "w_up": rows(lw["w_up"]), "w_down": down})
    return out
