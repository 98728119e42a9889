"""Sealed golden windows: a published record of what the fp32 oracle predicts on fixed token windows, and the check of an
engine against it (the logit-fidelity gate of the baseline card).

A golden file is JSON: the model's name and geometry digest, and per window the token ids, the oracle's top-1 token after every
position of the window's tail, and the oracle's top-k (ids and logits) after the last position.  It is written once from masters
the oracle can evaluate (`write_golden`: a snapshot or the tiny model) and travels with the checkpoint; any engine, layout or
quantisation of the same model is then checked without the oracle (`check_logits`):

  * top-1 agreement over the tail positions of every window (a quantised engine may differ where the oracle's own margin is thin:
    disagreements are only counted where the golden top-2 margin exceeds `margin`);
  * relative L2 error of the engine's logits on the golden top-k entries of the last position;
  * the window passes when agreement >= `min_agree` and the error <= `max_rel_l2`.

Reference: logit fidelity against eight sealed published windows, cuteafd-bench/src/baseline.rs:1-6, 226-227; layer-by-layer
golden comparison of the family engines, families/deepseek_v4/mod.rs:626-890 (here the comparison is on logits only).
"""
from __future__ import annotations

import hashlib
import json

import torch

from ..config import ModelSpec


def spec_digest(spec: ModelSpec) -> str:
    a, m = spec.attn, spec.moe
    key = (spec.name, spec.vocab, spec.hidden, spec.n_layers, a.kind, a.n_heads, a.n_kv_heads, a.head_dim, a.kv_lora_rank, m.n_experts, m.top_k,
           m.intermediate)
    return hashlib.sha256(repr(key).encode()).hexdigest()[:16]


def make_windows(vocab: int, n: int = 8, length: int = 64, seed: int = 2026) -> list[list[int]]:
    """`n` token windows of `length` ids: seeded, so the same call reproduces the published windows."""
    g = torch.Generator().manual_seed(seed)
    lo = min(16, vocab - 1)
    return [torch.randint(lo, vocab, (length,), generator=g).tolist() for _ in range(n)]


def oracle_windows(spec: ModelSpec, masters: dict, windows: list[list[int]], tail: int = 16, topk: int = 8) -> dict:
    """Evaluates the fp32 oracle teacher-forced on every window."""
    from ..ref.model import RefCache, RefModel
    ref = RefModel(spec, masters)
    out = []
    for w in windows:
        logits, _ = ref.forward(torch.tensor(w), 0, RefCache())            # [T, V]
        lf = logits.float()
        t = min(tail, len(w))
        top2 = lf[-t:].topk(2, -1)
        last = lf[-1].topk(topk)
        out.append({"tokens": list(w), "tail_top1": top2.indices[:, 0].tolist(), "tail_margin": (top2.values[:, 0] - top2.values[:, 1]).tolist(),
                    "last_topk_ids": last.indices.tolist(), "last_topk_logits": [round(float(v), 6) for v in last.values]})
    return {"format": 1, "model": spec.name, "digest": spec_digest(spec), "tail": tail, "topk": topk, "windows": out}


def write_golden(path: str, spec: ModelSpec, masters: dict, *, n: int = 8, length: int = 64, seed: int = 2026, tail: int = 16, topk: int = 8) -> dict:
    gold = oracle_windows(spec, masters, make_windows(spec.vocab, n, length, seed), tail, topk)
    with open(path, "w") as f:
        json.dump(gold, f)
    return gold


def read_golden(path: str) -> dict:
    with open(path) as f:
        gold = json.load(f)
    if gold.get("format") != 1 or "windows" not in gold:
        raise ValueError(f"{path}: not a golden-window file")
    return gold


def check_logits(logits_fn, gold: dict, *, spec: ModelSpec | None = None, min_agree: float = 0.9, max_rel_l2: float = 0.1, margin: float = 0.05) -> dict:
    """`logits_fn(tokens) -> [T, V]` (teacher-forced logits of every position, any device).  Returns the report; `report["pass"]`."""
    if spec is not None and gold.get("digest") != spec_digest(spec):
        raise ValueError(f"golden windows were written for {gold.get('model')!r} ({gold.get('digest')}), not for this model ({spec_digest(spec)})")
    rows = []
    for i, w in enumerate(gold["windows"]):
        lf = logits_fn(w["tokens"]).float().cpu()
        t = len(w["tail_top1"])
        got = lf[-t:].argmax(-1).tolist()
        decided = [j for j in range(t) if w["tail_margin"][j] > margin]
        agree = sum(got[j] == w["tail_top1"][j] for j in decided) / max(1, len(decided))
        ids = torch.tensor(w["last_topk_ids"])
        want = torch.tensor(w["last_topk_logits"])
        rel = float((lf[-1][ids] - want).norm() / want.norm().clamp_min(1e-12))
        rows.append({"window": i, "top1_agreement": round(agree, 4), "decided_positions": len(decided), "rel_l2_topk": round(rel, 5),
                     "pass": agree >= min_agree and rel <= max_rel_l2})
    return {"model": gold.get("model"), "windows": rows, "pass": all(r["pass"] for r in rows),
            "thresholds": {"min_agree": min_agree, "max_rel_l2": max_rel_l2, "margin": margin}}


def engine_logits_fn(eng):
    """Teacher-forced logits of one window through an engine's public step API (one prefill step, every row asks for logits)."""
    from ..engine.engine import StepShape
    from ..engine.kv import PagePool, SeqKV
    pool = PagePool(eng.n_pages)

    def fn(tokens: list[int]) -> torch.Tensor:
        T = len(tokens)
        s = SeqKV()
        s.ensure(pool, T + 1)
        if getattr(eng, "lin_layers", None):
            eng.reset_state_slots([0])
        eng.set_inputs(tokens, list(range(T)), [s.slot(p) for p in range(T)], list(range(T)), [T], [0], [T], [s.pages])
        lane = eng.run(StepShape(T=T, n_seq=1, max_q_len=T, n_logits=T, attn_splits=1), use_graph=False)
        out = lane.logits[:T].float().cpu()
        eng.check_status()
        s.release(pool)
        return out
    return fn
