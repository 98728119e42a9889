"""`cuteafd plan MODEL`: read a snapshot's config + safetensors headers, detect the family and every weight's
storage format, check them against what the kernels can execute, and (optionally) print the per-rank layout.
Unsupported combinations are reported as results with hints, never raised.
Reference: cuteafd-daemon/src/commands/plan.rs:118-298, cuteafd-loader/src/plan/mod.rs, AGENTS.md:274-275.
"""
from __future__ import annotations

import re

import json
from collections import Counter
from dataclasses import dataclass, field
from pathlib import Path

from ..config import ModelSpec, spec_from_snapshot, spec_by_name, NAMED_SPECS
from . import formats, placement
from .safetensors_io import catalog

# what each kernel family can run today: (operand format) -> kernel
EXECUTABLE = {
    "bf16": "tc_linear kind::f16", "nvfp4": "tc_linear kind::mxf4nvf4 (W4A4)", "mxfp4": "tc_linear kind::mxf4 (W4A4)",
    "fp8_block128": "fp8_linear kind::f8f6f4 with per-stage block scales",
    "f32": "cast to bf16 at load", "f16": "cast to bf16 at load",
}
HINTS = {
    "fp8_block32": "FP8 with 32 x 32 UE8M0 block scales has no kernel yet (tcgen05 kind::mxf8f6f4 scales along K only); re-quantise to 128 x 128 blocks with `cuteafd quantize`",
    "exl3": "EXL3 trellis weights are decoded by the dequant-GEMM path (K2-K5); check `cuteafd doctor` for the kernel",
}


@dataclass
class PlanReport:
    model: str
    family: str | None
    spec: ModelSpec | None
    supported: bool
    format_counts: dict = field(default_factory=dict)
    problems: list = field(default_factory=list)
    hints: list = field(default_factory=list)
    layout: placement.Layout | None = None
    files: list = field(default_factory=list)

    def to_json(self) -> dict:
        return {"model": self.model, "family": self.family, "supported": self.supported, "formats": self.format_counts,
                "problems": self.problems, "hints": self.hints,
                "layout": None if self.layout is None else {
                    "fits": self.layout.fits, "pool_tokens": self.layout.pool_tokens, "notes": self.layout.notes,
                    "ranks": [{"rank": r.rank, "role": r.role, "weights_gib": round(r.weight_bytes / placement.GIB, 2),
                               "kv_gib": round(r.kv_pool / placement.GIB, 2)} for r in self.layout.ranks]},
                "files": self.files}

    def text(self) -> str:
        out = [f"model    : {self.model}", f"family   : {self.family}", f"supported: {self.supported}"]
        out += [f"format   : {k} x{v}" for k, v in sorted(self.format_counts.items())]
        out += [f"problem  : {p}" for p in self.problems] + [f"hint     : {h}" for h in self.hints]
        if self.layout is not None:
            out.append(self.layout.table())
        return "\n".join(out)


def deployment_decisions(layout: "placement.Layout", model: str, port: int = 29500) -> dict:
    """Typed launch decisions for a solved layout: who does what, and the command that starts every rank of the node
    (reference: `cuteafd plan --deployment`, which turns a layout into per-role / per-host daemon arguments)."""
    dep = layout.deployment
    groups = [{"group": g, "ranks": list(dep.group_ranks(g))} for g in range(dep.attn_groups)]
    roles = []
    for r in layout.ranks:
        entry = {"rank": r.rank, "role": r.role, "device": r.rank}
        if r.rank in dep.attn_ranks:
            entry["attention_group"] = dep.group_of(r.rank)
            entry["tp_rank"] = list(dep.group_ranks(dep.group_of(r.rank))).index(r.rank)
        if r.rank in dep.expert_ranks:
            entry["ep_rank"] = list(dep.expert_ranks).index(r.rank)
        roles.append(entry)
    return {"parallelism": dep.describe(), "world": dep.world, "attention_groups": groups, "expert_ranks": list(dep.expert_ranks),
            "pool_tokens_per_group": layout.pool_tokens, "ranks": roles,
            "launch": {"serve": f"python -m cuteafd_b200.cli serve --model {model}" if dep.world == 1 else
                                (f"python -m torch.distributed.run --nnodes=1 --nproc-per-node {dep.world} --master-addr 127.0.0.1 --master-port {port} "
                                 f"-m cuteafd_b200.cli serve --model {model}") if dep.attn_groups == 1 and not dep.colocated else None,
                       "decode_bench": (f"python -m torch.distributed.run --nnodes=1 --nproc-per-node {dep.world} --master-addr 127.0.0.1 "
                                        f"--master-port {port} bench.py --gpus {dep.world} --attn-groups {dep.attn_groups}") if dep.world > 1
                                       else "python bench.py --gpus 1"},
            "env": {"NCCL_NVLS_ENABLE": "0"} if dep.world > 1 else {}}


_EXPERT_RE = re.compile(r"\.experts\.(\d+)\.")


def files_for_rank(snapshot: str | Path, deployment, rank: int, n_experts: int | None = None) -> dict:
    """Which safetensors files (and how many bytes of them) one rank of a deployment reads: attention ranks take every
    tensor that is not a routed expert, expert ranks the experts of their range.  This is what a role-sliced copy of a
    checkpoint contains (reference: `cuteafd plan --files --role`, docs/sliced-checkpoints.md)."""
    cat = catalog(Path(snapshot))
    if n_experts is None:                                  # no config at hand: the highest expert index named by a tensor
        n_experts = 1 + max((int(m.group(1)) for m in map(_EXPERT_RE.search, cat) if m), default=-1)
    lo = hi = -1
    if rank in deployment.expert_ranks:
        ep, i = max(1, deployment.ep), list(deployment.expert_ranks).index(rank)
        lo, hi = (i * n_experts) // ep, ((i + 1) * n_experts) // ep      # the ranges the expert ranks use at run time
    files: dict = {}
    for name, t in cat.items():
        m = _EXPERT_RE.search(name)
        if m:
            take = lo <= int(m.group(1)) < hi
        else:
            take = rank in deployment.attn_ranks
        if take:
            f = files.setdefault(Path(t.file).name, {"tensors": 0, "bytes": 0})
            f["tensors"] += 1
            f["bytes"] += t.nbytes
    role = "both" if rank in deployment.attn_ranks and rank in deployment.expert_ranks else ("attention" if rank in deployment.attn_ranks else "experts")
    return {"rank": rank, "role": role, "experts": [lo, hi] if lo >= 0 else None, "files": files,
            "bytes": sum(f["bytes"] for f in files.values())}


def plan(model: str, *, world: int = 8, layout: bool = False, files: bool = False, pool_tokens: int = 0, gpu_gib: int = 180,
         attn_groups: int = 1, stages: int = 0) -> PlanReport:
    """`model` is a snapshot directory (config.json + *.safetensors) or one of the named synthetic shapes."""
    problems, hints, counts, flist = [], [], Counter(), []
    p = Path(model)
    spec = family = None
    if p.is_dir():
        try:
            spec = spec_from_snapshot(p)
            family = spec.family
        except Exception as e:
            problems.append(f"config.json: {e}")
        try:
            cat = catalog(p)
            ops, bad = formats.detect_all(cat)
            for b in bad:
                problems.append(f"{b.stem}: {b.reason}")
            for op in ops.values():
                if len(op.logical) >= 2:
                    counts[op.format] += 1
            if files:
                flist = sorted({Path(t.file).name for t in cat.values()})
        except Exception as e:
            problems.append(f"safetensors: {e}")
    elif model in NAMED_SPECS:
        spec = spec_by_name(model)
        family = spec.family
        counts[spec.quant.experts] += 1
        counts[spec.quant.dense] += 1
    else:
        problems.append(f"{model!r} is neither a snapshot directory nor a known shape ({', '.join(sorted(NAMED_SPECS))})")
    for fmt in counts:
        base = fmt.split("_k")[0] if fmt.startswith("exl3") else fmt
        if base not in EXECUTABLE:
            (hints if base in HINTS else problems).append(HINTS.get(base, f"no kernel executes weights stored as {fmt}"))
    if spec is not None and spec.attn.kind == "gqa" and spec.attn.head_dim not in (32, 64, 128):
        problems.append(f"attention head_dim {spec.attn.head_dim} has no kernel (32, 64 or 128)")
    rep = PlanReport(model, family, spec, supported=spec is not None and not problems, format_counts=dict(counts), problems=problems,
                     hints=hints, files=flist)
    if layout and spec is not None:
        from ..config import default_deployment
        rep.layout = placement.solve(spec, world=world, gpu_bytes=gpu_gib * placement.GIB, pool_tokens=pool_tokens,
                                     deployment=default_deployment(world, attn_groups))
        if attn_groups > 1:
            rep.layout.notes.append(f"{attn_groups} data-parallel attention groups: the pool is per group "
                                    f"({attn_groups * rep.layout.pool_tokens} tokens in total)")
        if not rep.layout.fits:
            rep.supported = False
    if stages and spec is not None:         # a layer-range split instead of the attention / expert layout
        try:
            rep.layout = placement.solve_stages(spec, stages, gpu_bytes=gpu_gib * placement.GIB, pool_tokens=pool_tokens)
            if not rep.layout.fits:
                rep.supported = False
        except (ValueError, NotImplementedError) as e:
            rep.problems.append(f"layer-range split: {e}")
            rep.supported = False
    return rep
