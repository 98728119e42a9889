"""Re-quantisation of a snapshot, one unit (embeddings + head, then every layer) at a time, with a run store.

    cuteafd quantize SRC DST --dense nvfp4 --experts mxfp4

Each unit is decoded from the source snapshot (whatever format it is stored in), re-encoded in the target formats and
written as its own safetensors shard through a temporary name + rename, then recorded in `DST/quantize_run.json`.  A run
that dies is continued by running the same command again: finished units whose shard is still there with the recorded
size are skipped, everything else is redone.  The run store carries a *recovery identity* (hash of the source file
list with sizes, the model shape and the target formats); a store written for anything else is refused unless
`restart=True`.  Publication (the tensor index + config / tokenizer files) happens last and is itself repeatable, so a
crash between the last unit and the index is recovered by the next run.

Reference: quantization/{run_store,recovery_identity,recover_publication}.py (run store, recovery identity, publication
recovery of the distributed EXL3 quantisation pipeline).  Here the work is a single process over layers, and the
encoders are the format writers of `loader.checkpoint` (bf16, FP8 128x128, NVFP4, MXFP4).
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
from pathlib import Path

import torch

from ..config import ModelSpec
from .checkpoint import VECTORS, _dequant, _emit, _is_expert, _ops_of, _vector, layer_stems
from .safetensors_io import read_header, read_tensor, write_file

RUN_FILE = "quantize_run.json"
SIDE_FILES = ("config.json", "generation_config.json", "tokenizer.json", "tokenizer_config.json")


class Interrupted(RuntimeError):
    """Raised by the `stop_after` hook of tests to stand in for a crash between two units."""


def recovery_identity(src: Path, spec: ModelSpec, dense: str, experts: str) -> str:
    h = hashlib.sha256()
    for f in sorted(src.glob("*.safetensors")):
        h.update(f"{f.name}:{f.stat().st_size};".encode())
    h.update(f"{spec.name}|{spec.n_layers}|{spec.hidden}|{spec.moe.n_experts}|{dense}|{experts}".encode())
    return h.hexdigest()[:32]


def _atomic_json(path: Path, obj: dict):
    tmp = path.with_suffix(path.suffix + ".tmp")
    tmp.write_text(json.dumps(obj, indent=1))
    os.replace(tmp, path)


def _unit_names(spec: ModelSpec) -> list[str]:
    return ["head"] + [f"layer-{i:04d}" for i in range(spec.n_layers + spec.mtp_layers)]


def _encode_unit(ops: dict, spec: ModelSpec, unit: str, dense: str, experts: str) -> tuple[dict, dict]:
    out: dict = {}
    dt: dict = {}
    if unit == "head":
        out["model.embed_tokens.weight"] = read_tensor(ops["model.embed_tokens"].members["weight"]).to(torch.bfloat16)
        out["model.norm.weight"] = read_tensor(ops["model.norm"].members["weight"]).to(torch.bfloat16)
        if not spec.tie_embeddings:
            out["lm_head.weight"] = read_tensor(ops["lm_head"].members["weight"]).to(torch.bfloat16)
        return out, dt
    i = int(unit.split("-")[1])
    prefix = f"model.layers.{i}" if i >= spec.n_layers else None
    if prefix is not None:                                 # a multi-token-prediction layer: its extra tensors travel unchanged
        for name in ("enorm", "hnorm", "shared_head.norm"):
            out[f"{prefix}.{name}.weight"] = _vector(ops, f"{prefix}.{name}", "").to(torch.bfloat16)
        out[f"{prefix}.eh_proj.weight"] = _dequant(ops[f"{prefix}.eh_proj"]).to(torch.bfloat16)
    for key, stem in layer_stems(spec, i, prefix).items():
        if key in VECTORS:
            v = _vector(ops, stem, key)
            name = stem if key in ("router_bias", "sink") else f"{stem}.weight"
            out[name] = v.to(torch.float32 if key in ("router_bias", "sink") else torch.bfloat16)
        elif _is_expert(key):
            _emit(out, dt, stem, _dequant(ops[stem]), experts)
        elif key in ("router", "wkv_b"):
            _emit(out, dt, stem, _dequant(ops[stem]), "bf16")
        else:
            _emit(out, dt, stem, _dequant(ops[stem]), dense)
    return out, dt


def _publish(dst: Path, src: Path, run: dict):
    weight_map, total = {}, 0
    for unit, rec in sorted(run["done"].items()):
        hdr, _ = read_header(dst / rec["file"])
        for name in hdr:
            if name != "__metadata__":
                weight_map[name] = rec["file"]
        total += rec["bytes"]
    _atomic_json(dst / "model.safetensors.index.json", {"metadata": {"total_size": total}, "weight_map": weight_map})
    for name in SIDE_FILES:
        if (src / name).exists():
            shutil.copyfile(src / name, dst / name)
    from ..config import SPEC_FILE, spec_from_json, spec_to_json
    if (src / SPEC_FILE).exists():                         # synthetic snapshots carry their spec; record the new formats in it
        import dataclasses
        spec = spec_from_json(json.loads((src / SPEC_FILE).read_text()))
        spec = spec.replace(quant=dataclasses.replace(spec.quant, dense=run["dense"], experts=run["experts"]))
        (dst / SPEC_FILE).write_text(json.dumps(spec_to_json(spec), indent=1))


def quantize_snapshot(src: str | Path, dst: str | Path, spec: ModelSpec, *, dense: str = "nvfp4", experts: str = "mxfp4",
                      restart: bool = False, stop_after: int | None = None, log=None) -> dict:
    """Returns {"written": [...], "skipped": [...], "published": True}."""
    src, dst = Path(src), Path(dst)
    dst.mkdir(parents=True, exist_ok=True)
    ident = recovery_identity(src, spec, dense, experts)
    run_path = dst / RUN_FILE
    run = {"identity": ident, "dense": dense, "experts": experts, "done": {}, "state": "running"}
    if run_path.exists() and not restart:
        old = json.loads(run_path.read_text())
        if old.get("identity") != ident:
            raise ValueError(f"{run_path} belongs to another run (source, shape or formats differ); pass restart=True to discard it")
        run = old
        run["state"] = "running"
    elif restart:
        for f in dst.glob("unit-*.safetensors"):
            f.unlink()
    ops = _ops_of(src)
    written, skipped = [], []
    for n, unit in enumerate(_unit_names(spec)):
        rec = run["done"].get(unit)
        f = dst / f"unit-{unit}.safetensors"
        if rec and f.exists() and f.stat().st_size == rec["bytes"]:
            skipped.append(unit)
            continue
        tensors, dtypes = _encode_unit(ops, spec, unit, dense, experts)
        tmp = dst / f".unit-{unit}.partial"
        write_file(tmp, tensors, dtypes)
        os.replace(tmp, f)
        run["done"][unit] = {"file": f.name, "bytes": f.stat().st_size}
        _atomic_json(run_path, run)
        written.append(unit)
        if log:
            log(f"{unit}: {f.stat().st_size / 1e6:.1f} MB")
        if stop_after is not None and len(written) >= stop_after:
            raise Interrupted(f"stopped after {len(written)} units")
    _publish(dst, src, run)
    run["state"] = "published"
    _atomic_json(run_path, run)
    for stale in dst.glob(".unit-*.partial"):
        stale.unlink()
    return {"written": written, "skipped": skipped, "published": True}
