"""Vision tower weights out of a Hugging Face snapshot (the `visual.*` tensors of the Qwen-VL / GLM-V layouts) -> the fp32 masters
`ref/vision.py` and `models/vision.py` take.

Name map (prefix `visual.` or `model.visual.`):
    patch_embed.proj.weight [H, 3, (T,) P, P]   convolution over non-overlapping patches = a linear layer; a temporal axis (a still
                                               image is the same frame T times) is summed away
    patch_embed.proj.bias, pos_embed.weight
    blocks.N.norm1 / norm2 (.weight, .bias)
    blocks.N.attn.qkv, attn.proj, attn.q_norm / k_norm
    blocks.N.mlp.fc1 / fc2   or   mlp.linear_fc1 / linear_fc2   or   mlp.gate_proj / up_proj / down_proj (SwiGLU)
    merger.ln_q | merger.norm, merger.mlp.0 / mlp.2 | merger.linear_fc1 / linear_fc2

Reference: rust/crates/cuteafd-loader (per-family config readers and tensor catalog), native/shared/include/cuteafd_vision.h
(the tower's weight arena: patch, blocks, merger).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..ref.vision import VisionSpec
from .safetensors_io import catalog, read_tensor


def vision_spec_from_snapshot(snapshot: str | Path) -> tuple[VisionSpec, dict] | None:
    """(spec, token ids {"pad", "start", "end"}) of a snapshot with a `vision_config`; None for text-only models."""
    cfg = json.loads((Path(snapshot) / "config.json").read_text())
    v = cfg.get("vision_config")
    if not isinstance(v, dict):
        return None
    text = cfg.get("text_config") or cfg
    spec = VisionSpec.from_hf_config(v, out_hidden=int(v.get("out_hidden_size") or text.get("hidden_size")))
    ids = {"pad": cfg.get("image_token_id"), "start": cfg.get("vision_start_token_id"), "end": cfg.get("vision_end_token_id")}
    if ids["pad"] is None:
        raise ValueError("vision_config without image_token_id")
    return spec, ids


def read_vision_masters(snapshot: str | Path, spec: VisionSpec) -> dict:
    cat = catalog(snapshot)
    prefix = next((p for p in ("visual.", "model.visual.") if any(k.startswith(p) for k in cat)), None)
    if prefix is None:
        raise ValueError("no visual.* tensors in the snapshot")

    def get(*names, required=True):
        for n in names:
            if prefix + n in cat:
                return read_tensor(cat[prefix + n]).float()
        if required:
            raise KeyError(f"vision tensor missing: {prefix}{names[0]}")
        return None

    pw = get("patch_embed.proj.weight")
    if pw.dim() == 5:
        pw = pw.sum(dim=2)
    w = {"patch_w": pw.reshape(pw.shape[0], -1), "patch_b": get("patch_embed.proj.bias", required=False)}
    if w["patch_b"] is None:
        w["patch_b"] = torch.zeros(pw.shape[0])
    if spec.pos_grid:
        w["pos_embed"] = get("pos_embed.weight")
    blocks = []
    for i in range(spec.depth):
        b = f"blocks.{i}."
        d = {"norm1_w": get(b + "norm1.weight"), "norm2_w": get(b + "norm2.weight"), "qkv_w": get(b + "attn.qkv.weight"),
             "proj_w": get(b + "attn.proj.weight"), "proj_b": get(b + "attn.proj.bias", required=False)}
        H = d["proj_w"].shape[0]
        if d["proj_b"] is None:
            d["proj_b"] = torch.zeros(H)
        for k, n in (("norm1_b", "norm1.bias"), ("norm2_b", "norm2.bias"), ("qkv_b", "attn.qkv.bias"), ("q_norm", "attn.q_norm.weight"),
                     ("k_norm", "attn.k_norm.weight")):
            t = get(b + n, required=False)
            if t is not None:
                d[k] = t
        if spec.mlp == "swiglu":
            gate, up = get(b + "mlp.gate_proj.weight"), get(b + "mlp.up_proj.weight")
            d["fc1_w"] = torch.cat([gate, up])
            gb, ub = get(b + "mlp.gate_proj.bias", required=False), get(b + "mlp.up_proj.bias", required=False)
            d["fc1_b"] = torch.cat([gb if gb is not None else torch.zeros(gate.shape[0]), ub if ub is not None else torch.zeros(up.shape[0])])
            d["fc2_w"] = get(b + "mlp.down_proj.weight")
            d["fc2_b"] = get(b + "mlp.down_proj.bias", required=False)
        else:
            d["fc1_w"], d["fc1_b"] = get(b + "mlp.fc1.weight", b + "mlp.linear_fc1.weight"), get(b + "mlp.fc1.bias", b + "mlp.linear_fc1.bias")
            d["fc2_w"] = get(b + "mlp.fc2.weight", b + "mlp.linear_fc2.weight")
            d["fc2_b"] = get(b + "mlp.fc2.bias", b + "mlp.linear_fc2.bias", required=False)
        if d["fc2_b"] is None:
            d["fc2_b"] = torch.zeros(H)
        blocks.append(d)
    w["blocks"] = blocks
    w["merger_norm_w"] = get("merger.ln_q.weight", "merger.norm.weight")
    mb = get("merger.ln_q.bias", "merger.norm.bias", required=False)
    if mb is not None:
        w["merger_norm_b"] = mb
    w["merger_fc1_w"], w["merger_fc1_b"] = get("merger.mlp.0.weight", "merger.linear_fc1.weight"), get("merger.mlp.0.bias", "merger.linear_fc1.bias")
    w["merger_fc2_w"], w["merger_fc2_b"] = get("merger.mlp.2.weight", "merger.linear_fc2.weight"), get("merger.mlp.2.bias", "merger.linear_fc2.bias")
    return w


def write_vision_snapshot(path: str | Path, spec: VisionSpec, w: dict, temporal: int = 2):
    """Masters -> `visual.*` tensors of a snapshot shard (tests, synthetic snapshots).  The patch convolution is written with a temporal
    axis of `temporal` frames holding equal shares of the still-image weight."""
    from .safetensors_io import write_file
    P = spec.patch
    t = {"visual.patch_embed.proj.weight": (w["patch_w"].reshape(-1, 3, 1, P, P) / temporal).repeat(1, 1, temporal, 1, 1),
         "visual.patch_embed.proj.bias": w["patch_b"]}
    if "pos_embed" in w:
        t["visual.pos_embed.weight"] = w["pos_embed"]
    I = spec.intermediate
    for i, b in enumerate(w["blocks"]):
        p = f"visual.blocks.{i}."
        t[p + "norm1.weight"], t[p + "norm2.weight"] = b["norm1_w"], b["norm2_w"]
        for k, n in (("norm1_b", "norm1.bias"), ("norm2_b", "norm2.bias"), ("qkv_b", "attn.qkv.bias"), ("q_norm", "attn.q_norm.weight"),
                     ("k_norm", "attn.k_norm.weight")):
            if k in b:
                t[p + n] = b[k]
        t[p + "attn.qkv.weight"], t[p + "attn.proj.weight"], t[p + "attn.proj.bias"] = b["qkv_w"], b["proj_w"], b["proj_b"]
        if spec.mlp == "swiglu":
            t[p + "mlp.gate_proj.weight"], t[p + "mlp.up_proj.weight"] = b["fc1_w"][:I], b["fc1_w"][I:]
            t[p + "mlp.gate_proj.bias"], t[p + "mlp.up_proj.bias"] = b["fc1_b"][:I], b["fc1_b"][I:]
            t[p + "mlp.down_proj.weight"], t[p + "mlp.down_proj.bias"] = b["fc2_w"], b["fc2_b"]
        else:
            t[p + "mlp.fc1.weight"], t[p + "mlp.fc1.bias"], t[p + "mlp.fc2.weight"], t[p + "mlp.fc2.bias"] = b["fc1_w"], b["fc1_b"], b["fc2_w"], b["fc2_b"]
    t["visual.merger.ln_q.weight"] = w["merger_norm_w"]
    if "merger_norm_b" in w:
        t["visual.merger.ln_q.bias"] = w["merger_norm_b"]
    t["visual.merger.mlp.0.weight"], t["visual.merger.mlp.0.bias"] = w["merger_fc1_w"], w["merger_fc1_b"]
    t["visual.merger.mlp.2.weight"], t["visual.merger.mlp.2.bias"] = w["merger_fc2_w"], w["merger_fc2_b"]
    write_file(path, {k: v.contiguous() for k, v in t.items()})
