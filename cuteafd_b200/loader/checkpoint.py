"""Checkpoint reader: an HF-layout snapshot (safetensors shards, tensors named as the model families ship them) ->
weights in the formats the kernels consume, WITHOUT repacking the payloads:

  * bf16 / f16 / f32 linears -> bf16 operands;
  * FP8 E4M3 with fp32 `weight_scale_inv` per 128 x 128 block -> the FP8 block-scaled GEMM kind (bytes and scale grid as stored);
  * NVFP4 (`weight` packed E2M1, `weight_scale` E4M3 per 16, `weight_scale_2` fp32, optional `input_scale`) and MXFP4
    (`blocks` packed E2M1 + `scales` UE8M0 per 32) -> the FP4 kinds (payload as stored; the block scales are re-tiled once
    on the device into the tensor-core scale-factor atom layout);
  * EXL3 (`trellis`, `suh`, `svh`) -> `ops.Exl3Weight` as stored.

Two consumers:
  `read_masters(snapshot, spec)`         fp32 masters on the CPU (dequantised with the format oracles) for `ref.model.RefModel`;
  `load_device_weights(snapshot, ...)`   `models.weights.DeviceWeights` on a GPU for the engines (optionally one expert range).
`export_snapshot` writes masters back out in that layout (optionally quantised) - the synthetic checkpoints of the tests.

Tensor names follow the HF modelling code of the families (Qwen3-MoE style GQA decoders, DeepSeek-V3 style MLA decoders);
reference counterparts: cuteafd-loader/src/{catalog,formats,files}.rs and the per-family tensor maps
(families/deepseek_v4/tensors.rs, families/qwen4/tensors.rs).
"""
from __future__ import annotations

from pathlib import Path

import torch

from ..config import ModelSpec
from ..ref import quant
from . import formats
from .safetensors_io import catalog, read_tensor, write_file


# ------------------------------------------------------------------ names
def layer_stems(spec: ModelSpec, i: int, prefix: str | None = None) -> dict:
    """Logical weight name -> tensor-name stem (without `.weight`) of decoder layer i."""
    p = prefix or f"model.layers.{i}"
    a, m = spec.attn, spec.moe
    s = {"attn_norm": f"{p}.input_layernorm", "ffn_norm": f"{p}.post_attention_layernorm"}
    if a.kind == "mla":
        if a.q_lora_rank:
            s.update(wq_a=f"{p}.self_attn.q_a_proj", q_a_norm=f"{p}.self_attn.q_a_layernorm", wq_b=f"{p}.self_attn.q_b_proj")
        else:
            s.update(wq=f"{p}.self_attn.q_proj")
        s.update(wkv_a=f"{p}.self_attn.kv_a_proj_with_mqa", kv_a_norm=f"{p}.self_attn.kv_a_layernorm",
                 wkv_b=f"{p}.self_attn.kv_b_proj", wo=f"{p}.self_attn.o_proj")
        if a.index_topk:           # sparse-attention indexer
            s.update(wq_idx=f"{p}.self_attn.indexer.wq_b", wk_idx=f"{p}.self_attn.indexer.wk", w_idx=f"{p}.self_attn.indexer.weights_proj")
    elif spec.layer_is_linear(i) and prefix is None:      # gated delta-rule layer (MTP draft layers are full-attention layers)
        q = f"{p}.linear_attn"
        s.update(w_qkvz=f"{q}.in_proj_qkvz", w_ba=f"{q}.in_proj_ba", conv_w=f"{q}.conv1d", dt_bias=f"{q}.dt_bias", a_log=f"{q}.A_log",
                 lin_norm=f"{q}.norm", wo=f"{q}.out_proj")
    else:
        s.update(wq=f"{p}.self_attn.q_proj", wk=f"{p}.self_attn.k_proj", wv=f"{p}.self_attn.v_proj", wo=f"{p}.self_attn.o_proj")
        if a.qk_norm:
            s.update(q_norm=f"{p}.self_attn.q_norm", k_norm=f"{p}.self_attn.k_norm")
        if spec.layer_has_sink(i):
            s.update(sink=f"{p}.self_attn.sinks")
    if spec.hyper_streams:          # hyper-connections: projection / scale / base of the boundary in front of each block
        for blk in ("attn", "ffn"):
            s.update({f"hc_{blk}_fn": f"{p}.hc_{blk}.fn", f"hc_{blk}_scale": f"{p}.hc_{blk}.scale", f"hc_{blk}_base": f"{p}.hc_{blk}.base"})
    if spec.is_moe_layer(i):
        s.update(router=f"{p}.mlp.gate")
        if m.use_bias:
            s.update(router_bias=f"{p}.mlp.gate.e_score_correction_bias")
        for e in range(m.n_experts):
            s.update({f"w_gate.{e}": f"{p}.mlp.experts.{e}.gate_proj", f"w_up.{e}": f"{p}.mlp.experts.{e}.up_proj",
                      f"w_down.{e}": f"{p}.mlp.experts.{e}.down_proj"})
        if m.shared_inter:
            s.update(ws_gate=f"{p}.mlp.shared_experts.gate_proj", ws_up=f"{p}.mlp.shared_experts.up_proj",
                     ws_down=f"{p}.mlp.shared_experts.down_proj")
    else:
        s.update(wd_gate=f"{p}.mlp.gate_proj", wd_up=f"{p}.mlp.up_proj", wd_down=f"{p}.mlp.down_proj")
    return s


VECTORS = ("attn_norm", "ffn_norm", "q_norm", "k_norm", "q_a_norm", "kv_a_norm", "sink", "router_bias", "lin_norm")
# small fp32 tensors stored as they are (`<stem>.weight`, F32): convolution taps, decay parameters, hyper-connection coefficients
PLAIN_F32 = ("conv_w", "dt_bias", "a_log", "hc_attn_fn", "hc_attn_scale", "hc_attn_base", "hc_ffn_fn", "hc_ffn_scale", "hc_ffn_base")


def _is_expert(key: str) -> bool:
    return key.split(".")[0] in ("w_gate", "w_up", "w_down")


# ------------------------------------------------------------------ export (synthetic checkpoints)
def _emit(out: dict, dtypes: dict, stem: str, w: torch.Tensor, fmt: str, input_amax: float | None = None):
    """One linear [N, K] in format `fmt` under HF-style member names.  `input_amax` (NVFP4) adds the calibrated
    `input_scale` = amax / (448 * 6) a ModelOpt export carries."""
    if fmt == "bf16":
        out[f"{stem}.weight"] = w.to(torch.bfloat16)
    elif fmt == "fp8_block128":
        q, s = quant.fp8_block_quantize(w)
        out[f"{stem}.weight"], out[f"{stem}.weight_scale_inv"] = q, s.float()
        dtypes[f"{stem}.weight"] = "F8_E4M3"
    elif fmt == "nvfp4":
        p, s, gs = quant.nvfp4_quantize(w)
        out[f"{stem}.weight"], out[f"{stem}.weight_scale"] = p, s
        out[f"{stem}.weight_scale_2"] = torch.tensor(float(gs), dtype=torch.float32).reshape(())
        dtypes[f"{stem}.weight_scale"] = "F8_E4M3"
        if input_amax is not None:
            out[f"{stem}.input_scale"] = torch.tensor(float(input_amax) / (448.0 * 6.0), dtype=torch.float32).reshape(())
    elif fmt == "mxfp4":
        p, s = quant.mxfp4_quantize(w)
        out[f"{stem}.blocks"], out[f"{stem}.scales"] = p, s          # packed codes [N, K / 2], UE8M0 [N, K / 32]
    else:
        raise ValueError(f"export: unknown format {fmt}")


def export_snapshot(spec: ModelSpec, masters: dict, path: str | Path, *, dense: str = "bf16", experts: str = "bf16",
                    shard_layers: int = 0, input_amax: float | None = None) -> Path:
    """Writes `masters` (the oracle's weight dict) as an HF-layout snapshot: one safetensors shard per `shard_layers` layers
    (0 = one file).  `dense` / `experts` choose the storage format of the projections and of the routed experts."""
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    shards: dict[int, tuple[dict, dict]] = {}

    def shard(i):
        return shards.setdefault(i // shard_layers if shard_layers else 0, ({}, {}))

    out, dt = shard(0)
    out["model.embed_tokens.weight"] = masters["embed"].to(torch.bfloat16)
    out["model.norm.weight"] = masters["final_norm"].to(torch.bfloat16)
    if spec.hyper_streams:
        for k in ("fn", "scale", "base"):
            out[f"model.hc_head.{k}.weight"] = masters[f"hc_head_{k}"].to(torch.float32).contiguous()
    if not spec.tie_embeddings:
        out["lm_head.weight"] = masters["lm_head"].to(torch.bfloat16)

    def put_layer(i, lw, prefix=None):
        out, dt = shard(min(i, spec.n_layers - 1))
        stems = layer_stems(spec, i, prefix)
        for key, stem in stems.items():
            base = key.split(".")[0]
            if key in VECTORS:
                name = stem if key == "router_bias" or key == "sink" else f"{stem}.weight"
                out[name] = lw[key].to(torch.float32 if key in ("router_bias", "sink") else torch.bfloat16)
            elif key in PLAIN_F32:
                out[f"{stem}.weight"] = lw[key].to(torch.float32).contiguous()
            elif key in ("w_ba", "wq_idx", "wk_idx", "w_idx"):      # projections the kernels keep in bf16 whatever the dense format
                _emit(out, dt, stem, lw[key], "bf16")
            elif _is_expert(key):
                _emit(out, dt, stem, lw[base][int(key.split(".")[1])], experts, input_amax)
            elif key == "router" or key == "wkv_b":
                _emit(out, dt, stem, lw[key], "bf16")
            else:
                _emit(out, dt, stem, lw[key], dense, input_amax)

    for i, lw in enumerate(masters["layers"]):
        put_layer(i, lw)
    for d, mw in enumerate(masters.get("mtp", [])):
        i = spec.n_layers + d
        p = f"model.layers.{i}"
        out, dt = shard(spec.n_layers - 1)
        out[f"{p}.enorm.weight"], out[f"{p}.hnorm.weight"] = mw["enorm"].to(torch.bfloat16), mw["hnorm"].to(torch.bfloat16)
        out[f"{p}.eh_proj.weight"] = mw["eh_proj"].to(torch.bfloat16)
        out[f"{p}.shared_head.norm.weight"] = mw["norm"].to(torch.bfloat16)
        put_layer(i, mw["layer"], p)
    n = len(shards)
    for k, (tensors, dtypes) in sorted(shards.items()):
        write_file(path / f"model-{k + 1:05d}-of-{n:05d}.safetensors", tensors, dtypes)
    import dataclasses
    import json
    from ..config import SPEC_FILE, QuantSpec, spec_to_json
    stored = spec.replace(quant=dataclasses.replace(spec.quant, dense=dense, experts=experts) if isinstance(spec.quant, QuantSpec) else spec.quant)
    (path / SPEC_FILE).write_text(json.dumps(spec_to_json(stored), indent=1))
    return path


# ------------------------------------------------------------------ decode on the host (oracle input)
def _dequant(op: formats.QuantOperand) -> torch.Tensor:
    """fp32 [N, K] of one detected operand."""
    m = op.members
    f = op.format
    if f in ("bf16", "f16", "f32"):
        return read_tensor(m.get("weight") or m[""]).float()
    if f == "fp8_block128":
        return quant.fp8_block_dequantize(read_tensor(m["weight"]), read_tensor(m["weight_scale_inv"]).float())
    if f == "nvfp4":
        return quant.nvfp4_dequantize(read_tensor(m["weight"]), read_tensor(m["weight_scale"]), float(read_tensor(m["weight_scale_2"])))
    if f == "mxfp4":
        b = read_tensor(m["blocks"])
        return quant.mxfp4_dequantize(b.reshape(b.shape[0], -1), read_tensor(m["scales"]))
    if f.startswith("exl3"):
        from ..ref import exl3
        w = exl3.dequantize(read_tensor(m["trellis"]).view(torch.uint16).numpy(), read_tensor(m["suh"]).float().numpy(),
                            read_tensor(m["svh"]).float().numpy())
        return torch.from_numpy(w).float().T.contiguous()          # EXL3 stores input-major [K, N]
    raise NotImplementedError(f"{op.stem}: format {f} has no host decoder")


def _ops_of(snapshot) -> dict:
    ops, bad = formats.detect_all(catalog(snapshot))
    if bad:
        raise ValueError("malformed tensors in snapshot: " + "; ".join(f"{b.stem}: {b.reason}" for b in bad[:5]))
    return ops


def _vector(ops: dict, stem: str, key: str) -> torch.Tensor:
    op = ops.get(stem)
    if op is None:                      # a member of another tensor's group, e.g. `<gate>.e_score_correction_bias`
        base, member = formats.split_stem(stem)
        if member and base in ops and member in ops[base].members:
            return read_tensor(ops[base].members[member]).float()
        raise KeyError(f"tensor {stem} missing from the snapshot")
    return read_tensor(op.members.get("weight") or op.members.get("") or next(iter(op.members.values()))).float()


def read_masters(snapshot: str | Path, spec: ModelSpec) -> dict:
    """fp32 masters (the oracle's dict layout) decoded from a snapshot."""
    ops = _ops_of(snapshot)

    def layer(i, prefix=None):
        lw, stems = {}, layer_stems(spec, i, prefix)
        experts: dict = {}
        for key, stem in stems.items():
            if key in VECTORS or key in PLAIN_F32:
                lw[key] = _vector(ops, stem, key)
            elif _is_expert(key):
                experts.setdefault(key.split(".")[0], []).append(_dequant(ops[stem]))
            else:
                lw[key] = _dequant(ops[stem])
        for k, v in experts.items():
            lw[k] = torch.stack(v)
        return lw

    w = {"embed": read_tensor(ops["model.embed_tokens"].members["weight"]).float(),
         "final_norm": read_tensor(ops["model.norm"].members["weight"]).float(),
         "layers": [layer(i) for i in range(spec.n_layers)]}
    w["lm_head"] = w["embed"] if spec.tie_embeddings else read_tensor(ops["lm_head"].members["weight"]).float()
    if spec.hyper_streams:
        for k in ("fn", "scale", "base"):
            w[f"hc_head_{k}"] = _vector(ops, f"model.hc_head.{k}", "")
    if spec.mtp_layers:
        w["mtp"] = []
        for d in range(spec.mtp_layers):
            p = f"model.layers.{spec.n_layers + d}"
            w["mtp"].append({"enorm": _vector(ops, f"{p}.enorm", ""), "hnorm": _vector(ops, f"{p}.hnorm", ""),
                             "eh_proj": _dequant(ops[f"{p}.eh_proj"]), "layer": layer(spec.n_layers + d, p),
                             "norm": _vector(ops, f"{p}.shared_head.norm", "")})
    return w


# ------------------------------------------------------------------ device weights in native formats
def _tc_from_operands(group: list, device, act_gs: float):
    """TcWeight over one or several operands of the same format and shape (several = the experts of a layer),
    keeping the stored payload bytes."""
    from .. import ops as K
    from ..ops import TcWeight, encode_tmap, swizzle_sf
    f = group[0].format
    if any(o.format != f or o.logical[-2:] != group[0].logical[-2:] for o in group):
        raise ValueError(f"{group[0].stem}: operands of one group differ in format or shape")
    N, Kd = group[0].logical[-2:]
    G = len(group)
    rd = lambda o, k: read_tensor(o.members[k])
    if f in ("bf16", "f16", "f32"):
        data = torch.stack([rd(o, "weight").to(torch.bfloat16) for o in group]).to(device).contiguous()
        return TcWeight(K.KIND_BF16, G, N, Kd, data, encode_tmap(data, 128))
    if f == "fp8_block128":
        data = torch.stack([rd(o, "weight") for o in group]).to(device).contiguous()
        sw = torch.stack([rd(o, "weight_scale_inv").float() for o in group]).to(device).contiguous()
        return TcWeight(K.KIND_FP8B, G, N, Kd, data, encode_tmap(data, 128), sw)
    if f == "nvfp4":
        data = torch.stack([rd(o, "weight") for o in group]).to(device).contiguous()
        sf = torch.stack([swizzle_sf(rd(o, "weight_scale").to(device), 16) for o in group]).contiguous()
        gs = [float(rd(o, "weight_scale_2")) for o in group]
        # The activation scale is the checkpoint's calibrated `input_scale` (ModelOpt: amax / (448 * 6)); operands launched as
        # one grouped GEMM quantise their input once, so the group shares the largest of its members' scales.  `act_gs` is
        # only the fallback for snapshots that ship no `input_scale`: a fixed scale clips blocks above 6 * 448 * act_gs.
        if all("input_scale" in o.members for o in group):
            act_gs = max(float(rd(o, "input_scale")) for o in group)
        alpha = torch.tensor([g * act_gs for g in gs], dtype=torch.float32, device=device)
        return TcWeight._finish(K.KIND_NVFP4, G, N, Kd, data, sf, alpha, act_gs)
    if f == "mxfp4":
        kind = K.KIND_BY_NAME["mxfp4"]          # W4A8 (FP8 activations) or W4A4, same stored payload and scales
        data = torch.stack([rd(o, "blocks").reshape(N, Kd // 2) for o in group]).to(device).contiguous()
        sf = torch.stack([swizzle_sf(rd(o, "scales").to(device), K.SF_PER_STAGE[kind]) for o in group]).contiguous()
        return TcWeight._finish(kind, G, N, Kd, data, sf, torch.ones(G, dtype=torch.float32, device=device), act_gs)
    raise NotImplementedError(f"{group[0].stem}: format {f} has no tensor-core operand form (EXL3 linears load as ops.Exl3Weight)")


def _share_act_scale(a, b):
    """Two NVFP4 operands that multiply the SAME quantised activation (gate and up of a SwiGLU) must agree on its global
    scale: both take the larger one and their output scales (weight scale x activation scale) follow."""
    from .. import ops as K
    if a is None or b is None or a.kind != K.KIND_NVFP4 or b.kind != K.KIND_NVFP4:
        return
    ga, gb = 1.0 / float(a.inv_act_gs[0]), 1.0 / float(b.inv_act_gs[0])
    g = max(ga, gb)
    for w, old in ((a, ga), (b, gb)):
        if old != g:
            w.alpha.mul_(g / old)
            w.inv_act_gs.fill_(1.0 / g)


def _fuse_rows(parts: list, device, act_gs: float):
    """Row-wise concatenation of projections that share their input (q, k, v) into one operand."""
    from .. import ops as K
    from ..ops import TcWeight, encode_tmap
    ws = [_tc_from_operands([p], device, act_gs) for p in parts]
    kind = ws[0].kind
    if any(w.kind != kind for w in ws):
        raise ValueError("q/k/v projections are stored in different formats")
    N, Kd = sum(w.N for w in ws), ws[0].K
    if kind == K.KIND_BF16:
        data = torch.cat([w.data for w in ws], 1).contiguous()
        return TcWeight(kind, 1, N, Kd, data, encode_tmap(data, 128))
    if kind == K.KIND_FP8B:
        if any(w.N % 128 for w in ws[:-1]):
            raise NotImplementedError("fusing FP8 projections needs row counts that are multiples of the 128-row scale block")
        data = torch.cat([w.data for w in ws], 1).contiguous()
        return TcWeight(kind, 1, N, Kd, data, encode_tmap(data, 128), torch.cat([w.sf for w in ws], 1).contiguous())
    raise NotImplementedError("FP4 q/k/v projections carry separate global scales; store them fused or as bf16 / FP8")


def load_device_weights(snapshot: str | Path, spec: ModelSpec, device, *, experts_range: tuple | None = None, act_gs: float = 1.0 / 64):
    """`DeviceWeights` of a GQA decoder straight from a snapshot (payloads as stored; see the module docstring)."""
    from ..models.weights import DeviceWeights, LayerWeights
    from ..ops import TcWeight
    if spec.attn.kind != "gqa":
        raise NotImplementedError("load_device_weights builds GQA decoders; MLA snapshots go through read_masters + engine.mla")
    if spec.attn.linear_every or spec.hyper_streams:
        # stacks with gated delta-rule layers or hyper-connections: decoded on the host and re-packed (their projections are bf16)
        if experts_range is not None:
            raise NotImplementedError("expert ranges of hybrid / hyper-connection snapshots")
        return DeviceWeights.from_masters(spec, read_masters(snapshot, spec), device, act_gs)
    ops = _ops_of(snapshot)
    m = spec.moe
    e_lo, e_hi = experts_range if experts_range is not None else (0, m.n_experts)
    f32 = lambda t: t.float().to(device).contiguous()
    one = lambda stem: _tc_from_operands([ops[stem]], device, act_gs)

    def layer(i, prefix=None) -> LayerWeights:
        s = layer_stems(spec, i, prefix)
        lw = LayerWeights(attn_norm=f32(_vector(ops, s["attn_norm"], "")), ffn_norm=f32(_vector(ops, s["ffn_norm"], "")),
                          wqkv=_fuse_rows([ops[s["wq"]], ops[s["wk"]], ops[s["wv"]]], device, act_gs), wo=one(s["wo"]))
        if "q_norm" in s:
            lw.q_norm, lw.k_norm = f32(_vector(ops, s["q_norm"], "")), f32(_vector(ops, s["k_norm"], ""))
        if "sink" in s:
            lw.sink = f32(_vector(ops, s["sink"], ""))
        if "router" in s:
            lw.router = one(s["router"])
            if "router_bias" in s:
                lw.router_bias = f32(_vector(ops, s["router_bias"], ""))
            if e_hi > e_lo:
                for name in ("w_gate", "w_up", "w_down"):
                    setattr(lw, name, _tc_from_operands([ops[s[f"{name}.{e}"]] for e in range(e_lo, e_hi)], device, act_gs))
                _share_act_scale(lw.w_gate, lw.w_up)
            if "ws_gate" in s:
                lw.ws_gate, lw.ws_up, lw.ws_down = one(s["ws_gate"]), one(s["ws_up"]), one(s["ws_down"])
        else:
            lw.ws_gate, lw.ws_up, lw.ws_down = one(s["wd_gate"]), one(s["wd_up"]), one(s["wd_down"])
        _share_act_scale(lw.ws_gate, lw.ws_up)
        return lw

    embed = read_tensor(ops["model.embed_tokens"].members["weight"]).to(torch.bfloat16).to(device).contiguous()
    head = embed if spec.tie_embeddings else read_tensor(ops["lm_head"].members["weight"]).to(torch.bfloat16).to(device).contiguous()
    dw = DeviceWeights(spec=spec, embed=embed, final_norm=f32(_vector(ops, "model.norm", "")),
                       lm_head=TcWeight.from_master(head.float().cpu(), "bf16", device), act_gs=act_gs)
    dw.layers = [layer(i) for i in range(spec.n_layers)]
    dw.layer_map = list(range(spec.n_layers))
    for d in range(spec.mtp_layers):
        p = f"model.layers.{spec.n_layers + d}"
        dw.mtp.append((f32(_vector(ops, f"{p}.enorm", "")), f32(_vector(ops, f"{p}.hnorm", "")), one(f"{p}.eh_proj"),
                       layer(spec.n_layers + d, p), f32(_vector(ops, f"{p}.shared_head.norm", ""))))
    return dw
