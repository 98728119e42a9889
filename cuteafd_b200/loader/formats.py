"""Storage-format detection: group checkpoint tensors that share a stem into one logical weight (`QuantOperand`)
and say how it is encoded, from names, dtypes and shapes alone - never from a side file.

Recognised layouts (all as shipped in HF snapshots):
  bf16 / f16 / f32               x.weight
  FP8 block                      x.weight (F8_E4M3) + x.weight_scale_inv (F32 [N/128, K/128], or F8_E8M0 [N/32, K/32])
  MXFP4                          x.weight | x.blocks (U8, K/2) + x.weight_scale | x.scales (U8/F8_E8M0, K/32)
  NVFP4 (ModelOpt)               x.weight (U8, K/2) + x.weight_scale (F8_E4M3, K/16) + x.weight_scale_2 (F32) [+ x.input_scale]
  EXL3                           x.trellis (I16 [K/16, N/16, 16*bits]) + x.suh + x.svh [+ x.mcg / x.mul1]
A group that does not describe one consistent operand comes back as `Malformed` with the reason; "unsupported is a
result, not a crash".  Reference: cuteafd-loader/src/plan/format.rs:1-110, formats/exl3_format.rs:1-36,
formats/modelopt.rs, formats/fp8_experts.rs.
"""
from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass, field

from .safetensors_io import TensorInfo

SUFFIXES = ("weight_scale_inv", "weight_scale_2", "weight_scale", "input_scale", "weight", "blocks", "scales", "trellis",
            "suh", "svh", "mcg", "mul1", "bias", "e_score_correction_bias")


@dataclass
class QuantOperand:
    stem: str
    encoding: str                       # bf16 f16 f32 e4m3 e5m2 e2m1 exl3 int
    logical: tuple                      # dequantised shape [N, K]
    stored: tuple
    scale_encoding: str | None = None   # f32 bf16 ue8m0 e4m3
    block: tuple | None = None          # (rows, cols) elements per scale
    global_scale: bool = False
    input_scale: bool = False
    bits: float = 16.0
    members: dict = field(default_factory=dict)

    @property
    def format(self) -> str:
        if self.encoding in ("bf16", "f16", "f32"):
            return self.encoding
        if self.encoding == "e4m3":
            return f"fp8_block{self.block[0]}" if self.block else "fp8"
        if self.encoding == "e2m1":
            return "nvfp4" if self.scale_encoding == "e4m3" else "mxfp4"
        if self.encoding == "exl3":
            return f"exl3_k{self.bits:g}"
        return self.encoding

    @property
    def nbytes(self) -> int:
        return sum(t.nbytes for t in self.members.values())


@dataclass
class Malformed:
    stem: str
    reason: str


def split_stem(name: str) -> tuple[str, str]:
    for s in SUFFIXES:
        if name.endswith("." + s):
            return name[:-len(s) - 1], s
    return name, ""


def group(cat: dict[str, TensorInfo]) -> dict[str, dict[str, TensorInfo]]:
    g: dict = defaultdict(dict)
    for name, info in cat.items():
        stem, suf = split_stem(name)
        g[stem][suf] = info
    return g


def detect(stem: str, m: dict[str, TensorInfo]) -> QuantOperand | Malformed:
    if "trellis" in m:
        t = m["trellis"]
        if len(t.shape) != 3 or t.shape[2] % 16 or "suh" not in m or "svh" not in m:
            return Malformed(stem, "EXL3 group needs trellis [K/16, N/16, 16*bits] with suh and svh")
        bits = t.shape[2] // 16
        K, N = t.shape[0] * 16, t.shape[1] * 16
        if m["suh"].shape != (K,) or m["svh"].shape != (N,):
            return Malformed(stem, f"EXL3 sign vectors {m['suh'].shape}/{m['svh'].shape} do not match trellis geometry ({K}, {N})")
        return QuantOperand(stem, "exl3", (N, K), t.shape, bits=float(bits), members=m)
    w = m.get("weight") or m.get("blocks")
    if w is None:
        return Malformed(stem, "no weight / blocks / trellis member")
    if len(w.shape) < 2:
        enc = {"BF16": "bf16", "F16": "f16", "F32": "f32"}.get(w.dtype, "int")
        return QuantOperand(stem, enc, w.shape, w.shape, members=m)
    *lead, N, Kst = w.shape
    scale = m.get("weight_scale_inv") or m.get("weight_scale") or m.get("scales")
    if w.dtype in ("BF16", "F16", "F32"):
        if scale is not None:
            return Malformed(stem, f"{w.dtype} weight with a scale tensor")
        return QuantOperand(stem, w.dtype.lower(), tuple(w.shape), tuple(w.shape), members=m)
    if w.dtype in ("F8_E4M3", "F8_E5M2"):
        enc = "e4m3" if w.dtype == "F8_E4M3" else "e5m2"
        if scale is None:
            return QuantOperand(stem, enc, tuple(w.shape), tuple(w.shape), bits=8.0, members=m)
        if len(scale.shape) < 2:
            return QuantOperand(stem, enc, tuple(w.shape), tuple(w.shape), scale_encoding=scale.dtype.lower(), block=(N, Kst), bits=8.0, members=m)
        sr, sc = scale.shape[-2:]
        br, bc = -(-N // sr), -(-Kst // sc)
        if (br, bc) not in ((128, 128), (32, 32), (1, 128), (1, 32)):
            return Malformed(stem, f"FP8 scale grid {scale.shape} does not tile weight {w.shape} by a known block")
        se = {"F32": "f32", "BF16": "bf16", "F8_E8M0": "ue8m0", "U8": "ue8m0"}.get(scale.dtype)
        if se is None:
            return Malformed(stem, f"FP8 scale dtype {scale.dtype} not recognised")
        return QuantOperand(stem, enc, tuple(w.shape), tuple(w.shape), scale_encoding=se, block=(br, bc), bits=8.0 + 32.0 / (br * bc), members=m)
    if w.dtype in ("U8", "I8"):
        K = Kst * 2
        if scale is None:
            return Malformed(stem, "packed 4-bit weight without block scales")
        per = K // scale.shape[-1] if scale.shape[-1] else 0
        if scale.dtype == "F8_E4M3" and per == 16:
            if "weight_scale_2" not in m:
                return Malformed(stem, "NVFP4 weight without weight_scale_2")
            return QuantOperand(stem, "e2m1", (*lead, N, K), tuple(w.shape), scale_encoding="e4m3", block=(1, 16), global_scale=True,
                                input_scale="input_scale" in m, bits=4.5, members=m)
        if scale.dtype in ("U8", "F8_E8M0") and per == 32:
            return QuantOperand(stem, "e2m1", (*lead, N, K), tuple(w.shape), scale_encoding="ue8m0", block=(1, 32), bits=4.25, members=m)
        return Malformed(stem, f"4-bit weight with {scale.dtype} scales per {per} elements matches neither MXFP4 nor NVFP4")
    return Malformed(stem, f"unrecognised weight dtype {w.dtype}")


def detect_all(cat: dict[str, TensorInfo]):
    ops, bad = {}, []
    for stem, m in group(cat).items():
        r = detect(stem, m)
        if isinstance(r, Malformed):
            if "" in m and len(m) == 1:         # a plain tensor without a known suffix (norm gains, tables)
                t = m[""]
                ops[stem] = QuantOperand(stem, {"BF16": "bf16", "F16": "f16", "F32": "f32"}.get(t.dtype, "int"), t.shape, t.shape, members=m)
            else:
                bad.append(r)
        else:
            ops[stem] = r
    return ops, bad
