"""Numeric-format oracles (pure PyTorch, CPU, fp32/fp64).

Formats handled exactly as checkpoints ship them:
  * E4M3 (finite, max 448) bytes, E2M1 (FP4) nibbles packed low-nibble-first,
  * UE8M0 power-of-two scales (value 2**(b-127)),
  * MXFP4  = E2M1 + one UE8M0 scale per 32 elements along K,
  * NVFP4  = E2M1 + one E4M3 scale per 16 elements + one fp32 per-tensor scale (ModelOpt),
  * FP8 block = E4M3 + fp32 scale per 128x128 (or 32x32 UE8M0) weight block,
  * activation "wire rows": E4M3 + UE8M0 per 32 (amax floor 1e-4, scale = 2**ceil(log2(amax/448))).

Behavioural references: python/reference/cuteafd_reference/quant_ref.py:13-159,
python/reference/families/deepseek_v4/kernel_torch.py:21-140, native/shared/cuda/common.h.
Every CUDA kernel in `csrc/` that touches these formats is tested against these functions.
"""
from __future__ import annotations

import math

import torch

E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                            -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=torch.float32)
E4M3_MAX = 448.0
E2M1_MAX = 6.0


# ---------------------------------------------------------------- E4M3 ----
def e4m3_decode(b: torch.Tensor) -> torch.Tensor:
    """uint8 E4M3 (fn variant: no inf, 0x7f/0xff = NaN) -> fp32."""
    b = b.to(torch.int32)
    sign = torch.where((b & 0x80) != 0, -1.0, 1.0)
    exp = (b >> 3) & 0xF
    man = (b & 7).float()
    sub = man / 8.0 * 2.0 ** -6
    nor = (1.0 + man / 8.0) * torch.pow(2.0, (exp - 7).float())
    out = torch.where(exp == 0, sub, nor) * sign
    return torch.where((b & 0x7F) == 0x7F, torch.full_like(out, float("nan")), out)


_E4M3_TABLE = None


def _e4m3_table() -> torch.Tensor:
    global _E4M3_TABLE
    if _E4M3_TABLE is None:
        _E4M3_TABLE = e4m3_decode(torch.arange(127, dtype=torch.uint8))  # non-negative finite codes, ascending
    return _E4M3_TABLE


def e4m3_encode(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> uint8 E4M3, round-to-nearest-even, saturating at +-448."""
    x = x.float()
    if hasattr(torch, "float8_e4m3fn"):
        return x.clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)
    tab = _e4m3_table()
    mag = x.abs().clamp(max=E4M3_MAX)
    idx = torch.bucketize(mag, tab).clamp(1, 126)
    lo, hi = tab[idx - 1], tab[idx]
    pick_hi = (hi - mag < mag - lo) | ((hi - mag == mag - lo) & (idx % 2 == 0))
    code = torch.where(pick_hi, idx, idx - 1).to(torch.uint8)
    return code | ((x < 0).to(torch.uint8) << 7)


# --------------------------------------------------------------- UE8M0 ----
def ue8m0_decode(b: torch.Tensor) -> torch.Tensor:
    return torch.pow(2.0, b.to(torch.int32).float() - 127.0)


def ue8m0_ceil_encode(scale: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= scale, as UE8M0 byte."""
    e = torch.ceil(torch.log2(scale.float().clamp_min(2.0 ** -127)))
    return (e + 127).clamp(0, 254).to(torch.uint8)


# ---------------------------------------------------------------- E2M1 ----
def e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    return E2M1_VALUES.to(codes.device)[codes.long() & 0xF]


def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit code, round-to-nearest, ties to even code; saturating at 6."""
    mag = x.float().abs().clamp(max=E2M1_MAX)
    # midpoints between consecutive magnitudes; tie goes to the even code
    code = torch.zeros_like(mag, dtype=torch.uint8)
    bounds = [(0.25, False), (0.75, True), (1.25, False), (1.75, True), (2.5, False), (3.5, True), (5.0, False)]
    for i, (b, up_on_tie) in enumerate(bounds):
        code = torch.where((mag > b) | ((mag == b) & up_on_tie), torch.full_like(code, i + 1), code)
    neg = (x < 0) & (code != 0)
    return code | (neg.to(torch.uint8) << 3)


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """[..., K] 4-bit codes -> [..., K/2] bytes, even index in the low nibble."""
    c = codes.to(torch.uint8)
    return (c[..., 0::2] & 0xF) | ((c[..., 1::2] & 0xF) << 4)


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    p = packed.to(torch.uint8)
    out = torch.stack([p & 0xF, (p >> 4) & 0xF], dim=-1)
    return out.reshape(*p.shape[:-1], p.shape[-1] * 2)


# --------------------------------------------------------------- MXFP4 ----
def mxfp4_quantize(w: torch.Tensor):
    """[..., K] fp32 -> (packed [..., K/2] uint8, scales [..., K/32] uint8 UE8M0).
    OCP MX rule: shared exponent = floor(log2(amax)) - 2 (emax of E2M1)."""
    *lead, K = w.shape
    assert K % 32 == 0
    blk = w.float().reshape(*lead, K // 32, 32)
    amax = blk.abs().amax(-1)
    e = torch.floor(torch.log2(amax.clamp_min(2.0 ** -120))) - 2.0
    sb = (e + 127).clamp(0, 254).to(torch.uint8)
    scale = ue8m0_decode(sb).unsqueeze(-1)
    codes = e2m1_encode(blk / scale).reshape(*lead, K)
    return pack_nibbles(codes), sb


def mxfp4_dequantize(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    vals = e2m1_decode(unpack_nibbles(packed))
    *lead, K = vals.shape
    return (vals.reshape(*lead, K // 32, 32) * ue8m0_decode(scales).unsqueeze(-1)).reshape(*lead, K)


# --------------------------------------------------------------- NVFP4 ----
def nvfp4_global_scale(x: torch.Tensor) -> torch.Tensor:
    """ModelOpt per-tensor scale (`weight_scale_2` / `input_scale`): amax / (448 * 6)."""
    return (x.float().abs().amax() / (E4M3_MAX * E2M1_MAX)).clamp_min(1e-12)


def nvfp4_quantize(x: torch.Tensor, global_scale: torch.Tensor | float | None = None):
    """[..., K] -> (packed [..., K/2], block scales [..., K/16] E4M3 bytes, global fp32 scale).
    value ~= e2m1 * e4m3_block_scale * global_scale."""
    *lead, K = x.shape
    assert K % 16 == 0
    xf = x.float()
    gs = nvfp4_global_scale(xf) if global_scale is None else torch.as_tensor(global_scale, dtype=torch.float32)
    blk = xf.reshape(*lead, K // 16, 16)
    target = (blk.abs().amax(-1) / gs / E2M1_MAX).clamp(max=E4M3_MAX)
    sb = e4m3_encode(target)
    eff = (e4m3_decode(sb) * gs).unsqueeze(-1)
    q = torch.where(eff > 0, blk / eff.clamp_min(1e-30), torch.zeros_like(blk))
    codes = e2m1_encode(q).reshape(*lead, K)
    return pack_nibbles(codes), sb, gs


def nvfp4_dequantize(packed: torch.Tensor, block_scales: torch.Tensor, global_scale) -> torch.Tensor:
    vals = e2m1_decode(unpack_nibbles(packed))
    *lead, K = vals.shape
    s = e4m3_decode(block_scales) * torch.as_tensor(global_scale, dtype=torch.float32)
    return (vals.reshape(*lead, K // 16, 16) * s.unsqueeze(-1)).reshape(*lead, K)


# ----------------------------------------------------------- FP8 blocks ----
def fp8_block_quantize(w: torch.Tensor, block: int = 128, pow2: bool = False):
    """[N, K] -> (E4M3 bytes [N, K], scales [ceil(N/b), ceil(K/b)] fp32). Dequant = byte * scale."""
    N, K = w.shape
    nb, kb = -(-N // block), -(-K // block)
    pad = torch.zeros(nb * block, kb * block, dtype=torch.float32)
    pad[:N, :K] = w.float()
    t = pad.reshape(nb, block, kb, block)
    amax = t.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / E4M3_MAX
    if pow2:
        scale = ue8m0_decode(ue8m0_ceil_encode(scale))
    q = e4m3_encode(t / scale[:, None, :, None]).reshape(nb * block, kb * block)[:N, :K]
    return q.contiguous(), scale


def fp8_block_dequantize(q: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    N, K = q.shape
    s = scale.repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return e4m3_decode(q) * s


def act_quant_fp8_ue8m0(x: torch.Tensor, group: int = 32, amax_floor: float = 1e-4):
    """Activation wire rows: [rows, H] -> (E4M3 bytes [rows, H], UE8M0 [rows, H/group]).
    Input is BF16-rounded first; scale = 2**ceil(log2(amax/448))."""
    rows, H = x.shape
    assert H % group == 0
    xb = x.to(torch.bfloat16).float().reshape(rows, H // group, group)
    amax = xb.abs().amax(-1).clamp_min(amax_floor)
    sb = ue8m0_ceil_encode(amax / E4M3_MAX)
    q = e4m3_encode(xb / ue8m0_decode(sb).unsqueeze(-1)).reshape(rows, H)
    return q, sb


def act_dequant_fp8_ue8m0(q: torch.Tensor, sb: torch.Tensor, group: int = 32) -> torch.Tensor:
    rows, H = q.shape
    return (e4m3_decode(q).reshape(rows, H // group, group) * ue8m0_decode(sb).unsqueeze(-1)).reshape(rows, H)


def act_quant_fp8_block(x: torch.Tensor, group: int = 128):
    """Per-token per-128 fp32-scaled FP8 (DeepSeek-V3 activation recipe)."""
    rows, H = x.shape
    xb = x.float().reshape(rows, H // group, group)
    scale = xb.abs().amax(-1).clamp_min(1e-4) / E4M3_MAX
    return e4m3_encode(xb / scale.unsqueeze(-1)).reshape(rows, H), scale


# ------------------------------------------------------- SF atom layout ----
def swizzle_sf_128x4(sf: torch.Tensor) -> torch.Tensor:
    """Re-tile a [rows, n_sf] byte matrix of block scales into the 128x4 scale-factor atom
    layout tcgen05 block-scaled MMAs read from tensor memory: 512-byte chunks
    [row_block(128 rows)][k_chunk(4 SFs)], inside a chunk byte offset = (r%32)*16 + (r//32)*4 + s.
    Rows and SFs are zero-padded up to multiples of 128 and 4.  (Same job as the reference's
    native/shared/cuda/nvfp4_scale.cu:22 swizzle kernel; one-time, at load.)"""
    rows, n = sf.shape
    R, C = -(-rows // 128) * 128, -(-n // 4) * 4
    pad = torch.zeros(R, C, dtype=torch.uint8)
    pad[:rows, :n] = sf
    t = pad.reshape(R // 128, 4, 32, C // 4, 4)        # [rb, r//32, r%32, kc, s]
    return t.permute(0, 3, 2, 1, 4).contiguous().reshape(-1)  # [rb, kc, r%32, r//32, s]


def unswizzle_sf_128x4(flat: torch.Tensor, rows: int, n: int) -> torch.Tensor:
    R, C = -(-rows // 128) * 128, -(-n // 4) * 4
    t = flat.reshape(R // 128, C // 4, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(R, C)
    return t[:rows, :n].contiguous()


def log2_ceil(x: float) -> int:
    return int(math.ceil(math.log2(x)))
