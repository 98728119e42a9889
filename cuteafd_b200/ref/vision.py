"""fp32 oracle of the vision tower: the ViT encoder whose output rows replace the image placeholder tokens of a prompt.

Shape of the tower (Qwen-VL / GLM-V / MoonViT lines): resized RGB image -> `patch` x `patch` patches in merge-group order ->
linear patch embedding (+ optional learned position table, bilinearly resampled to the image's grid) -> `depth` pre-norm blocks
(LayerNorm or RMSNorm; bidirectional multi-head attention with a 2-D rotary embedding: half of the rotary pairs turn with the
patch row, half with the patch column; GELU or SwiGLU MLP) -> final norm -> the `merge` x `merge` patches of a group concatenated
-> two-layer GELU projector to the decoder's hidden size.

Reference: native/shared/include/cuteafd_vision.h (tower description: blocks, merger, fp32 residual),
native/shared/cuda/vision.cu (rope_qkv, norms, activations), native/shared/cuda/vision_qwen.cuh (grid / position table).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class VisionSpec:
    hidden: int = 128
    depth: int = 2
    n_heads: int = 2
    head_dim: int = 64
    intermediate: int = 256
    patch: int = 16
    merge: int = 2
    out_hidden: int = 256
    norm: str = "layernorm"        # "layernorm" | "rmsnorm"
    mlp: str = "gelu"              # "gelu" | "gelu_tanh" | "swiglu"
    qkv_bias: bool = True
    qk_norm: bool = False          # per-head RMSNorm of q and k before the rotation (GLM-V)
    pos_grid: int = 0              # learned position table of pos_grid x pos_grid rows (0: rotary only)
    rope_theta: float = 10000.0
    eps: float = 1e-6
    image_mean: tuple = (0.5, 0.5, 0.5)
    image_std: tuple = (0.5, 0.5, 0.5)
    min_tokens: int = 4            # bounds on merged tokens per image (the resize rule)
    max_tokens: int = 4096

    def replace(self, **kw) -> "VisionSpec":
        return replace(self, **kw)

    @property
    def patch_dim(self) -> int:
        return 3 * self.patch * self.patch

    @staticmethod
    def from_hf_config(v: dict, out_hidden: int | None = None) -> "VisionSpec":
        """Vision section of a Hugging Face config (`vision_config` of the Qwen-VL / GLM-V layouts)."""
        hidden = int(v.get("hidden_size", v.get("embed_dim", 1152)))
        heads = int(v.get("num_heads", v.get("num_attention_heads", 16)))
        act = str(v.get("hidden_act", "gelu"))
        mlp = "swiglu" if act == "silu" else ("gelu_tanh" if "tanh" in act or act == "gelu_new" else "gelu")
        return VisionSpec(hidden=hidden, depth=int(v.get("depth", v.get("num_hidden_layers", 27))), n_heads=heads, head_dim=hidden // heads,
                          intermediate=int(v.get("intermediate_size", 4 * hidden)), patch=int(v.get("patch_size", 16)),
                          merge=int(v.get("spatial_merge_size", 2)), out_hidden=int(out_hidden or v.get("out_hidden_size", hidden)),
                          norm="rmsnorm" if mlp == "swiglu" else "layernorm", mlp=mlp, qk_norm=bool(v.get("qk_norm", False)),
                          pos_grid=int(math.isqrt(int(v.get("num_position_embeddings", 0)))), eps=float(v.get("rms_norm_eps", 1e-6)))


def init_vision_weights(spec: VisionSpec, seed: int = 0) -> dict:
    g = torch.Generator().manual_seed(seed)
    H, I, HD = spec.hidden, spec.intermediate, spec.n_heads * spec.head_dim

    def mat(n, k, std=None):
        return torch.randn(n, k, generator=g) * (std if std is not None else k ** -0.5)

    def vec(n, std=0.1):
        return torch.randn(n, generator=g) * std

    w = {"patch_w": mat(H, spec.patch_dim), "patch_b": vec(H)}
    if spec.pos_grid:
        w["pos_embed"] = torch.randn(spec.pos_grid * spec.pos_grid, H, generator=g) * 0.1
    blocks = []
    for _ in range(spec.depth):
        b = {"norm1_w": 1 + vec(H), "norm2_w": 1 + vec(H), "qkv_w": mat(3 * HD, H), "proj_w": mat(H, HD), "proj_b": vec(H)}
        if spec.norm == "layernorm":
            b["norm1_b"], b["norm2_b"] = vec(H), vec(H)
        if spec.qkv_bias:
            b["qkv_b"] = vec(3 * HD)
        if spec.qk_norm:
            b["q_norm"], b["k_norm"] = 1 + vec(spec.head_dim), 1 + vec(spec.head_dim)
        b["fc1_w"] = mat((2 if spec.mlp == "swiglu" else 1) * I, H)        # swiglu: rows [gate | up]
        b["fc1_b"] = vec((2 if spec.mlp == "swiglu" else 1) * I)
        b["fc2_w"], b["fc2_b"] = mat(H, I), vec(H)
        blocks.append(b)
    w["blocks"] = blocks
    M = spec.merge * spec.merge * H
    w["merger_norm_w"] = 1 + vec(H)
    if spec.norm == "layernorm":
        w["merger_norm_b"] = vec(H)
    w["merger_fc1_w"], w["merger_fc1_b"] = mat(M, M), vec(M)
    w["merger_fc2_w"], w["merger_fc2_b"] = mat(spec.out_hidden, M), vec(spec.out_hidden)
    return w


def vision_bf16_round(w):
    """Matrices as the device holds them (bf16); vectors stay fp32."""
    if isinstance(w, dict):
        return {k: vision_bf16_round(v) if isinstance(v, (dict, list)) else (v.bfloat16().float() if v.dim() == 2 else v) for k, v in w.items()}
    return [vision_bf16_round(v) for v in w]


def smart_grid(height: int, width: int, spec: VisionSpec) -> tuple[int, int]:
    """Patch grid (rows, columns) for an image: both sides rounded to whole merge groups, the merged token count kept inside
    [min_tokens, max_tokens] with the aspect ratio preserved as far as rounding allows."""
    unit = spec.patch * spec.merge
    gh, gw = max(1, round(height / unit)), max(1, round(width / unit))
    if gh * gw > spec.max_tokens:
        s = math.sqrt(height * width / (spec.max_tokens * unit * unit))
        gh, gw = max(1, math.floor(height / s / unit)), max(1, math.floor(width / s / unit))
    if gh * gw < spec.min_tokens:
        s = math.sqrt(spec.min_tokens * unit * unit / (height * width))
        gh, gw = max(1, math.ceil(height * s / unit)), max(1, math.ceil(width * s / unit))
    return gh * spec.merge, gw * spec.merge


def patch_order(gh: int, gw: int, m: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(row, column) of every patch in merge-group order: groups row-major, the m x m patches of a group row-major inside it."""
    ys, xs = torch.meshgrid(torch.arange(gh), torch.arange(gw), indexing="ij")
    ys = ys.reshape(gh // m, m, gw // m, m).permute(0, 2, 1, 3).reshape(-1)
    xs = xs.reshape(gh // m, m, gw // m, m).permute(0, 2, 1, 3).reshape(-1)
    return ys, xs


def normalisation_lut(spec: VisionSpec) -> torch.Tensor:
    """fp32 [3, 256]: (byte / 255 - mean) / std per channel."""
    v = torch.arange(256, dtype=torch.float32) / 255.0
    return torch.stack([(v - m) / s for m, s in zip(spec.image_mean, spec.image_std)])


def rgb_to_patches(rgb: torch.Tensor, spec: VisionSpec) -> torch.Tensor:
    """uint8 [gh * P, gw * P, 3] -> fp32 [gh * gw, 3 * P * P] (merge-group order, columns (channel, py, px))."""
    P, m = spec.patch, spec.merge
    gh, gw = rgb.shape[0] // P, rgb.shape[1] // P
    lut = normalisation_lut(spec)
    x = torch.stack([lut[c][rgb[..., c].long()] for c in range(3)])                       # [3, Hpx, Wpx]
    x = x.reshape(3, gh, P, gw, P).permute(1, 3, 0, 2, 4).reshape(gh, gw, 3 * P * P)
    ys, xs = patch_order(gh, gw, m)
    return x[ys, xs]


def rope_table(gh: int, gw: int, spec: VisionSpec) -> torch.Tensor:
    """fp32 [gh * gw, head_dim]: cos[hd / 2] | sin[hd / 2]; the first hd / 4 angles follow the patch row, the rest its column."""
    q = spec.head_dim // 4
    inv = spec.rope_theta ** (-torch.arange(q, dtype=torch.float32) * 2 / (spec.head_dim // 2))
    ys, xs = patch_order(gh, gw, spec.merge)
    ang = torch.cat([ys[:, None].float() * inv, xs[:, None].float() * inv], dim=1)        # [N, hd / 2]
    return torch.cat([ang.cos(), ang.sin()], dim=1)


def position_rows(table: torch.Tensor, gh: int, gw: int, spec: VisionSpec) -> torch.Tensor:
    """Learned position table [pos_grid^2, H] resampled bilinearly (corner-aligned) to the gh x gw grid, in merge-group order."""
    n = spec.pos_grid
    t = table.reshape(n, n, -1).permute(2, 0, 1)[None]
    r = F.interpolate(t, size=(gh, gw), mode="bilinear", align_corners=True)[0].permute(1, 2, 0)
    ys, xs = patch_order(gh, gw, spec.merge)
    return r[ys, xs]


def _norm(x, w, b, eps):
    if b is not None:
        return F.layer_norm(x, (x.shape[-1],), w, b, eps)
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _act(y, kind):
    if kind == "swiglu":
        g, u = y.chunk(2, dim=-1)
        return F.silu(g) * u
    return F.gelu(y, approximate="tanh" if kind == "gelu_tanh" else "none")


def _rotate(x, cs):
    """x [N, nh, hd]; pairs (d, d + hd / 2)."""
    half = x.shape[-1] // 2
    c, s = cs[:, None, :half], cs[:, None, half:]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def vision_forward(spec: VisionSpec, w: dict, patches: torch.Tensor, gh: int, gw: int, taps: dict | None = None) -> torch.Tensor:
    """One image: patches fp32 [gh * gw, 3 P^2] -> [gh * gw / merge^2, out_hidden]."""
    N, nh, hd = patches.shape[0], spec.n_heads, spec.head_dim
    x = patches @ w["patch_w"].T + w["patch_b"]
    if spec.pos_grid:
        x = x + position_rows(w["pos_embed"], gh, gw, spec)
    cs = rope_table(gh, gw, spec)
    if taps is not None:
        taps["embed"] = x.clone()
    x = encoder_blocks(spec, w["blocks"], x, cs, taps)
    h = _norm(x, w["merger_norm_w"], w.get("merger_norm_b"), spec.eps).reshape(N // spec.merge ** 2, -1)
    h = F.gelu(h @ w["merger_fc1_w"].T + w["merger_fc1_b"])
    return h @ w["merger_fc2_w"].T + w["merger_fc2_b"]


def encoder_blocks(spec, blocks: list, x: torch.Tensor, cs: torch.Tensor | None, taps: dict | None = None) -> torch.Tensor:
    """Pre-norm bidirectional transformer blocks over one item's rows x [N, hidden]; `cs`: rotary table or None (no rotation)."""
    N, nh, hd = x.shape[0], spec.n_heads, spec.head_dim
    for i, b in enumerate(blocks):
        h = _norm(x, b["norm1_w"], b.get("norm1_b"), spec.eps)
        qkv = h @ b["qkv_w"].T + (b["qkv_b"] if "qkv_b" in b else 0)
        q, k, v = (t.reshape(N, nh, hd) for t in qkv.chunk(3, dim=-1))
        if spec.qk_norm:
            q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + spec.eps) * b["q_norm"]
            k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + spec.eps) * b["k_norm"]
        if cs is not None:
            q, k = _rotate(q, cs), _rotate(k, cs)
        p = torch.softmax(torch.einsum("qhd,khd->hqk", q, k) * hd ** -0.5, dim=-1)
        o = torch.einsum("hqk,khd->qhd", p, v).reshape(N, nh * hd)
        x = x + o @ b["proj_w"].T + b["proj_b"]
        h = _norm(x, b["norm2_w"], b.get("norm2_b"), spec.eps)
        x = x + _act(h @ b["fc1_w"].T + b["fc1_b"], spec.mlp) @ b["fc2_w"].T + b["fc2_b"]
        if taps is not None:
            taps[f"block{i}"] = x.clone()
    return x
