"""Vision tower on the GPU: images -> rows of the decoder's hidden size that replace the image placeholder tokens of a prompt.

The tower is a ViT encoder (`ref/vision.py` is its fp32 oracle and holds `VisionSpec`).  On the device every matrix product is a
bf16 `tc_linear` (tcgen05), the attention is `gqa_prefill_kernel` in its bidirectional mode (window = -1) reading a scratch paged
store, with the heads zero-padded from `head_dim` to the kernel's 128 dimensions (zero key dimensions add nothing to a score, zero
value dimensions come out as zero and meet zero columns of the padded output projection), and the glue is `csrc/vision.cu`: the
residual stays fp32, every GEMM reads bf16 rows written by the fused add + norm / bias + activation kernels.  All images of a call
are packed into one batch: one GEMM per projection for all of them, one attention launch with a sequence per image.

Reference: rust/crates/cuteafd-daemon/src/shared/vision.rs (encoder owner: admission, one encode per image, ledger),
native/shared/cuda/vision_runtime.cu (tower driver), native/shared/src/vision_attention_aot.cc (bf16 varlen attention export).
"""
from __future__ import annotations

import base64
import io

import torch

from .. import ops
from ..ops import KIND_BF16, ActBuffer, TcWeight, native
from ..ops.native import ptr
from ..ref.vision import VisionSpec, normalisation_lut, position_rows, rope_table, smart_grid

PAGE = 64
ACTS = {"none": 0, "gelu": 1, "gelu_tanh": 2, "swiglu": 3}


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


def load_image(data, spec: VisionSpec) -> torch.Tensor:
    """bytes / base64 `data:` URI / PIL image / uint8 [H, W, 3] tensor -> uint8 [gh * P, gw * P, 3] resized to the tower's grid."""
    from PIL import Image
    if isinstance(data, torch.Tensor):
        img = Image.fromarray(data.numpy())
    elif isinstance(data, Image.Image):
        img = data
    else:
        if isinstance(data, str):
            if not data.startswith("data:"):
                raise ValueError("images are passed inline (a data: URI); remote URLs are not fetched")
            data = base64.b64decode(data.split(",", 1)[1])
        img = Image.open(io.BytesIO(data))
    img = img.convert("RGB")
    gh, gw = smart_grid(img.height, img.width, spec)
    img = img.resize((gw * spec.patch, gh * spec.patch), Image.BICUBIC)
    import numpy as np
    return torch.from_numpy(np.asarray(img, dtype=np.uint8).copy())


def image_tokens(rgb: torch.Tensor, spec: VisionSpec) -> int:
    """Rows the tower emits for a resized image (= placeholder tokens its prompt needs)."""
    return (rgb.shape[0] // spec.patch) * (rgb.shape[1] // spec.patch) // spec.merge ** 2


class EncoderTower:
    """Blocks, merger and buffers shared by the vision and audio towers; a subclass adds the front end that fills the fp32 residual
    `x` and the first normed rows `h`.  `group`: rows concatenated by the merger (merge^2 patches, 2 audio frames)."""

    def __init__(self, spec, masters: dict, device, max_rows: int, max_items: int, group: int):
        native.require_gpu_lib()
        if spec.head_dim > 128 or spec.head_dim % 4 or spec.hidden % 8 or spec.intermediate % 8 or spec.out_hidden % 8:
            raise ValueError("encoder tower: head_dim <= 128 and a multiple of 4; widths multiples of 8")
        self.spec, self.device = spec, torch.device(device)
        self.max_patches = N = -(-max_rows // 256) * 256
        self.max_images = max_items
        self.group = group
        H, nh, hd, I = spec.hidden, spec.n_heads, spec.head_dim, spec.intermediate
        dev = self.device
        mat, vec = self._mat, self._vec

        def proj_padded(w):              # [H, nh * hd] -> [H, nh * 128]: zero columns where the attention output is padding
            out = w.new_zeros(w.shape[0], nh, 128)
            out[:, :, :hd] = w.reshape(w.shape[0], nh, hd)
            return out.reshape(w.shape[0], nh * 128)

        self.blocks = []
        for b in masters["blocks"]:
            self.blocks.append({
                "norm1": (vec(b["norm1_w"]), vec(b.get("norm1_b"))), "norm2": (vec(b["norm2_w"]), vec(b.get("norm2_b"))),
                "qkv": mat(b["qkv_w"]), "qkv_b": vec(b.get("qkv_b")), "q_norm": vec(b.get("q_norm")), "k_norm": vec(b.get("k_norm")),
                "proj": mat(proj_padded(b["proj_w"].float())), "proj_b": vec(b["proj_b"]),
                "fc1": mat(b["fc1_w"]), "fc1_b": vec(b["fc1_b"]), "fc2": mat(b["fc2_w"]), "fc2_b": vec(b["fc2_b"])})
        self.merger_norm = (vec(masters["merger_norm_w"]), vec(masters.get("merger_norm_b")))
        self.mfc1 = self.mfc1_b = None              # a single projection (audio) or fc1 -> GELU -> fc2 (vision)
        if "merger_fc1_w" in masters:
            self.mfc1, self.mfc1_b = mat(masters["merger_fc1_w"]), vec(masters["merger_fc1_b"])
        self.mfc2, self.mfc2_b = mat(masters["merger_fc2_w"]), vec(masters["merger_fc2_b"])

        M, fc1_n = group * H, (2 if spec.mlp == "swiglu" else 1) * I
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.x = torch.zeros(N, H, dtype=torch.float32, device=dev)
        self.h = torch.zeros(N, H, **bf)                          # normed rows: input of qkv / fc1 / (as [N / m^2, m^2 H]) the merger
        self.y = torch.zeros(N, H, **bf)                          # GEMM outputs that go into the residual
        self.qkv = torch.zeros(N, 3 * nh * hd, **bf)
        self.q = torch.zeros(N, nh * 128, **bf)
        self.attn = torch.zeros(N, nh * 128, **bf)
        self.f = torch.zeros(N, max(fc1_n, M), **bf)              # fc1 / merger fc1 output before the activation
        self.a = torch.zeros(N, max(I, M), **bf)                  # activated rows
        self.out = torch.zeros(N // group, spec.out_hidden, **bf)
        self.o_raw = torch.zeros(N // group, spec.out_hidden, **bf)
        n_pages = N // PAGE + max_items
        self.kv = torch.zeros(1, n_pages * PAGE, 2, nh, 128, **bf)
        self.kv_tmap = ops.encode_kv_tmaps(self.kv)[0]
        self.cs = torch.zeros(N, hd, dtype=torch.float32, device=dev)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        self._acts: dict = {}
        self._grids: dict = {}
        self.encodes = 0

    # ------------------------------------------------------------------
    def _mat(self, w, k_pad=None):
        w = w.float()
        if k_pad and k_pad != w.shape[1]:
            w = torch.cat([w, w.new_zeros(w.shape[0], k_pad - w.shape[1])], dim=1)
        return TcWeight.from_master(w, KIND_BF16, self.device)

    def _vec(self, v):
        return None if v is None else v.float().to(self.device).contiguous()

    def nbytes(self) -> int:
        w = (self.mfc1.nbytes if self.mfc1 else 0) + self.mfc2.nbytes + sum(b[k].nbytes for b in self.blocks for k in ("qkv", "proj", "fc1", "fc2"))
        s = sum(t.numel() * t.element_size() for t in (self.x, self.h, self.y, self.qkv, self.q, self.attn, self.f, self.a,
                                                       self.out, self.o_raw, self.kv, self.cs))
        return w + s

    def _act(self, name: str, t: torch.Tensor, rows: int) -> ActBuffer:
        tn = ops.pick_tn(rows)
        key = (name, tn)
        if key not in self._acts:
            self._acts[key] = ActBuffer(KIND_BF16, t.shape[0], t.shape[1], tn, t, ops.encode_tmap(t, tn))    # row pitch may exceed K (views)
        return self._acts[key]

    def _linear(self, w: TcWeight, name: str, src: torch.Tensor, dst: torch.Tensor, rows: int):
        ops.tc_linear(w, self._act(name, src, rows), dst[:, :w.N] if dst.shape[1] != w.N else dst, rows=rows, status=self.status)

    def _add_norm(self, y, ybias, norm, out, rows, init=False):
        native.call("cuteafd_vision_add_norm", ptr(self.x), ptr(y), y.stride(0) if y is not None else 0, ptr(ybias), ptr(norm[0]) if norm else None,
                    ptr(norm[1]) if norm else None, ptr(out), rows, self.spec.hidden, self.spec.eps, 1 if init else 0, native.stream())

    def _bias_act(self, y, bias, out, rows, n_out, act):
        native.call("cuteafd_vision_bias_act", ptr(y), y.stride(0), ptr(bias), ptr(out), out.stride(0), rows, n_out, ACTS[act], native.stream())

    def _first_norm(self):
        return self.blocks[0]["norm1"] if self.blocks else self.merger_norm

    def _finish(self, counts: list[int]) -> list[torch.Tensor]:
        """Blocks + merger over the rows a front end left in `x` (fp32 residual) and `h` (first norm applied); one sequence per item."""
        spec, dev = self.spec, self.device
        H, nh, hd, I, g = spec.hidden, spec.n_heads, spec.head_dim, spec.intermediate, self.group
        N = sum(counts)
        max_pages = max(-(-c // PAGE) for c in counts)
        page_table = torch.zeros(len(counts), max_pages, dtype=torch.int32)
        slots, page = [], 0
        for i, c in enumerate(counts):
            np_ = -(-c // PAGE)
            page_table[i, :np_] = torch.arange(page, page + np_, dtype=torch.int32)
            slots.append(page * PAGE + torch.arange(c, dtype=torch.int32))
            page += np_
        slot = torch.cat(slots).to(dev)
        lens = torch.tensor(counts, dtype=torch.int32)
        q_start = (torch.cumsum(lens, 0) - lens).to(torch.int32).to(dev)
        lens_d, page_table = lens.to(dev), page_table.to(dev)
        for li, b in enumerate(self.blocks):
            self._linear(b["qkv"], "h", self.h, self.qkv, N)
            native.call("cuteafd_vision_qkv_rope_store", ptr(self.qkv), ptr(b["qkv_b"]), ptr(self.cs), ptr(b["q_norm"]), ptr(b["k_norm"]), ptr(self.q),
                        ptr(self.kv), ptr(slot), N, nh, hd, spec.eps, ptr(self.status), native.stream())
            native.call("cuteafd_gqa_prefill_attention", ptr(self.q), ptr(self.kv_tmap), ptr(page_table), ptr(lens_d), ptr(q_start), ptr(lens_d), None,
                        ptr(self.attn), N, len(counts), max(counts), nh * 128, nh, nh, max_pages, -1, hd ** -0.5, ptr(self.status), native.stream())
            self._linear(b["proj"], "attn", self.attn, self.y, N)
            self._add_norm(self.y, b["proj_b"], b["norm2"], self.h, N)
            self._linear(b["fc1"], "h", self.h, self.f, N)
            self._bias_act(self.f, b["fc1_b"], self.a, N, I, spec.mlp)
            self._linear(b["fc2"], "a", self.a[:, :I], self.y, N)
            nxt = self.blocks[li + 1]["norm1"] if li + 1 < len(self.blocks) else self.merger_norm
            self._add_norm(self.y, b["fc2_b"], nxt, self.h, N)
        Nm, M = N // g, g * H
        if self.mfc1 is not None:
            self._linear(self.mfc1, "hm", self.h.view(-1, M), self.f, Nm)
            self._bias_act(self.f, self.mfc1_b, self.a, Nm, M, "gelu")
            self._linear(self.mfc2, "am", self.a[:, :M], self.o_raw, Nm)
        else:
            self._linear(self.mfc2, "hm", self.h.view(-1, M), self.o_raw, Nm)
        self._bias_act(self.o_raw, self.mfc2_b, self.out, Nm, spec.out_hidden, "none")
        word = int(self.status[0])
        if word:
            self.status.zero_()
            raise RuntimeError(f"encoder tower: device status {native.decode_status(word)}")
        self.encodes += 1
        outs, o = [], 0
        for c in counts:
            outs.append(self.out[o:o + c // g].clone())
            o += c // g
        return outs



class VisionTower(EncoderTower):
    def __init__(self, spec: VisionSpec, masters: dict, device, max_patches: int = 16384, max_images: int = 16):
        super().__init__(spec, masters, device, max_patches, max_images, spec.merge ** 2)
        self.Kp = _pad8(spec.patch_dim)
        self.patch_w, self.patch_b = self._mat(masters["patch_w"], self.Kp), self._vec(masters["patch_b"])
        self.pos_embed = masters.get("pos_embed")
        self.lut = normalisation_lut(spec).to(self.device).contiguous()
        self.patches = torch.zeros(self.max_patches, self.Kp, dtype=torch.bfloat16, device=self.device)

    def nbytes(self) -> int:
        return super().nbytes() + self.patch_w.nbytes + self.patches.numel() * 2

    @torch.no_grad()
    def encode(self, images: list[torch.Tensor]) -> list[torch.Tensor]:
        """`images`: resized uint8 [gh * P, gw * P, 3] tensors (`load_image`).  Returns one bf16 [tokens, out_hidden] tensor per image."""
        spec = self.spec
        P, m, H, nh, hd, I = spec.patch, spec.merge, spec.hidden, spec.n_heads, spec.head_dim, spec.intermediate
        if not images:
            return []
        if len(images) > self.max_images:
            raise ValueError(f"vision tower: {len(images)} images in one call (limit {self.max_images})")
        grids = [(im.shape[0] // P, im.shape[1] // P) for im in images]
        counts = [gh * gw for gh, gw in grids]
        N = sum(counts)
        if N > self.max_patches:
            raise ValueError(f"vision tower: {N} patches in one call (limit {self.max_patches})")
        cs_rows, pos_rows = [], []
        off = 0
        for im, (gh, gw), c in zip(images, grids, counts):
            if im.dtype != torch.uint8 or im.shape[0] % (P * m) or im.shape[1] % (P * m) or im.shape[2] != 3:
                raise ValueError("vision tower: images are uint8 [gh * P, gw * P, 3] with whole merge groups")
            rgb = im.contiguous().to(self.device)
            native.call("cuteafd_vision_rgb_patches", ptr(rgb), ptr(self.lut), ptr(self.patches[off:]), gh, gw, P, m, self.Kp, native.stream())
            if (gh, gw) not in self._grids:          # rotary angles and resampled position rows depend on the grid only
                if len(self._grids) >= 64:
                    self._grids.clear()
                self._grids[(gh, gw)] = (rope_table(gh, gw, spec).to(self.device),
                                         position_rows(self.pos_embed.float(), gh, gw, spec).to(self.device) if self.pos_embed is not None else None)
            cs_rows.append(self._grids[(gh, gw)][0])
            if self.pos_embed is not None:
                pos_rows.append(self._grids[(gh, gw)][1])
            off += c
        self.cs[:N].copy_(torch.cat(cs_rows))
        self._linear(self.patch_w, "patches", self.patches, self.y, N)
        if pos_rows:
            self.x[:N].copy_(torch.cat(pos_rows))
        self._add_norm(self.y, self.patch_b, self._first_norm(), self.h, N, init=not pos_rows)
        return self._finish(counts)
