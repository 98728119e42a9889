"""Tensor-level wrappers over the native sm_100a kernels.

Each function validates shapes/dtypes, then launches on the current CUDA stream (so callers can capture
whole steps into CUDA graphs).  Nothing here falls back to PyTorch math on a GPU: if the native library is
missing the call raises.  The fp32 oracles live in `cuteafd_b200.ref`.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import native
from .native import call, ptr, stream

KIND_BF16, KIND_NVFP4, KIND_MXFP4, KIND_FP8B = 0, 1, 2, 3      # FP8B: E4M3 with fp32 scales per 128 x 128 (weights) / 1 x 128 (activations)
KIND_W4A8 = 4      # MXFP4 weights x FP8 E4M3 activations, UE8M0 scales per 32 on both (tcgen05 kind::mxf8f6f4)
# MXFP4 expert weights run with MXFP4 activations (W4A4) unless CUTEAFD_MXFP4_ACT=fp8 selects FP8 activations (W4A8, the
# reference's default expert arithmetic; also reachable per model as the "mxfp4_w4a8" format name)
import os as _os
MXFP4_ACT = _os.environ.get("CUTEAFD_MXFP4_ACT", "fp4")
KIND_BY_NAME = {"bf16": KIND_BF16, "nvfp4": KIND_NVFP4, "mxfp4": KIND_W4A8 if MXFP4_ACT == "fp8" else KIND_MXFP4, "mxfp4_w4a4": KIND_MXFP4,
                "mxfp4_w4a8": KIND_W4A8, "fp8_block128": KIND_FP8B}
FP4_KINDS = (KIND_NVFP4, KIND_MXFP4)
# activation formats the norm kernels (add_rmsnorm, moe_combine with the next layer's norm) can write in the same launch, and the
# code the native side knows them by
FUSED_QUANT_KINDS = (KIND_NVFP4, KIND_MXFP4, KIND_FP8B)
_QKIND = {KIND_NVFP4: 1, KIND_MXFP4: 2, KIND_FP8B: 3}
EPI_BF16, EPI_BF16_RESIDUAL, EPI_F32 = 0, 1, 3
SCORING = {"sigmoid": 0, "softmax": 1, "sqrtsoftplus": 2}


def _chk(t: torch.Tensor, dtype, name: str):
    if t.dtype != dtype or not t.is_cuda or not t.is_contiguous():
        raise ValueError(f"{name}: expected contiguous CUDA {dtype}, got {t.dtype} cuda={t.is_cuda} contiguous={t.is_contiguous()}")


# ------------------------------------------------------------------ launch mode / tracing
def set_pdl(mask: int) -> None:
    """Programmatic dependent launch per kernel class (bit 0 glue kernels, bit 1 GEMMs, bit 2 attention; 0 = off, the
    default; CUTEAFD_PDL=<mask> sets it from the environment).  Graphs captured earlier keep their mode."""
    native.lib().cuteafd_set_pdl(int(mask))


_CLUSTER_CAP: dict = {}


def cluster_capacity(kind: int, tn: int, splits: int) -> int:
    """Clusters of `splits` CTAs of the cluster split-K GEMM that fit the device at once (cached per device)."""
    key = (torch.cuda.current_device(), kind, tn, splits)
    if key not in _CLUSTER_CAP:
        out = ctypes.c_int(0)
        call("cuteafd_tc_cluster_capacity", kind, tn, splits, ctypes.addressof(out))
        _CLUSTER_CAP[key] = out.value
    return _CLUSTER_CAP[key]


def fp8_cluster_capacity(tn: int, splits: int, K: int) -> int:
    """Clusters of `splits` CTAs of the FP8 block-scaled GEMM that fit the device at once for this K (cached per device)."""
    key = (torch.cuda.current_device(), "fp8", tn, splits, K)
    if key not in _CLUSTER_CAP:
        out = ctypes.c_int(0)
        call("cuteafd_fp8_cluster_capacity", tn, splits, K, ctypes.addressof(out))
        _CLUSTER_CAP[key] = out.value
    return _CLUSTER_CAP[key]


def tc_trace(buf: torch.Tensor | None, units: int = 0) -> None:
    """Per-unit device time stamps of later `tc_linear` launches: int64 [grid, units, 8] (None = off).  `units < 0`: the cluster
    split-K kernel records instead - its launches with N == -units write eight global-timer stamps per CTA into int64 [grid, 8]
    (entry, -, released by the previous kernel, first stage landed, last MMA committed, accumulator complete, cluster barrier
    passed, epilogue done); usable inside a replayed step graph, where the last such launch of the step survives."""
    call("cuteafd_tc_trace", ptr(buf), units)


# ------------------------------------------------------------------ TMA descriptors
def encode_tmap(t: torch.Tensor, box_rows: int, unpack4: bool = False) -> torch.Tensor:
    """Descriptor array (uint8 [G, 128], on t's device) for a K-major operand [G, rows, K] or [rows, K].
    bf16 tensors describe K elements; uint8 tensors describe K bytes (packed fp4 / fp8).  `unpack4`: a uint8 tensor of packed
    4-bit elements whose tiles TMA expands into 8-bit containers in shared memory (the weight operand of the W4A8 kind)."""
    if t.dim() == 2:
        t = t.unsqueeze(0)
    G, rows, kdim = t.shape
    eb = {torch.bfloat16: 2, torch.uint8: 1}[t.dtype]
    if t.stride(2) != 1:
        raise ValueError("operand must be K-contiguous")
    host = torch.zeros(G, 128, dtype=torch.uint8)
    for g in range(G):
        if unpack4:
            call("cuteafd_tmap_encode_kmajor", host[g].data_ptr(), t[g].data_ptr(), 0, kdim * 2, rows, 1, t.stride(1), 0, box_rows)
        else:
            call("cuteafd_tmap_encode_kmajor", host[g].data_ptr(), t[g].data_ptr(), eb, kdim, rows, 1,
                 t.stride(1) * eb, 0, box_rows)
    return host.to(t.device)


def swizzle_sf(sf: torch.Tensor, per_stage: int = 4) -> torch.Tensor:
    """[rows, n_sf] uint8 block scales -> flat 128x4-atom layout (any device); see ref.quant.swizzle_sf_128x4.
    The scale count per row is zero-padded to whole pipeline stages (`per_stage` scales: 16 NVFP4, 8 MXFP4)."""
    rows, n = sf.shape
    R, Cc = -(-rows // 128) * 128, -(-n // per_stage) * per_stage
    pad = sf.new_zeros(R, Cc)
    pad[:rows, :n] = sf
    return pad.reshape(R // 128, 4, 32, Cc // 4, 4).permute(0, 3, 2, 1, 4).contiguous().reshape(-1)


@dataclass
class TcWeight:
    """Weight set for `tc_linear`: G matrices [N, K] (G > 1 = experts), K-major as checkpoints ship them."""
    kind: int
    G: int
    N: int
    K: int
    data: torch.Tensor              # bf16 [G, N, K] | uint8 [G, N, K/2]
    tmap: torch.Tensor              # uint8 [G, 128]
    sf: torch.Tensor | None = None  # uint8 [G, swizzled bytes]
    sf_ptrs: torch.Tensor | None = None
    alpha: torch.Tensor | None = None   # fp32 [G]: weight global scale x activation global scale
    inv_act_gs: torch.Tensor | None = None  # fp32 [1]: 1 / activation global scale (NVFP4)

    @property
    def nbytes(self) -> int:
        return self.data.numel() * self.data.element_size() + (self.sf.numel() if self.sf is not None else 0)

    @staticmethod
    def from_master(w: torch.Tensor, kind: str | int, device, act_gs: float = 1.0 / 64) -> "TcWeight":
        """Quantise fp32 masters [G, N, K] (or [N, K]) with the CPU oracle and upload (tests, small models)."""
        from ..ref import quant
        kind = KIND_BY_NAME[kind] if isinstance(kind, str) else kind
        if w.dim() == 2:
            w = w.unsqueeze(0)
        G, N, K = w.shape
        if kind == KIND_BF16:
            data = w.to(torch.bfloat16).to(device).contiguous()
            return TcWeight(kind, G, N, K, data, encode_tmap(data, 128))
        if kind == KIND_FP8B:
            qs = [quant.fp8_block_quantize(w[g]) for g in range(G)]
            data = torch.stack([q for q, _ in qs]).to(device).contiguous()
            return TcWeight(kind, G, N, K, data, encode_tmap(data, 128), torch.stack([s for _, s in qs]).to(device).contiguous())
        packs, sfs, alphas = [], [], []
        for g in range(G):
            if kind == KIND_NVFP4:
                p, s, gs = quant.nvfp4_quantize(w[g])
                alphas.append(float(gs) * act_gs)
            else:
                p, s = quant.mxfp4_quantize(w[g])
                alphas.append(1.0)
            packs.append(p)
            sfs.append(swizzle_sf(s, SF_PER_STAGE[kind]))
        data = torch.stack(packs).to(device).contiguous()
        sf = torch.stack(sfs).to(device).contiguous()
        return TcWeight._finish(kind, G, N, K, data, sf, torch.tensor(alphas, dtype=torch.float32, device=device), act_gs)

    @staticmethod
    def fuse_rows_fp8(a: "TcWeight", b: "TcWeight") -> "TcWeight":
        """One FP8 block-scaled weight [N_a + N_b, K] out of two with the same K (gate and up projections read the same operand:
        one GEMM instead of two).  `a` and `b` become views into the fused storage, so nothing is held twice."""
        if a.kind != KIND_FP8B or b.kind != KIND_FP8B or a.G != 1 or b.G != 1 or a.K != b.K or a.N % 128 or b.N % 128:
            raise ValueError("fuse_rows_fp8: two dense FP8 weights with the same K and row counts that are multiples of 128")
        data = torch.cat([a.data, b.data], 1).contiguous()
        sf = torch.cat([a.sf, b.sf], 1).contiguous()
        fused = TcWeight(KIND_FP8B, 1, a.N + b.N, a.K, data, encode_tmap(data, 128), sf)
        na, ra = a.N, a.N // 128
        a.data, a.sf = data[:, :na], sf[:, :ra]
        b.data, b.sf = data[:, na:], sf[:, ra:]
        a.tmap, b.tmap = encode_tmap(a.data, 128), encode_tmap(b.data, 128)
        return fused

    @staticmethod
    def random(G: int, N: int, K: int, kind: str | int, device, std: float = 0.02, act_gs: float = 1.0 / 64,
               seed: int = 0, groups: tuple | None = None) -> "TcWeight":
        """Random-init weights generated directly in the storage format on the device (large synthetic models).
        `groups=(lo, hi)` keeps only groups [lo, hi) of the G generated ones, so an expert-parallel rank holds exactly
        the experts a single-GPU model of the same seed has at those indices."""
        kind = KIND_BY_NAME[kind] if isinstance(kind, str) else kind
        gen = torch.Generator(device=device).manual_seed(seed)
        lo, hi = groups if groups is not None else (0, G)
        cut = (lambda t: t[lo:hi].clone()) if (lo, hi) != (0, G) else (lambda t: t)
        if kind == KIND_BF16:
            data = cut(torch.empty(G, N, K, dtype=torch.bfloat16, device=device).normal_(0, std, generator=gen))
            return TcWeight(kind, hi - lo, N, K, data, encode_tmap(data, 128))
        if kind == KIND_FP8B:    # random sign and magnitude codes below the NaN pattern; |w| ~ std with one common block scale
            mag = torch.randint(0, 0x78, (G, N, K), dtype=torch.uint8, device=device, generator=gen)
            sign = torch.randint(0, 2, (G, N, K), dtype=torch.uint8, device=device, generator=gen) << 7
            data = cut(mag | sign)
            sw = torch.full((hi - lo, -(-N // 128), -(-K // 128)), std / 60.0, dtype=torch.float32, device=device)
            return TcWeight(kind, hi - lo, N, K, data, encode_tmap(data, 128), sw)
        data = cut(torch.randint(0, 256, (G, N, K // 2), dtype=torch.uint8, device=device, generator=gen))
        vec = 16 if kind == KIND_NVFP4 else 32
        kstage = 128 if kind == KIND_W4A8 else 256
        nsf = (-(-N // 128) * 128) * (-(-K // kstage) * (kstage // vec))
        if kind == KIND_NVFP4:   # E4M3 scales in [0.5, 1.875]
            sf = cut(torch.randint(0x30, 0x40, (G, nsf), dtype=torch.uint8, device=device, generator=gen))
            alpha = torch.full((hi - lo,), std / 3.4 * act_gs, dtype=torch.float32, device=device)
        else:                    # UE8M0 scales 2^-7 .. 2^-6 -> |w| ~ std
            sf = cut(torch.randint(120, 122, (G, nsf), dtype=torch.uint8, device=device, generator=gen))
            alpha = torch.full((hi - lo,), std / 0.034, dtype=torch.float32, device=device)
        return TcWeight._finish(kind, hi - lo, N, K, data, sf, alpha, act_gs)

    @staticmethod
    def _finish(kind, G, N, K, data, sf, alpha, act_gs):
        sf_ptrs = torch.tensor([sf[g].data_ptr() for g in range(G)], dtype=torch.int64, device=data.device)
        inv = torch.tensor([1.0 / act_gs], dtype=torch.float32, device=data.device)
        return TcWeight(kind, G, N, K, data, encode_tmap(data, 128, unpack4=kind == KIND_W4A8), sf, sf_ptrs, alpha, inv)

    def dequantize(self) -> torch.Tensor:
        """fp32 [G, N, K] on CPU, without the activation scale folded into alpha (test helper)."""
        from ..ref import quant
        if self.kind == KIND_BF16:
            return self.data.float().cpu()
        if self.kind == KIND_FP8B:
            return torch.stack([quant.fp8_block_dequantize(self.data[g].cpu(), self.sf[g].cpu()) for g in range(self.G)])
        vec = 16 if self.kind == KIND_NVFP4 else 32
        kstage = 128 if self.kind == KIND_W4A8 else 256
        out = []
        for g in range(self.G):
            s = quant.unswizzle_sf_128x4(self.sf[g].cpu(), self.N, -(-self.K // kstage) * (kstage // vec))[:, :self.K // vec]
            if self.kind == KIND_NVFP4:
                gs = float(self.alpha[g]) * float(self.inv_act_gs[0])
                out.append(quant.nvfp4_dequantize(self.data[g].cpu(), s, gs))
            else:
                out.append(quant.mxfp4_dequantize(self.data[g].cpu(), s) * float(self.alpha[g]))
        return torch.stack(out)


@dataclass
class ActBuffer:
    """Activation operand for `tc_linear`: bf16 rows, or fp4 rows + row-major block scales, with its TMA
    descriptor for a token tile of `tn` rows."""
    kind: int
    rows: int
    K: int
    tn: int
    data: torch.Tensor
    tmap: torch.Tensor
    sf: torch.Tensor | None = None

    @staticmethod
    def alloc(kind: int, rows: int, K: int, tn: int, device) -> "ActBuffer":
        if kind == KIND_BF16:
            data = torch.zeros(rows, K, dtype=torch.bfloat16, device=device)
            return ActBuffer(kind, rows, K, tn, data, encode_tmap(data, tn))
        if kind == KIND_FP8B:    # E4M3 bytes + one fp32 scale per row and 128 channels
            data = torch.zeros(rows, K, dtype=torch.uint8, device=device)
            return ActBuffer(kind, rows, K, tn, data, encode_tmap(data, tn), torch.zeros(rows, -(-K // 128), dtype=torch.float32, device=device))
        if kind == KIND_W4A8:    # E4M3 bytes + one UE8M0 scale per row and 32 channels (scale rows padded to whole 128-channel stages)
            data = torch.zeros(rows, K, dtype=torch.uint8, device=device)
            return ActBuffer(kind, rows, K, tn, data, encode_tmap(data, tn), torch.zeros(rows, -(-K // 128) * 4, dtype=torch.uint8, device=device))
        vec = 16 if kind == KIND_NVFP4 else 32
        data = torch.zeros(rows, K // 2, dtype=torch.uint8, device=device)
        sf = torch.zeros(rows, -(-K // 256) * (256 // vec), dtype=torch.uint8, device=device)   # padded to whole stages
        return ActBuffer(kind, rows, K, tn, data, encode_tmap(data, tn), sf)

    @staticmethod
    def wrap_bf16(x: torch.Tensor, tn: int) -> "ActBuffer":
        _chk(x, torch.bfloat16, "x")
        return ActBuffer(KIND_BF16, x.shape[0], x.shape[1], tn, x, encode_tmap(x, tn))


SF_PER_STAGE = {KIND_NVFP4: 16, KIND_MXFP4: 8, KIND_W4A8: 4}        # weight block scales per row and pipeline stage


def pick_tn(rows: int, swiglu: bool = False) -> int:
    for tn in (16, 32, 64, 128):
        if rows <= tn:
            return tn
    return 128 if swiglu else 256


_SPLITK_WS: dict = {}


def _splitk_scratch(device, n_float: int, n_cnt: int):
    key = str(device)
    ws, cnt = _SPLITK_WS.get(key, (None, None))
    if ws is None or ws.numel() < n_float:
        ws = torch.empty(max(n_float, 1 << 22), dtype=torch.float32, device=device)
    if cnt is None or cnt.numel() < n_cnt:
        cnt = torch.zeros(max(n_cnt, 1 << 16), dtype=torch.int32, device=device)
    _SPLITK_WS[key] = (ws, cnt)
    return ws, cnt


def tc_linear(w: TcWeight, x: ActBuffer, y: torch.Tensor | None, *, rows: int | None = None, w_up: TcWeight | None = None,
              residual: torch.Tensor | None = None, tiles: torch.Tensor | None = None, n_tiles: torch.Tensor | None = None,
              max_tiles: int = 0, splits: int = 1, status: torch.Tensor | None = None, max_ctas: int = 0,
              quant_out: ActBuffer | None = None, inv_gs_out: torch.Tensor | None = None, peer: dict | None = None) -> torch.Tensor | None:
    """y[rows, N] = x[rows, K] @ w[g]^T (per tile's expert g when `tiles` is given).  `w_up` switches on the fused
    SwiGLU epilogue (y = silu(x w^T) * (x w_up^T)).  y is bf16 (optionally + residual) or fp32.  `quant_out` (an FP4
    activation buffer of the operands' kind, K = N) also receives the output quantised for the GEMM that follows
    (`inv_gs_out`: that GEMM's activation scale, NVFP4); y may then be None.
    `peer` fuses the hand-off to other GPUs into the epilogue: {"y": [device addresses of 1-2 peers' bf16 buffers], "ld": row
    pitch in elements, "row_map": int32 tensor or None (row r lands in row_map[r]), "flags": [peer flag addresses],
    "ctl": control block tensor, "done": zeroed uint32 counter tensor}; the flags are released with the step number
    once the whole output has been stored (y may be None when only the peers need the result)."""
    rows = x.rows if rows is None else rows
    if w.kind != x.kind or w.K != x.K:
        raise ValueError("tc_linear: operand kinds / K differ")
    if y is None:
        epi = EPI_BF16
    else:
        epi = EPI_F32 if y.dtype == torch.float32 else (EPI_BF16_RESIDUAL if residual is not None else EPI_BF16)
    if w.kind == KIND_FP8B:
        if w_up is not None or tiles is not None or quant_out is not None or w.G != 1:
            raise ValueError("tc_linear: the FP8 block-scaled kernel is dense only (no SwiGLU / grouped / FP4 output)")
        if splits < 1 or (splits > 1 and x.tn > 64) or splits > (8 if x.tn == 16 else 4):
            splits = 1
        call("cuteafd_fp8_linear", x.tn, ptr(w.tmap), ptr(x.tmap), ptr(w.sf), ptr(x.sf), ptr(y), ptr(residual), y.stride(0), rows, w.N, w.K,
             epi, splits, ptr(status), stream())
        return y
    ws = cnt = None
    if splits > 1:
        n_items = -(-rows // x.tn)
        ws, cnt = _splitk_scratch(x.data.device, splits * rows * w.N, n_items * (-(-w.N // 128)) * 4)
    extra = None
    if quant_out is not None:
        if quant_out.kind != w.kind or quant_out.K != w.N:
            raise ValueError("tc_linear: quant_out must be an FP4 buffer of the operands' kind with K = N")
        extra = native.TcExtra()
        extra.q_out, extra.sf_out, extra.ldsf_out, extra.inv_gs_out = ptr(quant_out.data), ptr(quant_out.sf), quant_out.sf.shape[1], ptr(inv_gs_out)
    if peer is not None:
        ys, fl = list(peer["y"]), list(peer["flags"])
        extra = extra or native.TcExtra()
        extra.n_peer, extra.peer_ld = len(ys), peer["ld"]
        for i in range(len(ys)):
            extra.peer_y[i], extra.peer_flag[i] = ys[i], fl[i]
        extra.peer_row_map, extra.peer_ctl, extra.peer_done = ptr(peer.get("row_map")), ptr(peer["ctl"]), ptr(peer["done"])
    call("cuteafd_tc_linear", w.kind, 1 if w_up is not None else 0, x.tn, ptr(w.tmap), ptr(w_up.tmap) if w_up else None,
         ptr(x.tmap), ptr(w.sf_ptrs), ptr(w_up.sf_ptrs) if w_up else None, ptr(x.sf), x.sf.shape[1] if x.sf is not None else 0,
         ptr(w.alpha), ptr(w_up.alpha) if w_up else None, ptr(tiles), ptr(n_tiles), max_tiles, ptr(y), ptr(residual),
         y.stride(0) if y is not None else 0, rows, w.N, w.K, epi, splits, ptr(ws), ptr(cnt), ptr(status), max_ctas,
         ctypes.byref(extra) if extra is not None else None, stream())
    return y


# ------------------------------------------------------------------ EXL3 (trellis) weights
@dataclass
class Exl3Weight:
    """One EXL3 linear as shipped: trellis uint16 [K/16, N/16, 16*bits], suh fp16 [K], svh fp16 [N] (y = x @ W)."""
    trellis: torch.Tensor
    suh: torch.Tensor
    svh: torch.Tensor

    @property
    def K(self) -> int:
        return self.trellis.shape[0] * 16

    @property
    def N(self) -> int:
        return self.trellis.shape[1] * 16

    @property
    def bits(self) -> int:
        return self.trellis.shape[2] // 16


_EXL3_WS: dict = {}


def exl3_linear(w: Exl3Weight, x: torch.Tensor, y: torch.Tensor, *, rows: int | None = None, residual: torch.Tensor | None = None,
                k_splits: int = 0) -> torch.Tensor:
    """y[rows, N] = x[rows, K] @ W(+ residual) with W decoded from the trellis inside the GEMM (decode-sized batches)."""
    _chk(x, torch.bfloat16, "x")
    rows = x.shape[0] if rows is None else rows
    K, N = w.K, w.N
    if not k_splits:      # enough warps to fill the machine: N/16 strips x splits ~ 4 per SM sub-partition
        k_splits = max(1, min(K // 256, -(-148 * 16 // (N // 16))))
    pad = -(-rows // 16) * 16
    key = str(x.device)
    xr, part = _EXL3_WS.get(key, (None, None))
    if xr is None or xr.numel() < pad * K:
        xr = torch.empty(max(pad * K, 1 << 20), dtype=torch.float16, device=x.device)
    if part is None or part.numel() < k_splits * pad * N:
        part = torch.empty(max(k_splits * pad * N, 1 << 22), dtype=torch.float32, device=x.device)
    _EXL3_WS[key] = (xr, part)
    call("cuteafd_exl3_linear", ptr(x), ptr(w.trellis), ptr(w.suh), ptr(w.svh), ptr(residual), ptr(y), ptr(xr), ptr(part), rows, K, N, w.bits,
         k_splits, y.stride(0), stream())
    return y


# ------------------------------------------------------------------ elementwise
def embed_gather(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, status: torch.Tensor | None = None):
    _chk(tokens, torch.int32, "tokens"); _chk(table, torch.bfloat16, "table")
    call("cuteafd_embed_gather", ptr(tokens), ptr(table), ptr(out), tokens.numel(), table.shape[1], table.shape[0], ptr(status), stream())
    return out


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, w: torch.Tensor, y: torch.Tensor | None, eps: float, rows: int | None = None,
                quant: "ActBuffer | None" = None, inv_gs: torch.Tensor | None = None):
    """x += delta (if given, in place); y = rmsnorm(x) * w.  With `quant` (an FP4 activation buffer) the normalised
    rows are also written quantised in the same launch (y may then be None)."""
    _chk(x, torch.bfloat16, "x"); _chk(w, torch.float32, "w")
    n = x.shape[0] if rows is None else rows
    if quant is not None and quant.kind in FUSED_QUANT_KINDS:
        call("cuteafd_add_rmsnorm_quant", ptr(x), ptr(delta), ptr(w), ptr(y), n, x.shape[1], eps, ptr(quant.data), ptr(quant.sf),
             quant.sf.shape[1], ptr(inv_gs), _QKIND[quant.kind], stream())
    else:
        call("cuteafd_add_rmsnorm", ptr(x), ptr(delta), ptr(w), ptr(y), n, x.shape[1], eps, stream())
    return y


def qk_norm_rope_kvwrite(qkv, positions, slot_map, q_norm, k_norm, kv_cache, T, Hq, Hkv, D, theta, interleaved, eps, status=None):
    n_slots = kv_cache.shape[0]
    call("cuteafd_qk_norm_rope_kvwrite", ptr(qkv), ptr(positions), ptr(slot_map), ptr(q_norm), ptr(k_norm), ptr(kv_cache),
         T, Hq, Hkv, D, theta, 1 if interleaved else 0, eps, n_slots, ptr(status), stream())


def quant_fp4_rows(x: torch.Tensor, out: ActBuffer, *, src_rows: torch.Tensor | None = None, n_rows_dev: torch.Tensor | None = None,
                   rows: int | None = None, inv_gs: torch.Tensor | None = None):
    _chk(x, torch.bfloat16, "x")
    if out.kind == KIND_W4A8:
        call("cuteafd_act_quant_fp8_ue8m0", ptr(x), ptr(src_rows), ptr(n_rows_dev), ptr(out.data), ptr(out.sf), out.rows if rows is None else rows,
             out.K, x.stride(0), out.sf.shape[1], stream())
        return out
    if out.kind == KIND_FP8B:
        if src_rows is not None or n_rows_dev is not None:
            raise ValueError("FP8 activation quantisation has no gather form")
        call("cuteafd_act_quant_fp8_block128", ptr(x), ptr(out.data), ptr(out.sf), out.rows if rows is None else rows, out.K, x.stride(0), stream())
        return out
    call("cuteafd_quant_fp4_rows", 1 if out.kind == KIND_MXFP4 else 0, ptr(x), ptr(src_rows), ptr(n_rows_dev), ptr(out.data),
         ptr(out.sf), out.rows if rows is None else rows, out.K, x.stride(0), out.sf.shape[1], ptr(inv_gs), stream())
    return out


def gather_rows(x, src_rows, n_rows_dev, out, rows):
    call("cuteafd_gather_rows", ptr(x), ptr(src_rows), ptr(n_rows_dev), ptr(out), rows, x.shape[1], stream())
    return out


def kv_pages_copy(kv, pairs, pool, to_pool: bool):
    """Moves KV pages between the device store `kv` [layers, slots, ...] and a slab pool [slabs, layers, page...] (device
    memory or pinned host memory) in one launch.  `pairs` is an int32 device tensor [n, 2] of (device page, slab)."""
    L = kv.shape[0]
    page_bytes = pool[0, 0].numel() * pool.element_size()
    assert pool.shape[1] == L and kv.is_contiguous() and pool.is_contiguous() and pairs.dtype == torch.int32 and pairs.is_cuda
    call("cuteafd_kv_pages_copy", ptr(kv), kv.stride(0) * kv.element_size(), L, page_bytes, ptr(pairs), pairs.shape[0], pool.data_ptr(),
         pool.stride(0) * pool.element_size(), 0 if to_pool else 1, stream())


def l2_prefetch(t):
    """Hints the memory system to pull a tensor (e.g. the next layer's weights) into L2; returns immediately."""
    call("cuteafd_l2_prefetch", ptr(t), t.numel() * t.element_size(), stream())


def act_quant_fp8_ue8m0(x, q, sf):
    call("cuteafd_act_quant_fp8_ue8m0", ptr(x), None, None, ptr(q), ptr(sf), x.shape[0], x.shape[1], x.stride(0), sf.shape[1], stream())


def silu_mul(g, u, out, limit: float = 0.0):
    call("cuteafd_silu_mul", ptr(g), ptr(u), ptr(out), g.numel(), limit, stream())
    return out


def router_logits(x, w: "TcWeight", logits, T: int):
    """fp32 router logits of `T` token rows (bf16 `x` [rows, H]) against a bf16 router weight [E, H]: the SIMT kernel for
    decode-sized batches (the tensor-core GEMM is launch- and cluster-overhead bound at this size)."""
    assert w.kind == KIND_BF16 and w.G == 1 and x.dtype == torch.bfloat16 and x.stride(0) == w.K and logits.stride(0) == w.N
    call("cuteafd_router_logits", ptr(x), ptr(w.data), ptr(logits), T, w.N, w.K, stream())
    return logits


# ------------------------------------------------------------------ MoE control
def router_select(logits, bias, idx, wts, T, k, scoring, normalize, route_scale, n_group=1, topk_group=1):
    _chk(logits, torch.float32, "logits")
    call("cuteafd_router_select", ptr(logits), ptr(bias), ptr(idx), ptr(wts), T, logits.shape[1], k, SCORING[scoring],
         1 if normalize else 0, route_scale, n_group, topk_group, stream())


_TICKETS: dict = {}


def router_select_pack(logits, bias, idx, wts, T, k, scoring, normalize, route_scale, n_group, topk_group,
                       src_token, slot_row, counts, offsets, tiles, n_tiles, n_rows, e_lo, e_hi, tn, max_tiles, src_route=None):
    """`router_select` followed by `route_pack` in one launch (the select block that finishes last packs)."""
    _chk(logits, torch.float32, "logits")
    dev = logits.device
    if dev not in _TICKETS:
        _TICKETS[dev] = torch.zeros(1, dtype=torch.int32, device=dev)
    call("cuteafd_router_select_pack", ptr(logits), ptr(bias), ptr(idx), ptr(wts), T, logits.shape[1], k, SCORING[scoring],
         1 if normalize else 0, route_scale, n_group, topk_group, ptr(src_token), ptr(slot_row), ptr(counts), ptr(offsets),
         ptr(tiles), ptr(n_tiles), ptr(n_rows), e_lo, e_hi, tn, max_tiles, ptr(src_route), ptr(_TICKETS[dev]), stream())


def router_fused(x, w: "TcWeight", logits, bias, idx, wts, T, k, scoring, normalize, route_scale, n_group=1, topk_group=1, pack: dict | None = None):
    """The whole router of a decode-sized step in one launch: fp32 logits of `T` bf16 rows against the bf16 router weight, top-k
    selection with gate weights, and - with `pack` (src_token, slot_row, counts, offsets, tiles, n_tiles, n_rows, e_lo, e_hi, tn,
    max_tiles, optional src_route) - the expert-order route packing and tile table."""
    assert w.kind == KIND_BF16 and w.G == 1 and x.dtype == torch.bfloat16 and x.stride(0) == w.K and logits.stride(0) == w.N
    dev = logits.device
    if dev not in _TICKETS:
        _TICKETS[dev] = torch.zeros(1, dtype=torch.int32, device=dev)
    pk = pack or {}
    g = lambda name: ptr(pk.get(name))
    call("cuteafd_router_fused", ptr(x), ptr(w.data), ptr(logits), ptr(bias), ptr(idx), ptr(wts), T, w.N, w.K, k, SCORING[scoring],
         1 if normalize else 0, route_scale, n_group, topk_group, g("src_token"), g("slot_row"), g("counts"), g("offsets"), g("tiles"),
         g("n_tiles"), g("n_rows"), pk.get("e_lo", 0), pk.get("e_hi", 0), pk.get("tn", 1), pk.get("max_tiles", 0), g("src_route"),
         ptr(_TICKETS[dev]), stream())


def route_pack(idx, src_token, slot_row, counts, offsets, tiles, n_tiles, n_rows, T, k, e_lo, e_hi, tn, max_tiles, src_route=None, *,
               wait=None, lane_T=None, t_cap: int = 0):
    """Packs the routes of `T` tokens into expert order.  `wait` (a `native.FlagWaitArg`) makes the kernel wait for the peers
    that deliver the routing table; `lane_T` (int32 device tensor, one count per lane) + `t_cap` describe a table of several
    senders laid out [lane][t_cap][k] (T = lanes * t_cap) whose rows beyond each lane's count are skipped."""
    call("cuteafd_route_pack", ptr(idx), ptr(src_token), ptr(slot_row), ptr(counts), ptr(offsets), ptr(tiles), ptr(n_tiles),
         ptr(n_rows), T, k, e_lo, e_hi, tn, max_tiles, ptr(src_route), ctypes.byref(wait) if wait is not None else None,
         ptr(lane_T), t_cap, stream())


def route_gather(src_q, src_sf, src_token, n_rows, dst: "ActBuffer", rows_cap: int, status=None):
    """dst row c = slab row src_token[c] (payload and block scales) for c < n_rows: token-major slab -> expert order."""
    row_bytes = src_q.shape[-1] * src_q.element_size()
    sf_bytes = src_sf.shape[-1] if src_sf is not None else 0
    call("cuteafd_route_gather", ptr(src_q), ptr(src_sf), ptr(src_token), ptr(n_rows), ptr(dst.data), ptr(dst.sf) if src_sf is not None else None,
         row_bytes, sf_bytes, sf_bytes, dst.sf.shape[1] if src_sf is not None else 0, src_q.numel() * src_q.element_size() // row_bytes,
         rows_cap, ptr(status), stream())
    return dst


def router_hash_select(logits, tid2eid, tokens, idx, wts, T, k, route_scale: float = 1.0, status=None):
    """Hash routing: experts of token row t are tid2eid[tokens[t]] ([vocab, k] int32); gate weights are the normalised
    sqrt-softplus scores of `logits` at those experts times `route_scale`."""
    _chk(logits, torch.float32, "logits"); _chk(tid2eid, torch.int32, "tid2eid"); _chk(tokens, torch.int32, "tokens")
    call("cuteafd_router_hash_select", ptr(logits), ptr(tid2eid), ptr(tokens), ptr(idx), ptr(wts), T, logits.shape[1], k, tid2eid.shape[0],
         route_scale, ptr(status), stream())


def moe_combine(y, slot_row, wts, shared, residual, out, T, k, *, norm_w=None, eps: float = 0.0, xn=None, quant=None, inv_gs=None, wait=None):
    """out = residual + shared + sum_slot w * y[slot_row].  With `norm_w` the same launch also applies the next
    layer's RMSNorm to `out`, written as bf16 (`xn`) and/or FP4 (`quant`, an activation buffer).  `wait` (a
    `native.FlagWaitArg`): the kernel first waits for the peers that deliver `y`."""
    w = ctypes.byref(wait) if wait is not None else None
    if norm_w is None:
        call("cuteafd_moe_combine", ptr(y), ptr(slot_row), ptr(wts), ptr(shared), ptr(residual), ptr(out), T, y.shape[1], k, w, stream())
        return out
    fp4 = quant is not None and quant.kind in FUSED_QUANT_KINDS
    call("cuteafd_moe_combine_norm", ptr(y), ptr(slot_row), ptr(wts), ptr(shared), ptr(residual), ptr(out), T, y.shape[1], k, ptr(norm_w),
         eps, ptr(xn), ptr(quant.data) if fp4 else None, ptr(quant.sf) if fp4 else None, quant.sf.shape[1] if fp4 else 0,
         ptr(inv_gs) if fp4 else None, _QKIND[quant.kind] if fp4 else 0, w, stream())
    return out


# ------------------------------------------------------------------ attention
def paged_attention(q, kv, page_table, kv_len, q_start, q_len, out, *, T, n_seq, max_q_len, q_stride, Hq, Hkv, D, n_splits=1,
                    part_o=None, part_ml=None, window=0, sink=None, scale=None):
    call("cuteafd_paged_attention", ptr(q), ptr(kv), ptr(page_table), ptr(kv_len), ptr(q_start), ptr(q_len), ptr(sink), ptr(out),
         ptr(part_o), ptr(part_ml), T, n_seq, max_q_len, q_stride, Hq, Hkv, D, page_table.shape[1], n_splits, window,
         float(scale if scale is not None else D ** -0.5), stream())
    return out


def encode_kv_tmaps(kv: torch.Tensor) -> torch.Tensor:
    """TMA descriptors (uint8 [layers, 128]) for a paged K/V store [layers, slots, 2, Hkv, 128] bf16."""
    _chk(kv, torch.bfloat16, "kv")
    L, slots, two, Hkv, D = kv.shape
    if D != 128 or two != 2:
        raise ValueError("tensor-core attention needs head_dim 128")
    host = torch.zeros(L, 128, dtype=torch.uint8)
    for l in range(L):
        call("cuteafd_tmap_encode_kv", host[l].data_ptr(), kv[l].data_ptr(), Hkv, slots)
    return host.to(kv.device)


def paged_attention_tc(q, kv_map, page_table, kv_len, q_start, q_len, out, *, T, n_seq, max_q_len, q_stride, Hq, Hkv,
                       n_splits=1, part_o=None, part_ml=None, window=0, sink=None, scale=None, status=None, quant=None, inv_gs=None,
                       partials_only=False) -> bool:
    """Tensor-core (tcgen05) paged attention for head_dim 128; `kv_map` is one row of `encode_kv_tmaps`.
    `quant` (an FP4 activation buffer): with split-KV the merge also writes the output rows quantised for the output
    projection.  Returns True when that happened (False: the caller quantises `out` itself).
    `partials_only` (context split, needs n_splits >= 2): leave the unnormalised split outputs in `part_o` / `part_ml`
    ([n_splits, T, Hq, 128] / [n_splits, T, Hq, 2]) and do not merge; `attn_merge` finishes over all owners' partials."""
    fused = quant is not None and quant.kind in FP4_KINDS and n_splits > 1 and (Hq * 128) % 256 == 0 and not partials_only
    if partials_only:
        call("cuteafd_attn_partials_only")
    call("cuteafd_paged_attention_tc", ptr(q), ptr(kv_map), ptr(page_table), ptr(kv_len), ptr(q_start), ptr(q_len), ptr(sink),
         ptr(out), ptr(part_o), ptr(part_ml), T, n_seq, max_q_len, q_stride, Hq, Hkv, page_table.shape[1], n_splits, window,
         float(scale if scale is not None else 128 ** -0.5), ptr(status), ptr(quant.data) if fused else None,
         ptr(quant.sf) if fused else None, quant.sf.shape[1] if fused else 0, ptr(inv_gs) if fused else None,
         (2 if quant.kind == KIND_MXFP4 else 1) if fused else 0, stream())
    return fused


def attn_merge(part_o, part_ml, out, *, T, Hq, n_parts, sink=None):
    """Merges `n_parts` attention partials laid side by side (unnormalised outputs [n_parts, T, Hq, 128] fp32 and
    (max, sum) pairs [n_parts, T, Hq, 2]) into `out` [T, Hq * 128] bf16.  With a context split the parts are the
    splits of every GPU that owns a piece of the context."""
    call("cuteafd_attn_merge", ptr(part_o), ptr(part_ml), ptr(sink), ptr(out), T, Hq, n_parts, stream())
    return out


def context_split_attention(q, kv_maps, page_tables, kv_lens, q_start, q_len, out, *, T, n_seq, Hq, Hkv, splits_per_part=2, scale=None,
                            status=None, sink=None):
    """Decode attention over a context whose pages are held in several paged stores (one per owner): partial attention
    per owner, then one merge.  On one GPU the owners are just different stores, which is how the path is tested; across
    GPUs every owner runs its own part and ships its `part_o` / `part_ml` slices to the merging rank with the peer copy.
    Decode rows only (one query token per sequence): every cached key is visible, so each owner passes its own length."""
    n_own = len(kv_maps)
    s = splits_per_part
    part_o = torch.empty(n_own * s * T * Hq * 128, dtype=torch.float32, device=q.device)
    part_ml = torch.empty(n_own * s * T * Hq * 2, dtype=torch.float32, device=q.device)
    for o in range(n_own):
        po = part_o[o * s * T * Hq * 128:(o + 1) * s * T * Hq * 128]
        pm = part_ml[o * s * T * Hq * 2:(o + 1) * s * T * Hq * 2]
        paged_attention_tc(q, kv_maps[o], page_tables[o], kv_lens[o], q_start, q_len, out, T=T, n_seq=n_seq, max_q_len=1, q_stride=q.stride(0),
                           Hq=Hq, Hkv=Hkv, n_splits=s, part_o=po, part_ml=pm, scale=scale, status=status, partials_only=True)
    return attn_merge(part_o, part_ml, out, T=T, Hq=Hq, n_parts=n_own * s, sink=sink)


# ------------------------------------------------------------------ sampling
def argmax_rows(logits, tok, *, rows=None, V=None, masks=None, logprob=None, status=None):
    _chk(logits, torch.float32, "logits")
    call("cuteafd_argmax_rows", ptr(logits), logits.stride(0), logits.shape[0] if rows is None else rows,
         logits.shape[1] if V is None else V, ptr(masks), masks.shape[1] if masks is not None else 0, ptr(tok), ptr(logprob),
         ptr(status), stream())
    return tok


def pack_sample_params(params_list, positions) -> torch.Tensor:
    """[(temperature, top_p, top_k, min_p, seed)], positions -> uint8 [T, 32] host tensor for `sample_rows`."""
    import struct
    buf = bytearray()
    for p, pos in zip(params_list, positions):
        buf += struct.pack("<fffiQQ", p.temperature, p.top_p, p.min_p, p.top_k, p.seed & (2 ** 64 - 1), int(pos))
    return torch.frombuffer(buf, dtype=torch.uint8).reshape(-1, 32).clone()


def sample_rows(logits, params_dev, tok, status, *, masks=None):
    _chk(logits, torch.float32, "logits")
    call("cuteafd_sample_rows", ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], ptr(masks),
         masks.shape[1] if masks is not None else 0, ptr(params_dev), ptr(tok), ptr(status), stream())
    return tok


def verify_accept(inputs, target, n_drafts, accepted, n_emit, eos: int = -1):
    n_seq, width = inputs.shape
    call("cuteafd_verify_accept", ptr(inputs), ptr(target), ptr(n_drafts), ptr(accepted), ptr(n_emit), n_seq, width, eos, stream())


# ------------------------------------------------------------------ linear attention (GDN / KDA recurrent layers)
def gated_delta_step(q, k, v, g, beta, state, slot_of_seq, q_start, q_len, out, *, snapshots=None, status=None):
    """Gated delta rule over runs of tokens: q, k, v, out bf16 [T, H, 128]; g fp32 [T, H] (decay per head) or [T, H, 128] (per key
    channel); beta fp32 [T, H]; state fp32 [slots, H, 128, 128] updated in place for the slots named by `slot_of_seq`; run s covers
    rows [q_start[s], q_start[s] + q_len[s]).  `snapshots` (fp32 [T, H, 128, 128]) receives the state after every token."""
    _chk(q, torch.bfloat16, "q"); _chk(k, torch.bfloat16, "k"); _chk(v, torch.bfloat16, "v"); _chk(out, torch.bfloat16, "out")
    _chk(g, torch.float32, "g"); _chk(beta, torch.float32, "beta"); _chk(state, torch.float32, "state")
    T, H, D = q.shape
    if D != 128 or v.shape[-1] != 128 or state.shape[1:] != (H, 128, 128):
        raise ValueError("gated_delta_step: heads are 128 x 128")
    call("cuteafd_gated_delta_step", ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), ptr(state), ptr(slot_of_seq), ptr(q_start), ptr(q_len), ptr(out),
         ptr(snapshots), slot_of_seq.numel(), H, 1 if g.dim() == 3 else 0, state.shape[0], ptr(status), stream())
    return out


def short_conv4(x, w, carry, slot_of_seq, q_start, q_len, y, *, status=None):
    """Causal depthwise convolution of width 4 + SiLU: x, y bf16 [T, C]; w fp32 [C, 4]; carry bf16 [slots, 3, C] (the last three
    inputs of every sequence, updated in place)."""
    _chk(y, torch.bfloat16, "y"); _chk(w, torch.float32, "w"); _chk(carry, torch.bfloat16, "carry")      # x may be a column slice of wider rows
    call("cuteafd_short_conv4", ptr(x), ptr(w), ptr(carry), ptr(slot_of_seq), ptr(q_start), ptr(q_len), ptr(y), slot_of_seq.numel(), y.shape[1],
         x.stride(0), carry.shape[0], ptr(status), stream())
    return y


def compress_pool(kv, scores, state, state_slot, q_start, q_len, pos0, out_start, norm_w, out, *, n_seq: int, max_blocks: int, ratio: int,
                  eps: float = 1e-6):
    """Softmax pooling of KV candidate rows into one compressed cache row per `ratio` positions (see csrc/compressor.cu): fp32
    kv / scores [T, D], per-sequence open-block state [slots, 3, D], int32 step descriptors per sequence; rows of the blocks completed
    in this step land in `out` (bf16 [n, D]) from `out_start[s]` on.  `max_blocks`: the most blocks any sequence touches in the step."""
    call("cuteafd_compress_pool", ptr(kv), ptr(scores), ptr(state), ptr(state_slot), ptr(q_start), ptr(q_len), ptr(pos0), ptr(out_start),
         ptr(norm_w), ptr(out), n_seq, max_blocks, kv.shape[1], ratio, eps, stream())
    return out
