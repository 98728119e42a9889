"""N-gram memory on the GPU: per engram layer, gather the addressed table rows, project them, gate them into the residual stream(s).

`EngramModule` holds the tables (in device memory, or in pinned host memory that the gather kernel reads in place: a full model's
tables are two times ~100 GB, a step needs 24 rows of 264 bytes per token and layer), the projection (a bf16 `tc_linear`: width
24 * row_dim -> (streams + 1) * hidden) and the gate vectors.  A step's addresses are computed on the host from the token ids
(`ref/engram.py::EngramAddressing`) and arrive with ONE host-to-device copy for all engram layers (`set_hashes`); `apply` is three
launches per layer (gather + dequantise, GEMM, gate) and is safe to capture in a CUDA graph (it reads the same address buffer every
replay).

Reference: rust/crates/cuteafd-daemon/src/families/deepseek_v41/v41_engram.rs (gathered rows -> embedding -> gates),
native/families/deepseek_v41/cuda/engram.cu.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from ..ops import KIND_BF16, ActBuffer, TcWeight, native
from ..ops.native import ptr
from ..ref.engram import COLUMNS, EngramAddressing, EngramSpec


class EngramModule:
    def __init__(self, spec: EngramSpec, masters: dict, device, cap: int = 256, tables: str = "device"):
        native.require_gpu_lib()
        if tables not in ("device", "host"):
            raise ValueError("engram tables live in 'device' memory or pinned 'host' memory")
        self.spec, self.device, self.cap = spec, torch.device(device), cap
        self.addr = EngramAddressing(spec)
        S, H = spec.streams, spec.hidden
        self.layers = []
        for l, lw in enumerate(masters["layers"]):
            if lw["table_q"].shape != (self.addr.rows[l], spec.row_dim):
                raise ValueError(f"engram layer {l}: table of {tuple(lw['table_q'].shape)}, addressing needs {(self.addr.rows[l], spec.row_dim)}")
            place = (lambda t: t.contiguous().pin_memory()) if tables == "host" else (lambda t: t.contiguous().to(self.device))
            self.layers.append({"tq": place(lw["table_q"]), "te": place(lw["table_e"]), "proj": TcWeight.from_master(lw["proj"].float(), KIND_BF16, self.device),
                                "wq": lw["wq"].float().to(self.device).contiguous(), "wk": lw["wk"].float().to(self.device).contiguous()})
        n = len(self.layers)
        self.idx_host = torch.zeros(n, cap, COLUMNS, dtype=torch.int64).pin_memory()
        self.idx = torch.zeros(n, cap, COLUMNS, dtype=torch.int64, device=self.device)
        self.mask_host = torch.ones(cap, dtype=torch.uint8).pin_memory()
        self.mask = torch.ones(cap, dtype=torch.uint8, device=self.device)
        self.rows = torch.zeros(cap, spec.width, dtype=torch.bfloat16, device=self.device)
        self.kv = torch.zeros(cap, (S + 1) * H, dtype=torch.bfloat16, device=self.device)
        self._acts: dict = {}
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.use_mask = False

    def nbytes(self) -> dict:
        t = sum(l["tq"].numel() + l["te"].numel() for l in self.layers)
        return {"tables": t, "tables_on_device": bool(self.layers and self.layers[0]["tq"].is_cuda), "weights": sum(l["proj"].nbytes for l in self.layers)}

    def set_hashes(self, hashes: np.ndarray, text_mask=None) -> int:
        """hashes: uint64 [layers, T, 24] (`EngramAddressing.hashes`); text_mask: per token, False for image positions.  Returns bytes copied."""
        T = hashes.shape[1]
        if T > self.cap or hashes.shape[0] != len(self.layers):
            raise ValueError(f"engram: {T} rows in a step (capacity {self.cap})")
        self.idx_host[:, :T] = torch.from_numpy(hashes.astype(np.int64))
        self.idx.copy_(self.idx_host, non_blocking=True)
        self.use_mask = text_mask is not None
        if self.use_mask:
            self.mask_host[:T] = torch.as_tensor(text_mask, dtype=torch.uint8)
            self.mask.copy_(self.mask_host, non_blocking=True)
        return self.idx_host.numel() * 8

    def apply(self, e: int, x: torch.Tensor, T: int) -> int:
        """x: bf16 [>= T, streams * hidden] rows, updated in place.  Returns the number of launches."""
        spec, lw = self.spec, self.layers[e]
        mask = ptr(self.mask) if self.use_mask else None
        native.call("cuteafd_engram_gather", ptr(lw["tq"]), ptr(lw["te"]), ptr(self.idx[e]), mask, ptr(self.rows), T, spec.row_dim,
                    lw["tq"].shape[0], ptr(self.status), native.stream())
        tn = ops.pick_tn(T)
        if tn not in self._acts:
            self._acts[tn] = ActBuffer.wrap_bf16(self.rows, tn)
        ops.tc_linear(lw["proj"], self._acts[tn], self.kv, rows=T, status=self.status)
        native.call("cuteafd_engram_gate", ptr(x), ptr(self.kv), self.kv.shape[1], ptr(lw["wq"]), ptr(lw["wk"]), mask, T, spec.streams, spec.hidden,
                    native.stream())
        return 3

    def check_status(self):
        word = int(self.status[0])
        if word:
            self.status.zero_()
            raise RuntimeError(f"engram: device status {native.decode_status(word)}")
