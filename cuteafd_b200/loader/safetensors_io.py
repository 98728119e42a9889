"""Minimal safetensors reader/writer: header parsing, catalog over a snapshot directory, sliced reads.

Only the header (8-byte length + JSON) is parsed to build the catalog, so planning never touches tensor bytes.
`read_rows` uses positioned reads to fetch a window of rows (a TP shard or one expert) without mapping the file.
Reference: cuteafd-loader/src/catalog.rs (headers), tensors.rs (sliced readers, row windows for TP slices).
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

DTYPES = {"F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2), "U8": (torch.uint8, 1),
          "I8": (torch.int8, 1), "I32": (torch.int32, 4), "I64": (torch.int64, 8), "F8_E4M3": (torch.uint8, 1),
          "F8_E5M2": (torch.uint8, 1), "F8_E8M0": (torch.uint8, 1), "U16": (torch.int16, 2), "I16": (torch.int16, 2), "BOOL": (torch.bool, 1)}
TO_ST = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.uint8: "U8", torch.int8: "I8",
         torch.int32: "I32", torch.int64: "I64", torch.int16: "I16", torch.bool: "BOOL"}


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: tuple
    file: str
    begin: int          # absolute byte offset in the file
    end: int

    @property
    def nbytes(self) -> int:
        return self.end - self.begin


def read_header(path: str | Path) -> tuple[dict, int]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        if n > 1 << 31:
            raise ValueError(f"{path}: implausible safetensors header length {n}")
        return json.loads(f.read(n)), 8 + n


def catalog(snapshot: str | Path) -> dict[str, TensorInfo]:
    """All tensors of every *.safetensors file in a snapshot directory (or of a single file)."""
    p = Path(snapshot)
    files = [p] if p.is_file() else sorted(p.glob("*.safetensors"))
    out: dict[str, TensorInfo] = {}
    for f in files:
        hdr, base = read_header(f)
        for name, meta in hdr.items():
            if name == "__metadata__":
                continue
            b, e = meta["data_offsets"]
            if meta["dtype"] not in DTYPES:
                raise ValueError(f"{f}: tensor {name} has unknown dtype {meta['dtype']}")
            out[name] = TensorInfo(name, meta["dtype"], tuple(meta["shape"]), str(f), base + b, base + e)
    return out


def read_tensor(info: TensorInfo) -> torch.Tensor:
    dt, _ = DTYPES[info.dtype]
    with open(info.file, "rb") as f:
        buf = bytearray(info.nbytes)
        os.preadv(f.fileno(), [buf], info.begin)
    return torch.frombuffer(buf, dtype=dt).reshape(info.shape) if info.nbytes else torch.zeros(info.shape, dtype=dt)


def read_rows(info: TensorInfo, row0: int, row1: int) -> torch.Tensor:
    """Rows [row0, row1) of the leading dimension (one positioned read)."""
    dt, es = DTYPES[info.dtype]
    if not info.shape:
        raise ValueError("scalar tensor has no rows")
    row_bytes = es * int(np.prod(info.shape[1:], dtype=np.int64)) if len(info.shape) > 1 else es
    row0, row1 = max(0, row0), min(info.shape[0], row1)
    buf = bytearray((row1 - row0) * row_bytes)
    with open(info.file, "rb") as f:
        os.preadv(f.fileno(), [buf], info.begin + row0 * row_bytes)
    return torch.frombuffer(buf, dtype=dt).reshape((row1 - row0,) + tuple(info.shape[1:]))


def write_file(path: str | Path, tensors: dict[str, torch.Tensor], dtypes: dict[str, str] | None = None, metadata: dict | None = None):
    """Writes a safetensors file (tests and synthetic snapshots).  `dtypes` overrides the header dtype string,
    e.g. {"w": "F8_E4M3"} for uint8 payloads that are FP8 bytes."""
    hdr, off, blobs = {}, 0, []
    if metadata:
        hdr["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""      # reshape: 0-dim tensors too
        hdr[name] = {"dtype": (dtypes or {}).get(name, TO_ST[t.dtype]), "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    js = json.dumps(hdr, separators=(",", ":")).encode()
    js += b" " * ((8 - len(js) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(js)))
        f.write(js)
        for b in blobs:
            f.write(b)
