"""Expert wire protocol (host path): framed requests/responses for expert waves sent over TCP or in-process
transports - bootstrap, tests, multi-host expert pools and the reference-compatible `expertd` role.  Inside one
NVSwitch node the data path uses peer memory instead (`csrc/peer.cu`) and only (op, rows) control words cross the host.

Frame layout (little endian), following the reference's surface (cuteafd-transport/src/protocol_v2.rs:12-46,
270-331): magic `CUTEAFD3`, version 3, 96-byte request and response headers, 12-byte route entries
{row u32, expert u32, gate f32}, row payloads in one of the row dtypes (BF16, FP8 E4M3 + UE8M0/32 "wire rows",
NVFP4, F32), flags (debug checksum, warm-up, row-capacity error), responses tagged with the executor id so
partials are collected in rank order whatever the arrival order.
"""
from __future__ import annotations

import hashlib
import struct
from dataclasses import dataclass, field

import numpy as np

MAGIC, VERSION = b"CUTEAFD3", 3
KIND_REQUEST, KIND_RESPONSE = 1, 2
HEADER_LEN, ROUTE_LEN = 96, 12
FLAG_CHECKSUM, FLAG_WARMUP, FLAG_ROW_CAPACITY_ERROR = 1 << 0, 1 << 1, 1 << 17
DT_BF16, DT_F16, DT_NVFP4, DT_FP8_ROW, DT_F32, DT_FP8_UE8M0 = 1, 2, 4, 5, 6, 7
SRC_DECODE, SRC_PREFILL, SRC_VERIFY, SRC_BENCH = 0, 1, 2, 3
UNASSIGNED = 0xFFFFFFFF


class ProtocolError(ValueError):
    pass


def row_bytes(dtype: int, hidden: int) -> int:
    if dtype in (DT_BF16, DT_F16):
        return hidden * 2
    if dtype == DT_F32:
        return hidden * 4
    if dtype == DT_FP8_UE8M0:
        return hidden + hidden // 32
    if dtype == DT_FP8_ROW:
        return hidden + 4
    if dtype == DT_NVFP4:
        return hidden // 2 + hidden // 16
    raise ProtocolError(f"unknown row dtype {dtype}")


@dataclass
class Request:
    seq: int
    layer: int
    rows: int
    hidden: int
    top_k: int
    dtype: int = DT_FP8_UE8M0
    source: int = SRC_DECODE
    flags: int = 0
    routes: np.ndarray = field(default_factory=lambda: np.zeros(0, dtype=[("row", "<u4"), ("expert", "<u4"), ("gate", "<f4")]))
    payload: bytes = b""

    def encode(self) -> bytes:
        rt = self.routes.tobytes()
        body = rt + self.payload
        digest = hashlib.sha256(body).digest()[:4] if self.flags & FLAG_CHECKSUM else b"\0" * 4
        hdr = struct.pack("<8sHHIQIIIIIIII", MAGIC, VERSION, KIND_REQUEST, self.flags, self.seq, self.layer, self.rows, self.hidden,
                          self.top_k, self.dtype, self.source, len(self.routes), len(self.payload))
        hdr = hdr.ljust(HEADER_LEN - 4, b"\0") + digest
        return hdr + body


@dataclass
class Response:
    seq: int
    layer: int
    rows: int
    hidden: int
    executor_id: int
    dtype: int = DT_BF16
    flags: int = 0
    payload: bytes = b""

    def encode(self) -> bytes:
        digest = hashlib.sha256(self.payload).digest()[:4] if self.flags & FLAG_CHECKSUM else b"\0" * 4
        hdr = struct.pack("<8sHHIQIIIIII", MAGIC, VERSION, KIND_RESPONSE, self.flags, self.seq, self.layer, self.rows, self.hidden,
                          self.dtype, self.executor_id, len(self.payload))
        return hdr.ljust(HEADER_LEN - 4, b"\0") + digest + self.payload


def _check_magic(buf: bytes, kind: int):
    if len(buf) < HEADER_LEN:
        raise ProtocolError(f"truncated header: {len(buf)} of {HEADER_LEN} bytes")
    magic, ver, k = struct.unpack_from("<8sHH", buf)
    if magic != MAGIC:
        raise ProtocolError("bad magic")
    if ver != VERSION:
        raise ProtocolError(f"unsupported protocol version {ver}")
    if k != kind:
        raise ProtocolError(f"expected frame kind {kind}, got {k}")


def request_body_len(hdr: bytes) -> int:
    _check_magic(hdr, KIND_REQUEST)
    n_routes, n_payload = struct.unpack_from("<II", hdr, 8 + 2 + 2 + 4 + 8 + 4 * 6)
    return n_routes * ROUTE_LEN + n_payload


def response_body_len(hdr: bytes) -> int:
    _check_magic(hdr, KIND_RESPONSE)
    return struct.unpack_from("<I", hdr, 8 + 2 + 2 + 4 + 8 + 4 * 5)[0]


def decode_request(buf: bytes, n_experts: int | None = None) -> Request:
    """Parses and validates: top_k routes per row, no duplicate experts in a row, finite non-negative weights
    (reference: cuteafd-transport/src/expert.rs:83-160)."""
    _check_magic(buf, KIND_REQUEST)
    (flags, seq, layer, rows, hidden, top_k, dtype, source, n_routes, n_payload) = struct.unpack_from("<IQIIIIIIII", buf, 12)
    body = buf[HEADER_LEN:]
    if len(body) != n_routes * ROUTE_LEN + n_payload:
        raise ProtocolError(f"truncated payload: have {len(body)} bytes, header says {n_routes * ROUTE_LEN + n_payload}")
    if flags & FLAG_CHECKSUM and hashlib.sha256(body).digest()[:4] != buf[HEADER_LEN - 4:HEADER_LEN]:
        raise ProtocolError("checksum mismatch")
    if n_payload != rows * row_bytes(dtype, hidden):
        raise ProtocolError(f"payload of {n_payload} bytes does not hold {rows} rows of dtype {dtype}")
    if n_routes != rows * top_k:
        raise ProtocolError(f"{n_routes} routes for {rows} rows x top-{top_k}")
    routes = np.frombuffer(body[:n_routes * ROUTE_LEN], dtype=[("row", "<u4"), ("expert", "<u4"), ("gate", "<f4")]).copy()
    if n_routes:
        if (routes["row"] >= rows).any():
            raise ProtocolError("route names a row outside the request")
        if not np.isfinite(routes["gate"]).all() or (routes["gate"] < 0).any():
            raise ProtocolError("gate weights must be finite and non-negative")
        if n_experts is not None and ((routes["expert"] >= n_experts) & (routes["expert"] != UNASSIGNED)).any():
            raise ProtocolError("route names an unknown expert")
        per_row = routes["expert"].reshape(rows, top_k)
        srt = np.sort(per_row, axis=1)
        if ((srt[:, 1:] == srt[:, :-1]) & (srt[:, 1:] != UNASSIGNED)).any():
            raise ProtocolError("duplicate expert in one row")
    return Request(seq, layer, rows, hidden, top_k, dtype, source, flags, routes, body[n_routes * ROUTE_LEN:])


def decode_response(buf: bytes) -> Response:
    _check_magic(buf, KIND_RESPONSE)
    (flags, seq, layer, rows, hidden, dtype, executor_id, n_payload) = struct.unpack_from("<IQIIIIII", buf, 12)
    body = buf[HEADER_LEN:]
    if len(body) != n_payload:
        raise ProtocolError(f"truncated payload: have {len(body)} bytes, header says {n_payload}")
    if flags & FLAG_CHECKSUM and hashlib.sha256(body).digest()[:4] != buf[HEADER_LEN - 4:HEADER_LEN]:
        raise ProtocolError("checksum mismatch")
    if not flags & FLAG_ROW_CAPACITY_ERROR and n_payload != rows * row_bytes(dtype, hidden):
        raise ProtocolError("response payload size does not match its rows")
    return Response(seq, layer, rows, hidden, executor_id, dtype, flags, body)


def assign_owners(routes: np.ndarray, n_experts: int, n_groups: int, group: int) -> np.ndarray:
    """Replicated-group routing: routes whose expert another group owns become UNASSIGNED with weight 0
    (reference: expert.rs:275-323)."""
    out = routes.copy()
    lo, hi = (group * n_experts) // n_groups, ((group + 1) * n_experts) // n_groups
    other = (out["expert"] < lo) | (out["expert"] >= hi)
    out["expert"][other] = UNASSIGNED
    out["gate"][other] = 0.0
    return out
