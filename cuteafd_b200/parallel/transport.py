"""Host transports for expert waves: in-process and TCP (loopback or multi-host), with per-phase timeouts, bounded
retries on a fresh connection, and synthetic executors for tests.

A wave is never replayed after its response started arriving (a partial response means the executor may have
side effects in flight), a connection that died before any response byte is retried once on a new connection, a
dead server fails fast and recovers when it comes back, and every failure is reported to `Health`.
Reference: cuteafd-transport/src/lib.rs:100-141 (phase budgets, transports), protocol_v2_tcp.rs, synthetic.rs:51-131
(EchoExecutor / SyntheticRouteExecutor), tests/upstream_fault_injection.rs:331-749.
"""
from __future__ import annotations

import socket
import socketserver
import struct
import threading
import time

import numpy as np

from . import protocol as P
from .health import Health


class TransportError(RuntimeError):
    pass


# ------------------------------------------------------------------ executors
class EchoExecutor:
    """Returns the request rows (decoded to bf16 size) unchanged: transport tests."""
    def __init__(self, executor_id: int = 0):
        self.executor_id = executor_id

    def execute(self, req: P.Request) -> P.Response:
        n = req.rows * P.row_bytes(P.DT_BF16, req.hidden)
        data = (req.payload * (n // max(1, len(req.payload)) + 1))[:n] if req.payload else b"\0" * n
        return P.Response(req.seq, req.layer, req.rows, req.hidden, self.executor_id, P.DT_BF16, 0, data)


class SyntheticRouteExecutor:
    """Deterministic stand-in for GPU experts: out[row] = sum_routes gate * (expert + 1), broadcast over hidden."""
    def __init__(self, executor_id: int = 0, row_capacity: int = 4096):
        self.executor_id, self.row_capacity = executor_id, row_capacity

    def execute(self, req: P.Request) -> P.Response:
        if req.rows > self.row_capacity:          # answered, not dropped
            return P.Response(req.seq, req.layer, 0, self.row_capacity, self.executor_id, P.DT_F32, P.FLAG_ROW_CAPACITY_ERROR, b"")
        acc = np.zeros(req.rows, dtype=np.float32)
        live = req.routes["expert"] != P.UNASSIGNED
        np.add.at(acc, req.routes["row"][live], req.routes["gate"][live] * (req.routes["expert"][live] + 1).astype(np.float32))
        out = np.repeat(acc[:, None], req.hidden, axis=1).astype(np.float32)
        return P.Response(req.seq, req.layer, req.rows, req.hidden, self.executor_id, P.DT_F32, 0, out.tobytes())


# ------------------------------------------------------------------ in-process
class InProcTransport:
    def __init__(self, executor, health: Health | None = None):
        self.executor, self.health = executor, health or Health()

    def exchange(self, req: P.Request) -> P.Response:
        self.health.require_live()
        try:
            return P.decode_response(self.executor.execute(P.decode_request(req.encode())).encode())
        except Exception as e:
            self.health.record_failure(f"in-proc executor: {e}")
            raise TransportError(str(e)) from e


# ------------------------------------------------------------------ TCP
def _recv_exact(sock: socket.socket, n: int, deadline: float) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        left = deadline - time.monotonic()
        if left <= 0:
            raise socket.timeout("phase budget exhausted")
        sock.settimeout(left)
        chunk = sock.recv(n - len(buf))
        if not chunk:
            raise ConnectionError(f"peer closed after {len(buf)} of {n} bytes")
        buf += chunk
    return bytes(buf)


class ExpertServer:
    """Threaded TCP server around an executor (the `expertd` host path).  `fault` hooks let tests break it."""

    def __init__(self, executor, host: str = "127.0.0.1", port: int = 0):
        self.executor = executor
        self.fault: str | None = None       # None | "hang" | "header_then_stall" | "truncate" | "close"
        outer = self

        class Handler(socketserver.BaseRequestHandler):
            def handle(self):
                sock = self.request
                try:
                    while True:
                        hdr = _recv_exact(sock, P.HEADER_LEN, time.monotonic() + 3600)
                        body = _recv_exact(sock, P.request_body_len(hdr), time.monotonic() + 30)
                        fault, outer.fault = outer.fault, (None if outer.fault in ("close", "truncate", "header_then_stall") else outer.fault)
                        if fault == "close":
                            return
                        if fault == "hang":
                            time.sleep(outer.hang_s)
                            return
                        resp = outer.executor.execute(P.decode_request(hdr + body)).encode()
                        if fault == "header_then_stall":
                            sock.sendall(resp[:P.HEADER_LEN])
                            time.sleep(outer.hang_s)
                            return
                        if fault == "truncate":
                            sock.sendall(resp[:P.HEADER_LEN + max(0, (len(resp) - P.HEADER_LEN) // 2)])
                            return
                        sock.sendall(resp)
                except (ConnectionError, socket.timeout, OSError, P.ProtocolError):
                    return

        class Server(socketserver.ThreadingTCPServer):
            allow_reuse_address = True
            daemon_threads = True

        self.hang_s = 5.0
        self.server = Server((host, port), Handler)
        self.address = self.server.server_address
        self.thread = threading.Thread(target=self.server.serve_forever, daemon=True)
        self.thread.start()

    def stop(self):
        self.server.shutdown()
        self.server.server_close()


class TcpTransport:
    def __init__(self, address, health: Health | None = None, connect_s: float = 2.0, send_s: float = 5.0, recv_s: float = 5.0):
        self.address, self.health = address, health or Health()
        self.connect_s, self.send_s, self.recv_s = connect_s, send_s, recv_s
        self.sock: socket.socket | None = None
        self.stats = {"exchanges": 0, "retries": 0, "failures": 0}

    def _connect(self):
        self.sock = socket.create_connection(self.address, timeout=self.connect_s)
        self.sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)

    def close(self):
        if self.sock is not None:
            try:
                self.sock.close()
            finally:
                self.sock = None

    def exchange(self, req: P.Request, terminal: bool = True) -> P.Response:
        """One wave.  `terminal=False` reports a failure to the caller without marking the wire dead (probes)."""
        self.health.require_live()
        frame = req.encode()
        for attempt in (0, 1):
            started = False        # True once any response byte arrived: from then on the wave is never replayed
            try:
                if self.sock is None:
                    self._connect()
                self.sock.settimeout(self.send_s)
                self.sock.sendall(frame)
                hdr = _recv_exact(self.sock, 1, time.monotonic() + self.recv_s)
                started = True
                hdr += _recv_exact(self.sock, P.HEADER_LEN - 1, time.monotonic() + self.recv_s)
                body = _recv_exact(self.sock, P.response_body_len(hdr), time.monotonic() + self.recv_s)
                resp = P.decode_response(hdr + body)
                if resp.seq != req.seq or resp.layer != req.layer:
                    raise P.ProtocolError(f"response for wave {resp.seq}/{resp.layer}, expected {req.seq}/{req.layer}")
                self.stats["exchanges"] += 1
                return resp
            except (OSError, ConnectionError, socket.timeout, P.ProtocolError) as e:
                self.close()
                retryable = not started and attempt == 0 and isinstance(e, (ConnectionError, BrokenPipeError, ConnectionResetError)) \
                    and not isinstance(e, socket.timeout)
                if retryable:
                    self.stats["retries"] += 1
                    continue
                self.stats["failures"] += 1
                cause = f"expert wave {req.seq} layer {req.layer}: {type(e).__name__}: {e}"
                if terminal:
                    self.health.record_failure(cause)
                raise TransportError(cause) from e
        raise TransportError("unreachable")


def gather_in_rank_order(responses: list[P.Response], n_ranks: int) -> list[P.Response]:
    """Partials are reduced in executor-id order whatever the arrival order (the combine's determinism contract)."""
    by_id = {r.executor_id: r for r in responses}
    if sorted(by_id) != list(range(n_ranks)):
        raise TransportError(f"expected one response from each of {n_ranks} ranks, got ids {sorted(by_id)}")
    return [by_id[i] for i in range(n_ranks)]
