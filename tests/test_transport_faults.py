"""Wire protocol + transports with host-side fault injection (no GPU): truncated frames, stalls, dropped
connections, dead servers, rank-ordered gathering, terminal failure fan-out.  Mirrors the classes of
cuteafd-transport/tests/upstream_fault_injection.rs:331-749."""
import numpy as np
import pytest

from cuteafd_b200.parallel import protocol as P
from cuteafd_b200.parallel.health import Health, TerminalState
from cuteafd_b200.parallel.transport import (EchoExecutor, ExpertServer, InProcTransport, SyntheticRouteExecutor, TcpTransport,
                                            TransportError, gather_in_rank_order)


def make_request(seq=1, rows=3, hidden=64, top_k=2, n_experts=8, flags=P.FLAG_CHECKSUM):
    rng = np.random.default_rng(seq)
    routes = np.zeros(rows * top_k, dtype=[("row", "<u4"), ("expert", "<u4"), ("gate", "<f4")])
    for r in range(rows):
        routes["row"][r * top_k:(r + 1) * top_k] = r
        routes["expert"][r * top_k:(r + 1) * top_k] = rng.permutation(n_experts)[:top_k]
    routes["gate"] = rng.random(rows * top_k).astype(np.float32)
    payload = bytes(rng.integers(0, 255, rows * P.row_bytes(P.DT_FP8_UE8M0, hidden), dtype=np.uint8))
    return P.Request(seq, 5, rows, hidden, top_k, P.DT_FP8_UE8M0, P.SRC_DECODE, flags, routes, payload)


def test_frames_roundtrip_and_validation():
    req = make_request()
    buf = req.encode()
    assert len(buf) == P.HEADER_LEN + 6 * P.ROUTE_LEN + 3 * (64 + 2) and buf[:8] == b"CUTEAFD3"
    back = P.decode_request(buf, n_experts=8)
    assert back.seq == 1 and back.layer == 5 and np.array_equal(back.routes, req.routes) and back.payload == req.payload
    with pytest.raises(P.ProtocolError, match="truncated"):
        P.decode_request(buf[:-5])
    with pytest.raises(P.ProtocolError, match="checksum"):
        P.decode_request(buf[:-1] + bytes([buf[-1] ^ 1]))
    dup = make_request()
    dup.routes["expert"][1] = dup.routes["expert"][0]
    with pytest.raises(P.ProtocolError, match="duplicate"):
        P.decode_request(dup.encode())
    neg = make_request()
    neg.routes["gate"][0] = -1
    with pytest.raises(P.ProtocolError, match="gate"):
        P.decode_request(neg.encode())
    with pytest.raises(P.ProtocolError, match="magic"):
        P.decode_request(b"X" * 200)
    owned = P.assign_owners(req.routes, 8, 2, 1)
    assert ((owned["expert"] >= 4) | (owned["expert"] == P.UNASSIGNED)).all() and (owned["gate"][owned["expert"] == P.UNASSIGNED] == 0).all()


def test_synthetic_executor_and_rank_ordered_gather():
    req = make_request(rows=4)
    outs = []
    for g in (1, 0):                       # arrive out of order
        part = P.Request(req.seq, req.layer, req.rows, req.hidden, req.top_k, req.dtype, req.source, 0,
                         P.assign_owners(req.routes, 8, 2, g), req.payload)
        outs.append(InProcTransport(SyntheticRouteExecutor(executor_id=g)).exchange(part))
    ordered = gather_in_rank_order(outs, 2)
    assert [r.executor_id for r in ordered] == [0, 1]
    total = sum(np.frombuffer(r.payload, dtype=np.float32).reshape(4, 64) for r in ordered)
    want = np.zeros(4, dtype=np.float32)
    np.add.at(want, req.routes["row"], req.routes["gate"] * (req.routes["expert"] + 1))
    assert np.allclose(total[:, 0], want, rtol=1e-6)
    with pytest.raises(TransportError):
        gather_in_rank_order(outs[:1], 2)
    cap = InProcTransport(SyntheticRouteExecutor(row_capacity=2)).exchange(req)
    assert cap.flags & P.FLAG_ROW_CAPACITY_ERROR and cap.hidden == 2        # capacity errors are answered, not dropped


@pytest.fixture
def server():
    s = ExpertServer(EchoExecutor(executor_id=3))
    s.hang_s = 1.5
    yield s
    s.stop()


def test_tcp_exchange_and_retry_on_fresh_connection(server):
    t = TcpTransport(server.address, recv_s=1.0)
    assert t.exchange(make_request(seq=1)).executor_id == 3
    server.fault = "close"                                  # connection dies before any response byte: one retry
    assert t.exchange(make_request(seq=2)).seq == 2
    assert t.stats["retries"] == 1 and t.health.live


@pytest.mark.parametrize("fault,needle", [("hang", "timeout"), ("header_then_stall", "timeout"), ("truncate", "closed")])
def test_tcp_faults_are_terminal_and_never_replayed(server, fault, needle):
    heard = []
    h = Health()
    h.on_failure(heard.append)
    t = TcpTransport(server.address, health=h, recv_s=0.4)
    server.fault = fault
    with pytest.raises(TransportError) as e:
        t.exchange(make_request(seq=7))
    assert needle in str(e.value).lower() or "timed out" in str(e.value).lower()
    assert not h.live and h.state == TerminalState.ABORTING and len(heard) == 1 and t.stats["retries"] == 0
    with pytest.raises(RuntimeError, match="expert wire failed"):
        t.exchange(make_request(seq=8))                     # fail fast afterwards, nothing is queued
    h.drained(False)
    assert h.snapshot()["state"] == "retained"


def test_dead_server_fails_fast_and_probe_recovers():
    s = ExpertServer(EchoExecutor())
    addr = s.address
    s.stop()
    t = TcpTransport(addr, connect_s=0.3)
    with pytest.raises(TransportError):
        t.exchange(make_request(), terminal=False)          # a probe does not kill the wire
    assert t.health.live
    s2 = ExpertServer(EchoExecutor(), port=addr[1])
    try:
        assert t.exchange(make_request(seq=9)).seq == 9
    finally:
        s2.stop()
