"""Step mailbox: ordered delivery to several reader processes, payloads intact, timeouts and overruns reported."""
import multiprocessing as mp
import os

import numpy as np
import pytest

from cuteafd_b200.parallel.mailbox import Mailbox, MailboxTimeout


def _reader(name, n, q):
    mb = Mailbox(name, create=False, slots=8, payload_bytes=256)
    got = []
    for _ in range(n):
        op, a, b, payload = mb.read(timeout_s=20)
        got.append((op, a, b, payload))
    q.put(got)
    mb.close()


def test_messages_arrive_in_order_at_every_reader():
    name = f"cuteafd_test_{os.getpid()}"
    mb = Mailbox(name, create=True, slots=8, payload_bytes=256)
    try:
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        procs = [ctx.Process(target=_reader, args=(name, 5, q)) for _ in range(2)]
        for p in procs:
            p.start()
        for i in range(5):
            mb.post(1 + i, a=10 * i, b=-i, payload=np.arange(i * 3, dtype=np.int32))
        outs = [q.get(timeout=60) for _ in procs]
        for p in procs:
            p.join(timeout=30)
        for got in outs:
            assert [g[:3] for g in got] == [(1 + i, 10 * i, -i) for i in range(5)]
            assert [np.frombuffer(g[3], dtype=np.int32).tolist() for g in got] == [list(range(i * 3)) for i in range(5)]
    finally:
        mb.close()


def test_timeout_and_overrun_are_errors():
    name = f"cuteafd_test2_{os.getpid()}"
    mb = Mailbox(name, create=True, slots=4, payload_bytes=64)
    try:
        rd = Mailbox(name, create=False, slots=4, payload_bytes=64)
        with pytest.raises(MailboxTimeout):
            rd.read(timeout_s=0.05)
        for i in range(6):                       # the reader never kept up: message 1 is gone
            mb.post(7, a=i)
        with pytest.raises(RuntimeError, match="overrun"):
            rd.read(timeout_s=1)
        with pytest.raises(ValueError):
            mb.post(1, payload=b"x" * 100)
        rd.close()
    finally:
        mb.close()
