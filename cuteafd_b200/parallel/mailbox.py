"""Host-side step mailbox between the ranks of one node: a single-writer ring in POSIX shared memory.

The attention leader posts one small message per step (what to run, the active shapes, optionally the step's input block
for its tensor-parallel partner); every other rank polls the ring from its own process.  A post is two plain stores and a
read is a spin on one 64-bit word, so the control path costs about a microsecond instead of a collective on a CPU process
group - the data path (rows, routing tables, flags) never touches the host at all.

Layout: [write_seq u64 | pad to 64 B] then `slots` entries of (seq u64, op i64, a i64, b i64, nbytes i64, payload).  The
writer fills an entry, stores its sequence number last, then advances write_seq; a reader that wants message n spins
until entry n % slots carries seq n.  A reader more than `slots` messages behind has lost data and raises.
Reference: the GPU mailbox + host proxy thread of the device-driven lane (cuteafd-transport/src/expert/device.rs,
peer_exchange.cu:153-168 host_signal) plays the same role between coordinator and expert hosts.
"""
from __future__ import annotations

import time
from multiprocessing import shared_memory

import numpy as np

HEADER = 64
ENTRY_HEAD = 40


class MailboxTimeout(RuntimeError):
    pass


class Mailbox:
    def __init__(self, name: str, *, create: bool, slots: int = 64, payload_bytes: int = 1 << 16):
        self.slots, self.payload_bytes = slots, payload_bytes
        self.entry = ENTRY_HEAD + payload_bytes
        size = HEADER + slots * self.entry
        self.shm = shared_memory.SharedMemory(name=name, create=create, size=size)
        self.owner = create
        self.buf = np.frombuffer(self.shm.buf, dtype=np.uint8, count=size)
        self.head = self.buf[:8].view(np.int64)
        if create:
            self.buf[:] = 0
        self.next_read = 1
        self.next_write = 1

    def _entry(self, seq: int):
        off = HEADER + (seq % self.slots) * self.entry
        return self.buf[off:off + ENTRY_HEAD].view(np.int64), self.buf[off + ENTRY_HEAD:off + self.entry]

    # ---- writer
    def post(self, op: int, a: int = 0, b: int = 0, payload: bytes | np.ndarray | None = None) -> int:
        seq = self.next_write
        head, body = self._entry(seq)
        n = 0
        if payload is not None:
            raw = np.frombuffer(payload, dtype=np.uint8) if isinstance(payload, (bytes, bytearray, memoryview)) else payload.view(np.uint8).reshape(-1)
            n = raw.size
            if n > self.payload_bytes:
                raise ValueError(f"mailbox payload of {n} bytes exceeds the slot size {self.payload_bytes}")
            body[:n] = raw
        head[0] = 0                     # invalidate while the entry is rewritten
        head[1], head[2], head[3], head[4] = op, a, b, n
        head[0] = seq
        self.head[0] = seq
        self.next_write = seq + 1
        return seq

    # ---- readers
    def read(self, timeout_s: float = 120.0):
        """Next message in order: (op, a, b, payload bytes)."""
        seq = self.next_read
        head, body = self._entry(seq)
        t0, spins = time.monotonic(), 0
        while int(head[0]) != seq:
            if int(head[0]) > seq:
                raise RuntimeError(f"mailbox overrun: wanted message {seq}, slot already holds {int(head[0])}")
            spins += 1
            if spins & 0x3FF == 0:
                if time.monotonic() - t0 > timeout_s:
                    raise MailboxTimeout(f"no message {seq} within {timeout_s} s")
                if spins > 200000:
                    time.sleep(0.0002)      # a long-idle reader stops burning a core
        op, a, b, n = int(head[1]), int(head[2]), int(head[3]), int(head[4])
        payload = bytes(body[:n]) if n else b""
        if int(head[0]) != seq:
            raise RuntimeError(f"mailbox overrun while reading message {seq}")
        self.next_read = seq + 1
        return op, a, b, payload

    def close(self):
        self.head = self.buf = None
        try:
            self.shm.close()
            if self.owner:
                self.shm.unlink()
        except Exception:
            pass
