"""Failure bookkeeping for the expert wire: the first failure is terminal for the process (the serving loop stops
admitting, `/health` turns unavailable, queued and running requests are told why); later failures are counted
but do not overwrite the cause.  Reference: cuteafd-transport/src/lib.rs:13-25 (`health::record_failure`),
cuteafd-api/src/openai/health.rs, shared/peer_split.rs:62-84 (terminal state of a peer exchange)."""
from __future__ import annotations

import enum
import threading
import time


class TerminalState(enum.Enum):
    ACTIVE = "active"
    ABORTING = "aborting"
    DRAINED = "drained"
    RETAINED = "retained"      # drain failed: storage is kept alive because a device graph may still touch it


class Health:
    def __init__(self):
        self._lock = threading.Lock()
        self.cause: str | None = None
        self.failed_at: float | None = None
        self.failures = 0
        self.state = TerminalState.ACTIVE
        self.listeners: list = []

    def record_failure(self, cause: str):
        with self._lock:
            self.failures += 1
            first = self.cause is None
            if first:
                self.cause, self.failed_at, self.state = cause, time.time(), TerminalState.ABORTING
            listeners = list(self.listeners) if first else []
        for fn in listeners:
            fn(cause)

    def on_failure(self, fn):
        self.listeners.append(fn)

    def drained(self, ok: bool):
        with self._lock:
            self.state = TerminalState.DRAINED if ok else TerminalState.RETAINED

    @property
    def live(self) -> bool:
        return self.cause is None

    def require_live(self):
        if self.cause is not None:
            raise RuntimeError(f"expert wire failed: {self.cause}")

    def snapshot(self) -> dict:
        return {"live": self.live, "cause": self.cause, "failures": self.failures, "state": self.state.value}


def device_status_to_failure(word: int) -> str | None:
    """Maps a kernel status word (bounded wait ran out, bad index) to a failure cause, or None when clean."""
    if word == 0:
        return None
    from ..ops.native import decode_status
    return "device: " + decode_status(word)
