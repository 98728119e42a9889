"""Tracing and timing helpers: named host phases, per-layer device time with CUDA events (recorded between kernel
launches, never synchronising inside a step), NVTX ranges when a profiler is attached, speculation trace JSONL.
Reference: Phase profile (families/deepseek_v4/engine.rs:203-229), layer clocks (shared/draft/clock.rs),
CUTEAFD_SPECULATION_TRACE (shared/speculation_trace.rs:16-21)."""
from __future__ import annotations

import contextlib
import json
import os
import time
from collections import defaultdict


class PhaseProfile:
    def __init__(self):
        self.totals, self.counts = defaultdict(float), defaultdict(int)

    @contextlib.contextmanager
    def phase(self, name: str):
        t0 = time.perf_counter()
        try:
            yield
        finally:
            self.totals[name] += time.perf_counter() - t0
            self.counts[name] += 1

    def snapshot(self) -> dict:
        return {k: {"ms": round(v * 1e3, 3), "n": self.counts[k]} for k, v in self.totals.items()}


class DeviceClock:
    """Pairs of CUDA events around named spans; `collect()` reads elapsed times after the step has synchronised."""

    def __init__(self):
        self.spans: list = []

    @contextlib.contextmanager
    def span(self, name: str):
        import torch
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        try:
            yield
        finally:
            b.record()
            self.spans.append((name, a, b))

    def collect(self) -> dict:
        out = defaultdict(float)
        for name, a, b in self.spans:
            out[name] += a.elapsed_time(b)
        self.spans = []
        return dict(out)


@contextlib.contextmanager
def nvtx(name: str):
    try:
        import torch
        torch.cuda.nvtx.range_push(name)
        pushed = True
    except Exception:
        pushed = False
    try:
        yield
    finally:
        if pushed:
            torch.cuda.nvtx.range_pop()


class SpeculationTrace:
    """Appends one JSON line per speculative round when CUTEAFD_SPECULATION_TRACE names a file."""

    def __init__(self, path: str | None = None):
        self.path = path or os.environ.get("CUTEAFD_SPECULATION_TRACE")

    def record(self, rid: str, drafted: int, accepted: int, step_ms: float | None = None):
        if not self.path:
            return
        with open(self.path, "a") as f:
            f.write(json.dumps({"t": time.time(), "rid": rid, "drafted": drafted, "accepted": accepted, "step_ms": step_ms}) + "\n")
