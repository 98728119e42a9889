"""Census of the CUDA-graph bank: which exact shapes were captured, how often each is replayed, and a capture watch.

Decode steps replay graphs keyed by their exact shape; a serving process warms the shapes it will see (row buckets
1 / 4 / 16 / 64) and then `seal()`s the census - from there on every new capture is a steady-state capture, which the
serving loop treats as a defect to report (a capture costs milliseconds and allocates).  The census also keeps the two
timing arms per shape when a caller measures them (eager launch sequence vs graph replay), which is how the launch-bound
share of a step is read.

Reference: cuteafd-daemon/src/shared/decode_graph.rs:1-25 (bank keyed by exact shape, row buckets, zero steady-state
captures rule), decode_graph/census.rs:1-45 (graph vs eager arms).
"""
from __future__ import annotations

from dataclasses import dataclass, field

ROW_BUCKETS = (1, 4, 16, 64)


def bucket_rows(n: int, buckets=ROW_BUCKETS) -> int:
    """Smallest bucket holding `n` rows; beyond the largest bucket rows are rounded up to a multiple of it."""
    for b in buckets:
        if n <= b:
            return b
    top = buckets[-1]
    return -(-n // top) * top


@dataclass
class ShapeRecord:
    captures: int = 0
    replays: int = 0
    eager_runs: int = 0
    eager_ms: float | None = None
    graph_ms: float | None = None
    launches: int = 0


@dataclass
class GraphCensus:
    shapes: dict = field(default_factory=dict)
    sealed: bool = False
    steady_state_captures: list = field(default_factory=list)

    def _rec(self, key) -> ShapeRecord:
        r = self.shapes.get(key)
        if r is None:
            r = self.shapes[key] = ShapeRecord()
        return r

    def captured(self, key, launches: int = 0):
        r = self._rec(key)
        r.captures += 1
        r.launches = launches
        if self.sealed:
            self.steady_state_captures.append(key)

    def replayed(self, key):
        self._rec(key).replays += 1

    def ran_eager(self, key):
        self._rec(key).eager_runs += 1

    def arms(self, key, eager_ms: float, graph_ms: float):
        r = self._rec(key)
        r.eager_ms, r.graph_ms = eager_ms, graph_ms

    def seal(self):
        """Warm-up is over: captures from here on are reported."""
        self.sealed = True

    def invalidate(self):
        """The bank was dropped (buffers moved): capture counts restart, the seal is lifted until the next warm-up."""
        self.shapes.clear()
        self.sealed = False

    def snapshot(self) -> dict:
        tot_r = sum(r.replays for r in self.shapes.values())
        return {"shapes": len(self.shapes), "captures": sum(r.captures for r in self.shapes.values()), "replays": tot_r,
                "eager_runs": sum(r.eager_runs for r in self.shapes.values()), "sealed": self.sealed,
                "steady_state_captures": len(self.steady_state_captures),
                "arms": {str(k): {"eager_ms": r.eager_ms, "graph_ms": r.graph_ms, "launches": r.launches,
                                  "launch_bound_share": round(1 - r.graph_ms / r.eager_ms, 3) if r.eager_ms and r.graph_ms else None}
                         for k, r in self.shapes.items() if r.eager_ms is not None}}


def measure_arms(engine, sh, reps: int = 10) -> tuple[float, float]:
    """Times one step shape both ways on the engine's device (CUDA events) and records the arms in its census."""
    import torch
    engine.run(sh)                                       # makes sure the graph exists
    out = []
    for use_graph in (False, True):
        for _ in range(2):
            engine.run(sh, use_graph=use_graph)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            engine.run(sh, use_graph=use_graph)
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) / reps)
    engine.census.arms(sh.key(), out[0], out[1])
    return out[0], out[1]
