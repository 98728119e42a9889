"""Draft-width policies for speculative decoding.

`SimpleDraftPolicy`: fixed maximum width with a per-request acceptance cut-off (stop drafting for a request whose
recent drafts are mostly rejected, probe again later).
`ResourcePricedPolicy`: prices each candidate width by the expected tokens gained against the extra verify-row
cost measured from recent step times; it picks the width with the best expected tokens per millisecond and
respects the shared 64-row verify budget.
Reference: cuteafd-core/src/simple_draft.rs:1-37, draft_policy.rs:1-40 (resource-priced), serve.rs:404-426.
"""
from __future__ import annotations

from collections import defaultdict, deque


class DraftPolicy:
    def width(self, rid: str, rows_left: int) -> int: ...
    def observe(self, rid: str, drafted: int, accepted: int): ...
    def snapshot(self) -> dict: ...


class SimpleDraftPolicy(DraftPolicy):
    def __init__(self, max_width: int = 3, cutoff: float = 0.2, window: int = 8, probe_every: int = 16):
        self.max_width, self.cutoff, self.window, self.probe_every = max_width, cutoff, window, probe_every
        self.hist = defaultdict(lambda: deque(maxlen=window))
        self.skipped = defaultdict(int)
        self.total_drafted = self.total_accepted = 0

    def width(self, rid: str, rows_left: int) -> int:
        h = self.hist[rid]
        if len(h) >= 4:
            d, a = sum(x for x, _ in h), sum(y for _, y in h)
            if d and a / d < self.cutoff:
                self.skipped[rid] += 1
                if self.skipped[rid] % self.probe_every:
                    return 0
        return max(0, min(self.max_width, rows_left - 1))

    def observe(self, rid: str, drafted: int, accepted: int):
        if drafted:
            self.hist[rid].append((drafted, accepted))
            self.total_drafted += drafted
            self.total_accepted += accepted

    def snapshot(self) -> dict:
        return {"kind": "simple", "max_width": self.max_width, "drafted": self.total_drafted, "accepted": self.total_accepted,
                "acceptance": (self.total_accepted / self.total_drafted) if self.total_drafted else None}


class ResourcePricedPolicy(DraftPolicy):
    """Expected gain of width w with per-position acceptance p_i: sum_{j<=w} prod_{i<=j} p_i tokens, at a cost of
    `row_ms` per extra verify row plus `draft_ms` per drafted token.  Chooses argmax (1 + gain) / (base_ms + cost)."""

    def __init__(self, max_width: int = 7, base_ms: float = 30.0, row_ms: float = 0.3, draft_ms: float = 0.5, prior: float = 0.6):
        self.max_width, self.base_ms, self.row_ms, self.draft_ms = max_width, base_ms, row_ms, draft_ms
        self.acc = [[prior * 4, 4.0] for _ in range(max_width)]      # [accepted, tried] per draft position (with a prior)
        self.total_drafted = self.total_accepted = 0

    def set_costs(self, base_ms: float | None = None, row_ms: float | None = None, draft_ms: float | None = None):
        self.base_ms = base_ms if base_ms is not None else self.base_ms
        self.row_ms = row_ms if row_ms is not None else self.row_ms
        self.draft_ms = draft_ms if draft_ms is not None else self.draft_ms

    def width(self, rid: str, rows_left: int) -> int:
        best_w, best_rate, gain, reach = 0, 1.0 / self.base_ms, 0.0, 1.0
        for w in range(1, min(self.max_width, max(0, rows_left - 1)) + 1):
            a, n = self.acc[w - 1]
            reach *= a / n
            gain += reach
            rate = (1.0 + gain) / (self.base_ms + w * (self.row_ms + self.draft_ms))
            if rate > best_rate:
                best_w, best_rate = w, rate
        return best_w

    def observe(self, rid: str, drafted: int, accepted: int):
        for i in range(min(drafted, self.max_width)):
            if i <= accepted:                      # position i was reached only if all earlier drafts were accepted
                self.acc[i][1] += 1
                if i < accepted:
                    self.acc[i][0] += 1
        self.total_drafted += drafted
        self.total_accepted += accepted

    def snapshot(self) -> dict:
        return {"kind": "resource-priced", "per_position": [round(a / n, 3) for a, n in self.acc], "drafted": self.total_drafted,
                "accepted": self.total_accepted, "base_ms": self.base_ms, "row_ms": self.row_ms}
