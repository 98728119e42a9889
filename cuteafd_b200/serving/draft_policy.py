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


# ------------------------------------------------------------------------------------------------------------------
# Online resource-priced policy: verification lengths for ALL requests of a round, chosen jointly.
def concurrency_bucket(requests: int) -> int:
    """Evidence regimes of the cost fit and the calibration: 1, 2-4, 5-8, 9+ requests in a round."""
    return 0 if requests <= 1 else 1 if requests <= 4 else 2 if requests <= 8 else 3


class _Fit:
    """Recursive least squares with exponential forgetting and Huber-weighted residuals around a prior: y ~ theta . x.
    The prior enters as `prior_weight` pseudo-samples, so an unseen regime predicts the prior and a seen one moves away from it."""

    def __init__(self, prior, prior_weight: float = 4.0, decay: float = 0.995, huber: float = 3.0):
        n = len(prior)
        self.theta = [float(p) for p in prior]
        self.P = [[(1.0 / prior_weight if i == j else 0.0) for j in range(n)] for i in range(n)]
        self.decay, self.huber, self.samples, self.scale = decay, huber, 0, 0.0

    def predict(self, x) -> float:
        return sum(t * v for t, v in zip(self.theta, x))

    def update(self, x, y: float):
        err = y - self.predict(x)
        self.scale = abs(err) if self.samples == 0 else 0.95 * self.scale + 0.05 * abs(err)
        w = 1.0 if abs(err) <= self.huber * max(self.scale, 1e-9) else self.huber * self.scale / abs(err)      # outliers count less
        n = len(x)
        Px = [sum(self.P[i][j] * x[j] for j in range(n)) for i in range(n)]
        denom = self.decay / w + sum(x[i] * Px[i] for i in range(n))
        k = [v / denom for v in Px]
        self.theta = [max(0.0, t + ki * err) for t, ki in zip(self.theta, k)]             # costs are non-negative
        self.P = [[(self.P[i][j] - k[i] * Px[j]) / self.decay for j in range(n)] for i in range(n)]
        self.samples += 1


class OnlineDraftPolicy(DraftPolicy):
    """Chooses, each round, how many draft rows every request verifies so that expected committed tokens per predicted round time
    is largest.  A committed token's own row is paid whichever round verifies it, so the choice comes down to fixed plus wasted
    cost per committed token.

    Time model (milliseconds), fitted online per concurrency bucket from the scheduler's own step timings - no offline calibration:
        round = intercept + row_price * rows + mb_price * expert_megabytes        (verification step)
        draft = draft_fixed + draft_per_request * drafting requests               (drafter pass, when any request drafts)
    `expert_megabytes` forecasts routed-expert weight traffic: slice_mb * sum over experts of ceil(routes_e / group_rows), with the
    routes of a not-yet-executed draft row k forecast by the k-th most recent committed token of the same request (averaged over
    shifted windows) and the union taken over all rows of the round - so requests that share experts share their cost.  Without
    route capture the term is zero and the row price absorbs the traffic.

    Acceptance: per draft position, a decayed count of "reached" and "accepted" per bucket (calibration), blended per request with its
    own recent outcomes; a request whose drafts keep failing is skipped and probed again after a few rounds.  Until a bucket has seen
    `warm_rounds` rounds the policy behaves like the simple one (fixed width with cut-off).

    Reference: cuteafd-core/src/draft_policy.rs:1-60 (the policy's contract: maximise committed tokens per predicted lane time, resource
    classes with a per-layer cost and a per-megabyte cost, online fits with forgetting and Huber weights, route forecast from committed
    tokens, concurrency buckets), cuteafd-core/src/simple_draft.rs (cut-off and probing)."""

    HISTORY, WINDOWS = 24, 4

    def __init__(self, max_width: int = 7, *, n_experts: int = 0, top_k: int = 0, slice_mb: float = 0.0, group_rows: int = 16,
                 warm_rounds: int = 12, prior_accept: float = 0.6, prior_ms=(20.0, 0.05, 0.5), prior_draft_ms=(0.5, 0.05),
                 calibration_decay: float = 0.998, explore_skips: int = 8):
        self.max_width, self.n_experts, self.top_k, self.slice_mb, self.group_rows = max_width, n_experts, top_k, slice_mb, group_rows
        self.warm_rounds, self.explore_skips, self.cal_decay = warm_rounds, explore_skips, calibration_decay
        self.round_fit = [_Fit(prior_ms) for _ in range(4)]                  # [intercept, per row, per expert megabyte]
        self.draft_fit = [_Fit(prior_draft_ms) for _ in range(4)]            # [fixed, per drafting request]
        self.cal = [[[prior_accept * 2.0, 2.0] for _ in range(max_width)] for _ in range(4)]      # [accepted, reached] per bucket, position
        self.recent: dict = {}               # rid -> smoothed (accepted / drafted) of its own rounds
        self.skips: dict = defaultdict(int)
        self.routes: dict = defaultdict(lambda: deque(maxlen=self.HISTORY))          # rid -> expert sets of committed tokens, newest last
        self.fallback = SimpleDraftPolicy(min(max_width, 3))
        self.total_drafted = self.total_accepted = self.rounds = 0
        self.last_plan: dict = {}
        self.rel_error = 0.0
        self._pending_outcomes: list = []

    # ---------------------------------------------------------------- inputs from the serving loop
    def observe_routes(self, rid: str, expert_sets: list):
        """Expert ids of each newly committed token of a request (one collection per token), oldest first."""
        for s in expert_sets:
            self.routes[rid].append(frozenset(int(e) for e in s))

    def forget(self, rid: str):
        for d in (self.recent, self.skips, self.routes, self.last_plan):
            d.pop(rid, None)
        self.fallback.hist.pop(rid, None)

    # ---------------------------------------------------------------- forecasts
    def _accept_prob(self, rid: str, bucket: int, pos: int) -> float:
        a, n = self.cal[bucket][pos]
        p = a / n
        own = self.recent.get(rid)
        if own is not None:                   # the request's own recent outcomes shift the calibrated rate
            p = min(0.99, max(0.01, p * (0.5 + own) / (0.5 + self._global_rate(bucket))))
        return p

    def _global_rate(self, bucket: int) -> float:
        a = sum(x[0] for x in self.cal[bucket])
        n = sum(x[1] for x in self.cal[bucket])
        return a / n if n else 0.5

    def _forecast_routes(self, rid: str, k: int) -> list:
        """Expert-set forecasts for the anchor row and k draft rows: row j stands in for the j-th most recent committed token; the
        forecasts of several shifted windows are kept side by side (the traffic estimate averages over them)."""
        h = self.routes.get(rid)
        if not h:
            return []
        hist = list(h)[::-1]
        return [[hist[(j + s) % len(hist)] for j in range(k + 1)] for s in range(min(self.WINDOWS, len(hist)))]

    def expert_megabytes(self, widths: dict) -> float:
        if not self.slice_mb or not self.n_experts:
            return 0.0
        per_window = []
        windows = {rid: self._forecast_routes(rid, w) for rid, w in widths.items()}
        if not any(windows.values()):
            return 0.0
        for s in range(self.WINDOWS):
            counts: dict = defaultdict(int)
            for rid, ws in windows.items():
                if not ws:
                    continue
                for experts in ws[s % len(ws)]:
                    for e in experts:
                        counts[e] += 1
            per_window.append(sum(-(-c // self.group_rows) for c in counts.values()))
        return self.slice_mb * sum(per_window) / len(per_window)

    def predict_ms(self, widths: dict) -> float:
        b = concurrency_bucket(len(widths))
        rows = sum(1 + w for w in widths.values())
        ms = self.round_fit[b].predict((1.0, rows, self.expert_megabytes(widths)))
        drafting = sum(1 for w in widths.values() if w > 0)
        if drafting:
            ms += self.draft_fit[b].predict((1.0, drafting))
        return max(ms, 1e-3)

    def expected_tokens(self, widths: dict) -> float:
        b = concurrency_bucket(len(widths))
        total = 0.0
        for rid, w in widths.items():
            reach, gain = 1.0, 1.0                 # the anchor row always commits one token
            for pos in range(w):
                reach *= self._accept_prob(rid, b, pos)
                gain += reach
            total += gain
        return total

    # ---------------------------------------------------------------- decisions
    def plan_round(self, rids: list, rows_budget: int, room: dict | None = None) -> dict:
        """Draft rows per request for the coming round.  `room[rid]`: tokens the request may still emit beyond the anchor."""
        b = concurrency_bucket(len(rids))
        budget = rows_budget - len(rids)
        if self.round_fit[b].samples < self.warm_rounds:            # not enough evidence in this regime yet: the simple rule
            plan = {}
            for i, rid in enumerate(rids):
                plan[rid] = min(self.fallback.width(rid, budget + 1), (room or {}).get(rid, self.max_width), max(0, budget))
                budget -= plan[rid]
            self.last_plan = dict(plan)
            return plan
        widths = {rid: 0 for rid in rids}
        eligible = []
        for rid in rids:
            own = self.recent.get(rid)
            if own is not None and own < 0.1:                        # drafts of this request keep failing: skip, probe now and then
                self.skips[rid] += 1
                if self.skips[rid] % self.explore_skips:
                    continue
            eligible.append(rid)
        tokens, ms = self.expected_tokens(widths), self.predict_ms(widths)
        while budget > 0:
            best = None
            for rid in eligible:
                if widths[rid] >= min(self.max_width, (room or {}).get(rid, self.max_width)):
                    continue
                trial = dict(widths)
                trial[rid] += 1
                t2, m2 = self.expected_tokens(trial), self.predict_ms(trial)
                if t2 / m2 > tokens / ms and (best is None or t2 / m2 > best[1] / best[2]):
                    best = (rid, t2, m2)
            if best is None:
                break
            widths[best[0]] += 1
            tokens, ms = best[1], best[2]
            budget -= 1
        self.last_plan = dict(widths)
        return widths

    def width(self, rid: str, rows_left: int) -> int:
        """Per-request entry point of the plain policy interface: the planned width when a round was planned, else the simple rule."""
        if rid in self.last_plan:
            return max(0, min(self.last_plan[rid], rows_left - 1))
        return self.fallback.width(rid, rows_left)

    # ---------------------------------------------------------------- evidence
    def observe(self, rid: str, drafted: int, accepted: int):
        self.fallback.observe(rid, drafted, accepted)
        if not drafted:
            return
        self.total_drafted += drafted
        self.total_accepted += accepted
        own = accepted / drafted
        self.recent[rid] = own if rid not in self.recent else 0.5 * self.recent[rid] + 0.5 * own
        if own >= 0.1:
            self.skips[rid] = 0
        self._pending_outcomes.append((drafted, accepted))

    def observe_round(self, n_requests: int, rows: int, step_ms: float, widths: dict | None = None, draft_ms: float | None = None):
        """Timing of the round that was just verified (and of its drafter pass, when measured apart)."""
        b = concurrency_bucket(n_requests)
        mb = self.expert_megabytes(widths) if widths else 0.0
        predicted = self.round_fit[b].predict((1.0, rows, mb))
        self.round_fit[b].update((1.0, float(rows), mb), step_ms)
        if draft_ms is not None and widths:
            drafting = sum(1 for w in widths.values() if w > 0)
            if drafting:
                self.draft_fit[b].update((1.0, float(drafting)), draft_ms)
        if step_ms > 0:
            self.rel_error = 0.9 * self.rel_error + 0.1 * abs(predicted - step_ms) / step_ms
        for drafted, accepted in self._pending_outcomes:              # calibration by position, with forgetting
            for pos in range(min(drafted, self.max_width)):
                if pos <= accepted:
                    c = self.cal[b][pos]
                    c[0], c[1] = c[0] * self.cal_decay + (1.0 if pos < accepted else 0.0), c[1] * self.cal_decay + 1.0
        self._pending_outcomes = []
        self.rounds += 1

    def snapshot(self) -> dict:
        return {"kind": "online-resource-priced", "rounds": self.rounds, "drafted": self.total_drafted, "accepted": self.total_accepted,
                "acceptance": (self.total_accepted / self.total_drafted) if self.total_drafted else None,
                "fit": [{"samples": f.samples, "intercept_ms": round(f.theta[0], 3), "row_ms": round(f.theta[1], 4), "mb_ms": round(f.theta[2], 4)}
                        for f in self.round_fit],
                "per_position": [[round(a / n, 3) for a, n in bucket] for bucket in self.cal], "relative_error": round(self.rel_error, 3)}
