"""Benchmark history: every measured line (the JSON line of `bench.py`, a baseline card, a micro-benchmark) goes into a SQLite
store; runs can be listed, compared for regressions and rendered as a report (markdown table + an SVG trend of a metric).

    python bench.py --gpus 1 | python -m cuteafd_b200.cli bench-history add --label nightly -
    python -m cuteafd_b200.cli bench-history list --metric decode_tokens_per_s
    python -m cuteafd_b200.cli bench-history compare 12 17
    python -m cuteafd_b200.cli bench-history report --metric decode_tokens_per_s --svg trend.svg

A run is keyed by (metric, config): two lines compare only if they measured the same thing on the same shape - model, batch,
context, parallelism and GPU count - so a change of configuration never shows up as a regression.  Lines whose clock record shows a
thermal slowdown or a pinned clock are stored but flagged, and left out of trends and comparisons unless asked for.

Reference: rust/crates/cuteafd-bench (SQLite history of in-server benchmark runs, JSON / SVG reports, release smoke matrix).
"""
from __future__ import annotations

import hashlib
import json
import sqlite3
import time

REJECT_REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown")


def config_key(line: dict) -> str:
    """Identity of what was measured: metric + the fields of `config` that define the workload + GPU count + dtype."""
    cfg = line.get("config") or {}
    ident = {"metric": line.get("metric"), "n_gpus": line.get("n_gpus"), "dtype": line.get("dtype"),
             "config": {k: cfg.get(k) for k in ("model", "global_batch", "seq_len", "parallelism", "layers", "mtp_draft_tokens") if k in cfg}}
    return hashlib.sha256(json.dumps(ident, sort_keys=True).encode()).hexdigest()[:16]


def flagged(line: dict) -> str | None:
    """Why a line should not be trusted as a performance number, or None."""
    clocks = line.get("clocks") or {}
    bad = [r for r in clocks.get("reasons") or [] if r in REJECT_REASONS]
    if bad:
        return "throttled: " + ", ".join(bad)
    sm, mx = clocks.get("sm_mhz"), clocks.get("sm_max_mhz")
    if sm and mx and sm < 0.8 * mx and not (clocks.get("reasons") or []):
        return f"clocks pinned low ({sm} of {mx} MHz with no reason active)"
    if line.get("unavailable"):
        return "unavailable: " + str(line["unavailable"])
    return None


class BenchHistory:
    def __init__(self, path: str = ":memory:"):
        self.db = sqlite3.connect(path)
        self.db.execute("create table if not exists runs (id integer primary key, at real, label text, commit_id text, metric text, key text, "
                        "value real, unit text, higher_is_better integer, n_gpus integer, flag text, line text)")
        self.db.commit()

    def add(self, line: dict, label: str = "", commit_id: str = "", at: float | None = None) -> int:
        if "metric" not in line or "value" not in line:
            raise ValueError("a benchmark line needs at least `metric` and `value`")
        cur = self.db.execute("insert into runs (at, label, commit_id, metric, key, value, unit, higher_is_better, n_gpus, flag, line) values (?,?,?,?,?,?,?,?,?,?,?)",
                              (at if at is not None else time.time(), label, commit_id, line["metric"], config_key(line), float(line["value"]),
                               line.get("unit", ""), 1 if line.get("higher_is_better", True) else 0, int(line.get("n_gpus") or 1), flagged(line),
                               json.dumps(line, sort_keys=True)))
        self.db.commit()
        return cur.lastrowid

    def _rows(self, where: str = "", args: tuple = ()):
        q = "select id, at, label, commit_id, metric, key, value, unit, higher_is_better, n_gpus, flag, line from runs " + where + " order by at, id"
        names = ("id", "at", "label", "commit", "metric", "key", "value", "unit", "higher_is_better", "n_gpus", "flag", "line")
        return [dict(zip(names, r)) for r in self.db.execute(q, args)]

    def get(self, run_id: int) -> dict:
        rows = self._rows("where id = ?", (run_id,))
        if not rows:
            raise KeyError(f"no run {run_id}")
        return rows[0]

    def list(self, metric: str | None = None, key: str | None = None, include_flagged: bool = True) -> list:
        cond, args = [], []
        if metric:
            cond.append("metric = ?"); args.append(metric)
        if key:
            cond.append("key = ?"); args.append(key)
        if not include_flagged:
            cond.append("flag is null")
        return self._rows(("where " + " and ".join(cond)) if cond else "", tuple(args))

    def compare(self, base_id: int, new_id: int, tolerance: float = 0.02) -> dict:
        """Relative change of `new` against `base`; `verdict` is regression / improvement / same (inside `tolerance`) / incomparable."""
        a, b = self.get(base_id), self.get(new_id)
        out = {"base": a["id"], "new": b["id"], "metric": b["metric"], "base_value": a["value"], "new_value": b["value"], "unit": b["unit"]}
        if a["key"] != b["key"]:
            return {**out, "verdict": "incomparable", "why": "different metric or configuration"}
        if a["flag"] or b["flag"]:
            return {**out, "verdict": "incomparable", "why": a["flag"] or b["flag"]}
        rel = (b["value"] - a["value"]) / a["value"] if a["value"] else 0.0
        better = rel if b["higher_is_better"] else -rel
        out["relative_change"] = round(rel, 4)
        out["verdict"] = "same" if abs(rel) <= tolerance else ("improvement" if better > 0 else "regression")
        return out

    def latest_regressions(self, tolerance: float = 0.02) -> list:
        """For every (metric, configuration): the newest clean run against the best earlier clean run."""
        out = []
        keys = {r["key"] for r in self.list(include_flagged=False)}
        for k in sorted(keys):
            rows = self.list(key=k, include_flagged=False)
            if len(rows) < 2:
                continue
            new, earlier = rows[-1], rows[:-1]
            best = max(earlier, key=lambda r: r["value"]) if new["higher_is_better"] else min(earlier, key=lambda r: r["value"])
            c = self.compare(best["id"], new["id"], tolerance)
            if c["verdict"] == "regression":
                out.append(c)
        return out

    # ---------------------------------------------------------------- reports
    def report_markdown(self, metric: str | None = None) -> str:
        rows = self.list(metric)
        lines = ["| id | when (UTC) | label | commit | metric | gpus | value | unit | note |", "|---|---|---|---|---|---|---|---|---|"]
        for r in rows:
            when = time.strftime("%Y-%m-%d %H:%M", time.gmtime(r["at"]))
            lines.append(f"| {r['id']} | {when} | {r['label']} | {r['commit'][:10]} | {r['metric']} | {r['n_gpus']} | {r['value']:.2f} | {r['unit']} | {r['flag'] or ''} |")
        return "\n".join(lines)

    def report_svg(self, metric: str, key: str | None = None, width: int = 720, height: int = 260) -> str:
        """Trend of a metric over the clean runs of one configuration (the one with the most runs unless `key` names another)."""
        rows = self.list(metric, include_flagged=False)
        if not rows:
            raise ValueError(f"no clean runs of {metric}")
        if key is None:
            counts: dict = {}
            for r in rows:
                counts[r["key"]] = counts.get(r["key"], 0) + 1
            key = max(counts, key=lambda k: (counts[k], k))
        rows = [r for r in rows if r["key"] == key]
        vals = [r["value"] for r in rows]
        lo, hi = min(vals), max(vals)
        pad = (hi - lo) * 0.1 or abs(hi) * 0.05 or 1.0
        lo, hi = lo - pad, hi + pad
        L, R, T, B = 64, 16, 28, 36
        xs = [L + (width - L - R) * (i / max(1, len(rows) - 1)) for i in range(len(rows))]
        ys = [T + (height - T - B) * (1 - (v - lo) / (hi - lo)) for v in vals]
        pts = " ".join(f"{x:.1f},{y:.1f}" for x, y in zip(xs, ys))
        cfg = json.loads(rows[-1]["line"]).get("config") or {}
        title = f"{metric} - {cfg.get('model', '')} x{rows[-1]['n_gpus']} ({rows[-1]['unit']})"
        out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="monospace" font-size="11">',
               f'<rect width="{width}" height="{height}" fill="#111"/>', f'<text x="{L}" y="16" fill="#8bf">{title}</text>',
               f'<line x1="{L}" y1="{height - B}" x2="{width - R}" y2="{height - B}" stroke="#555"/>', f'<line x1="{L}" y1="{T}" x2="{L}" y2="{height - B}" stroke="#555"/>',
               f'<text x="4" y="{T + 4}" fill="#aaa">{hi:.1f}</text>', f'<text x="4" y="{height - B}" fill="#aaa">{lo:.1f}</text>',
               f'<polyline points="{pts}" fill="none" stroke="#4a8" stroke-width="2"/>']
        for x, y, r in zip(xs, ys, rows):
            out.append(f'<circle cx="{x:.1f}" cy="{y:.1f}" r="3" fill="#9c9"><title>#{r["id"]} {r["label"]} {r["value"]:.2f}</title></circle>')
        out.append(f'<text x="{L}" y="{height - 12}" fill="#aaa">run {rows[0]["id"]}</text>')
        out.append(f'<text x="{width - R - 60}" y="{height - 12}" fill="#aaa">run {rows[-1]["id"]}</text></svg>')
        return "\n".join(out)


def smoke_matrix() -> list:
    """The release smoke matrix: every (configuration, GPU count, layout) the benchmarks are expected to run, as command lines.
    `cuteafd bench-history matrix` prints it; an operator (or CI on a GPU box) runs the lines and pipes each result into `add`."""
    rows = []
    tr = "python -m torch.distributed.run --nnodes=1 --nproc-per-node {n} --master-addr 127.0.0.1 --master-port 29500 "
    for n in (1, 2, 4, 8):
        launch = "python " if n == 1 else tr.format(n=n)
        rows.append({"name": f"qwen3-235b decode x{n}", "gpus": n, "cmd": f"{launch}bench.py --gpus {n} --steps 20 --warmup 5"})
    for n, layout in ((8, "split"), (8, "colocated"), (4, "split")):
        rows.append({"name": f"deepseek-v3 decode x{n} {layout}", "gpus": n,
                     "cmd": f"{tr.format(n=n)}bench.py --gpus {n} --config deepseek-v3-plain --layout {layout} --batch-total 64 --context 8192 --steps 10 --warmup 3"})
    rows.append({"name": "deepseek-v3 MTP x8", "gpus": 8,
                 "cmd": f"{tr.format(n=8)}bench.py --gpus 8 --config deepseek-v3-decode --batch-total 64 --context 8192 --steps 10 --warmup 3"})
    for cfg in ("hybrid-gdn-decode", "hybrid-kda-decode"):
        rows.append({"name": f"{cfg} x1", "gpus": 1, "cmd": f"python bench.py --config {cfg} --steps 20 --warmup 5"})
    rows.append({"name": "vision tower x1", "gpus": 1, "cmd": "python -m cuteafd_b200.bench.vision --side 1024 --images 4"})
    rows.append({"name": "gpu tests x1", "gpus": 1, "cmd": "python -m pytest tests -q -m gpu"})
    return rows
