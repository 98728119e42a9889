"""Benchmark history: keys, flags, comparisons, regressions, reports, the CLI (CPU only)."""
import json

from cuteafd_b200.bench.history import BenchHistory, config_key, flagged, smoke_matrix


def line(value, **kw):
    base = {"metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
            "config": {"model": "qwen3-235b-a22b-shape", "global_batch": 16, "seq_len": 4096, "parallelism": "single", "setup_s": 0.8},
            "clocks": {"sm_mhz": 1965.0, "sm_max_mhz": 1965.0, "reasons": []}}
    base.update(kw)
    return base


def test_keys_ignore_what_is_not_the_workload_and_flags_catch_bad_clocks():
    a, b = line(700.0), line(740.0)
    b["config"]["setup_s"] = 3.0
    assert config_key(a) == config_key(b)
    assert config_key(a) != config_key(line(700.0, n_gpus=2)) != config_key(line(700.0, metric="ttft_ms"))
    c = line(700.0)
    c["config"]["seq_len"] = 8192
    assert config_key(c) != config_key(a)
    assert flagged(a) is None
    assert "throttled" in flagged(line(1.0, clocks={"sm_mhz": 1200, "sm_max_mhz": 1965, "reasons": ["hw_thermal_slowdown"]}))
    assert "pinned" in flagged(line(1.0, clocks={"sm_mhz": 1100, "sm_max_mhz": 1965, "reasons": []}))
    assert flagged(line(1.0, clocks={"sm_mhz": 1300, "sm_max_mhz": 1965, "reasons": ["sw_power_cap"]})) is None      # kept and noted, not rejected


def test_compare_regressions_and_reports(tmp_path):
    h = BenchHistory(str(tmp_path / "h.sqlite"))
    r1 = h.add(line(658.7), label="before", commit_id="aaaa", at=1000.0)
    r2 = h.add(line(743.4), label="after", commit_id="bbbb", at=2000.0)
    r3 = h.add(line(600.0, clocks={"sm_mhz": 900, "sm_max_mhz": 1965, "reasons": ["hw_slowdown"]}), label="hot box", at=3000.0)
    r4 = h.add(line(8874.6, n_gpus=8), label="x8", at=3500.0)
    r5 = h.add(line(21.5, metric="ms_per_step", unit="ms", higher_is_better=False), at=3600.0)
    r6 = h.add(line(24.0, metric="ms_per_step", unit="ms", higher_is_better=False), at=3700.0)
    c = h.compare(r1, r2)
    assert c["verdict"] == "improvement" and abs(c["relative_change"] - 0.1286) < 1e-3
    assert h.compare(r2, r1)["verdict"] == "regression" and h.compare(r1, r1)["verdict"] == "same"
    assert h.compare(r2, r3)["verdict"] == "incomparable" and "throttled" in h.compare(r2, r3)["why"]
    assert h.compare(r2, r4)["verdict"] == "incomparable"
    assert h.compare(r5, r6)["verdict"] == "regression"                      # lower is better for a time
    regs = h.latest_regressions()
    assert [r["new"] for r in regs] == [r6]                                  # the throttled run is not a regression of the clean ones
    md = h.report_markdown("decode_tokens_per_s")
    assert md.count("\n") == 5 and "hot box" in md and "throttled" in md and "743.40" in md
    svg = h.report_svg("decode_tokens_per_s")
    assert svg.startswith("<svg") and svg.count("<circle") == 2 and "qwen3-235b" in svg      # the single-GPU configuration: two clean runs
    again = BenchHistory(str(tmp_path / "h.sqlite"))
    assert len(again.list()) == 6 and len(again.list(include_flagged=False)) == 5


def test_cli_add_list_and_matrix(tmp_path, capsys, monkeypatch):
    import io
    import sys

    from cuteafd_b200 import cli
    db = str(tmp_path / "x" / "hist.sqlite")
    monkeypatch.setattr(sys, "stdin", io.StringIO("noise before the line\n" + json.dumps(line(741.66)) + "\n"))
    assert cli.main(["bench-history", "add", "-", "--db", db, "--label", "final"]) == 0
    assert cli.main(["bench-history", "list", "--db", db]) == 0
    out = capsys.readouterr().out
    assert "run 1: decode_tokens_per_s = 741.66" in out and "| final |" in out
    assert cli.main(["bench-history", "regressions", "--db", db]) == 0
    assert cli.main(["bench-history", "matrix"]) == 0
    names = [r["name"] for r in smoke_matrix()]
    assert "qwen3-235b decode x8" in names and any("deepseek-v3" in n for n in names) and all("bench.py" in r["cmd"] or "-m " in r["cmd"] for r in smoke_matrix())
