"""CLI, memory ledger, usage store, thermal monitor (fake NVML) - CPU only."""
import json

import pytest

from cuteafd_b200 import cli
from cuteafd_b200.serving.usage import UsageStore
from cuteafd_b200.utils.memory_ledger import BudgetExceeded, Ledger
from cuteafd_b200.utils.thermal import ThermalMonitor
from cuteafd_b200.utils.trace import PhaseProfile, SpeculationTrace


def test_plan_command_results(capsys):
    assert cli.main(["plan", "qwen3-235b", "--layout", "--json"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["supported"] and out["layout"]["fits"] and len(out["layout"]["ranks"]) == 8
    assert cli.main(["plan", "deepseek-v3", "--layout", "--gpus", "1"]) == 2         # does not fit one GPU: a result, not a crash
    assert cli.main(["plan", "/no/such/dir"]) == 2


def test_memory_ledger_scopes_and_budget():
    led = Ledger(budget_bytes=1000)
    with led.scope("weights"):
        led.charge(400, "experts")
        with led.scope("layer0"):
            led.charge(300)
    rep = led.report()
    assert rep["scopes"] == {"weights": 400, "weights/layer0": 300} and rep["total_bytes"] == 700
    with led.scope("kv"), pytest.raises(BudgetExceeded, match="kv"):
        led.charge(400, "pool")


def test_usage_store_rollups_and_redaction():
    u = UsageStore(log_prompts=True, keep_log_hours=1)
    u.record("a", "m", "key1", 100, 20, 64, 30.0, 500.0, "stop", prompt_text="mail me at bob@example.com with sk-abcdefgh1234", now=1_000_000)
    u.record("b", "m", "key1", 50, 10, 0, 10.0, 100.0, "length", now=1_000_100)
    d = u.daily()
    assert d[0]["requests"] == 2 and d[0]["prompt_tokens"] == 150 and d[0]["cache_hit_tokens"] == 64
    assert u.by_key()[0]["tokens"] == 180
    text = u.db.execute("select text from prompt_log").fetchone()[0]
    assert "bob@" not in text and "sk-" not in text
    u.record("c", "m", "k", 1, 1, 0, 1, 1, "stop", prompt_text="x", now=1_000_000 + 7200)
    assert u.db.execute("select count(*) from prompt_log").fetchone()[0] == 1            # older prompt text expired


class FakeNvml:
    NVML_CLOCK_SM, NVML_TEMPERATURE_GPU = 1, 0
    def __init__(self): self.mask = 0
    def nvmlDeviceGetHandleByIndex(self, i): return i
    def nvmlDeviceGetCurrentClocksThrottleReasons(self, h): return self.mask
    def nvmlDeviceGetClockInfo(self, h, k): return 1350
    def nvmlDeviceGetMaxClockInfo(self, h, k): return 1965
    def nvmlDeviceGetPowerUsage(self, h): return 998_000
    def nvmlDeviceGetTemperature(self, h, k): return 61


def test_thermal_monitor_reads_only():
    nv = FakeNvml()
    mon = ThermalMonitor(nvml=nv)
    assert mon.sample()["reasons"] == []
    nv.mask = 0x4 | 0x40
    s = mon.sample()
    assert s["reasons"] == ["sw_power_cap", "hw_thermal_slowdown"] and s["sm_mhz"] == 1350 and s["power_w"] == 998.0
    assert not [m for m in dir(nv) if "Set" in m or "Reset" in m]


def test_trace_helpers(tmp_path):
    p = PhaseProfile()
    with p.phase("router"):
        pass
    assert p.snapshot()["router"]["n"] == 1
    t = SpeculationTrace(str(tmp_path / "spec.jsonl"))
    t.record("r1", 3, 2, 31.0)
    assert json.loads((tmp_path / "spec.jsonl").read_text())["accepted"] == 2
