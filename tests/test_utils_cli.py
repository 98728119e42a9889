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


def test_throttle_report_windows_and_verdicts():
    from cuteafd_b200.utils.thermal import ThrottleReport
    rep = ThrottleReport(keep=100)
    for t in range(10):                          # ten clean seconds at full clock
        rep.push(100 + t, sm_mhz=1965, sm_max_mhz=1965, power_w=600.0, temp_c=55, util_pct=95)
    for t in range(10, 16):                      # six seconds under the power cap
        rep.push(100 + t, sm_mhz=1350, sm_max_mhz=1965, power_w=1000.0, temp_c=64, util_pct=99, reasons=("sw_power_cap",))
    rep.push(116, sm_mhz=900, sm_max_mhz=1965, power_w=700.0, temp_c=88, util_pct=99, reasons=("hw_thermal_slowdown", "sw_power_cap"))
    whole = rep.window(0)
    assert whole["samples"] == 17 and whole["seconds"] == 16 and whole["verdict"] == "thermal"
    assert whole["throttle_seconds"] == {"sw_power_cap": 7.0, "hw_thermal_slowdown": 1.0} and whole["reason_share"]["sw_power_cap"] == round(7 / 17, 3)
    assert whole["sm_mhz_busy"] == {"min": 900, "median": 1965, "max": 1965} and whole["temp_c"]["max"] == 88
    assert rep.window(100, 109)["verdict"] == "clean" and rep.window(110, 115)["verdict"] == "power_capped"
    assert rep.window(1000) == {"samples": 0}
    pinned = ThrottleReport()
    for t in range(5):
        pinned.push(t, sm_mhz=1100, sm_max_mhz=1965, util_pct=98)
    assert pinned.window(0)["verdict"] == "clocks_pinned_low"        # slow under load with no reason active: a leftover clock lock
    idle = ThrottleReport()
    for t in range(5):
        idle.push(t, sm_mhz=300, sm_max_mhz=1965, util_pct=2)
    assert idle.window(0)["verdict"] == "clean" and idle.window(0)["sm_mhz_busy"] is None
    small = ThrottleReport(keep=3)
    for t in range(10):
        small.push(t)
    assert small.window(0)["samples"] == 3


def test_thermal_monitor_feeds_the_report_and_the_sampler_only_reads():
    import time as _t
    nv = FakeNvml()
    mon = ThermalMonitor(nvml=nv)
    mon.sample()
    nv.mask = 0x4
    mon.sample()
    s = mon.summary(windows=(60,))
    assert s["now"]["reasons"] == ["sw_power_cap"] and s["windows"]["60s"]["samples"] == 3 and s["windows"]["60s"]["verdict"] == "power_capped"
    mon.start(hz=200)
    _t.sleep(0.1)
    mon.stop()
    assert len(mon.report.ring) > 5 and mon._thread is None


def test_run_detach_stop_and_restart(tmp_path):
    """Operator lifecycle: `run --detach` starts the configured command as its own process group and records the pid, `stop` ends
    exactly that group, `--restart` replaces it."""
    import socket
    import time as _t
    import urllib.request

    from cuteafd_b200 import cli
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    cfg = tmp_path / "demo.config"
    cfg.write_text(f"COMMAND=gateway\nLISTEN=127.0.0.1:{port}\n")          # the CPU stand-in server: no GPU, no model
    pidfile, log = str(tmp_path / "run" / "demo.pid"), str(tmp_path / "demo.log")
    assert cli.main(["run", "--config", str(cfg), "--dry-run"]) == 0
    assert cli.main(["stop", "--pidfile", pidfile]) == 0                       # nothing to stop is not an error
    assert cli.main(["run", "--config", str(cfg), "--detach", "--pidfile", pidfile, "--log", log]) == 0
    pid = int(open(pidfile).read())
    up = False
    for _ in range(200):
        try:
            up = urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=0.5).status == 200
            break
        except OSError:
            _t.sleep(0.1)
    assert up, open(log).read()[-2000:]
    assert cli.main(["run", "--config", str(cfg), "--detach", "--pidfile", pidfile]) == 1        # refuses a second copy
    assert cli.main(["run", "--config", str(cfg), "--detach", "--restart", "--pidfile", pidfile, "--log", log, "--stop-timeout", "10"]) == 0
    pid2 = int(open(pidfile).read())
    assert pid2 != pid and not cli._pid_alive(pid)
    assert cli.main(["stop", "--pidfile", pidfile, "--timeout", "10"]) == 0
    assert not cli._pid_alive(pid2) and not (tmp_path / "run" / "demo.pid").exists()
