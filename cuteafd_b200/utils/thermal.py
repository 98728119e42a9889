"""Read-only GPU telemetry (clocks, power, throttle reasons) through NVML for `/v1/thermal` and the bench harness.
Nothing here changes a GPU setting.  A fake NVML can be injected for tests.
Reference: shared/thermal.rs:1-21 (throttle seconds by cause)."""
from __future__ import annotations

import time

REASONS = {0x0000000000000004: "sw_power_cap", 0x0000000000000008: "hw_slowdown", 0x0000000000000020: "sw_thermal_slowdown",
           0x0000000000000040: "hw_thermal_slowdown", 0x0000000000000080: "hw_power_brake"}


class ThrottleReport:
    """A ring of readings of one GPU and window summaries over it: whether, why and how much a stretch of time was throttled -
    seconds and share of samples per clock-event reason, SM clock while busy, temperature, power.  Nothing here touches a device: a
    sampler pushes plain readings (reference: cuteafd-core/src/thermal.rs:1-30, the process-wide ring behind `/v1/thermal` and the
    per-phase throttle notes of the bench)."""

    KEEP = 2 * 3600          # readings kept (two hours at one per second); longer windows are summarised over what remains
    BUSY_PCT = 50            # a reading counts as busy at or above this utilisation

    def __init__(self, keep: int | None = None):
        from collections import deque
        self.ring = deque(maxlen=keep or self.KEEP)

    def push(self, t: float, *, sm_mhz=None, sm_max_mhz=None, power_w=None, temp_c=None, util_pct=None, reasons=()):
        self.ring.append((float(t), sm_mhz, sm_max_mhz, power_w, temp_c, util_pct, tuple(reasons)))

    def window(self, since: float, until: float | None = None) -> dict:
        """Summary of the readings with since <= t <= until (until: the newest reading)."""
        rows = [r for r in self.ring if r[0] >= since and (until is None or r[0] <= until)]
        if not rows:
            return {"samples": 0}
        secs: dict = {}
        share: dict = {}
        for prev, cur in zip(rows, rows[1:]):               # a reason active in a reading is charged the interval that led to it
            for name in cur[6]:
                secs[name] = secs.get(name, 0.0) + (cur[0] - prev[0])
        for r in rows:
            for name in r[6]:
                share[name] = share.get(name, 0) + 1

        def stats(vals):
            vals = sorted(v for v in vals if v is not None)
            return None if not vals else {"min": vals[0], "median": vals[len(vals) // 2], "max": vals[-1]}
        busy = [r for r in rows if r[5] is None or r[5] >= self.BUSY_PCT]
        out = {"samples": len(rows), "seconds": round(rows[-1][0] - rows[0][0], 3),
               "throttle_seconds": {k: round(v, 3) for k, v in secs.items()}, "reason_share": {k: round(v / len(rows), 3) for k, v in share.items()},
               "sm_mhz_busy": stats(r[1] for r in busy), "sm_max_mhz": next((r[2] for r in reversed(rows) if r[2] is not None), None),
               "temp_c": stats(r[4] for r in rows), "power_w": stats(r[3] for r in rows)}
        hot = {"hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"} & set(share)
        clk, mx = out["sm_mhz_busy"], out["sm_max_mhz"]
        pinned = bool(clk and mx and clk["median"] < 0.8 * mx and not share)          # slow with no reason active: a leftover clock lock
        out["verdict"] = "thermal" if hot else ("clocks_pinned_low" if pinned else ("power_capped" if "sw_power_cap" in share else "clean"))
        return out


class ThermalMonitor:
    def __init__(self, nvml=None, index: int = 0):
        self.nvml, self.index = nvml, index
        self.throttle_s: dict = {}
        self._last = None
        self.report = ThrottleReport()
        self._thread = self._stop = None
        if self.nvml is None:
            try:
                import pynvml
                pynvml.nvmlInit()
                self.nvml = pynvml
            except Exception:
                self.nvml = None

    def sample(self) -> dict:
        if self.nvml is None:
            return {"available": False}
        n = self.nvml
        h = n.nvmlDeviceGetHandleByIndex(self.index)
        now = time.time()
        mask = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(h))
        active = [name for bit, name in REASONS.items() if mask & bit]
        if self._last is not None:
            for name in active:
                self.throttle_s[name] = self.throttle_s.get(name, 0.0) + (now - self._last)
        self._last = now
        out = {"available": True, "sm_mhz": int(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)),
               "sm_max_mhz": int(n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM)),
               "power_w": n.nvmlDeviceGetPowerUsage(h) / 1000.0, "temp_c": int(n.nvmlDeviceGetTemperature(h, n.NVML_TEMPERATURE_GPU)),
               "reasons": active, "throttle_seconds": dict(self.throttle_s)}
        util = None
        try:
            util = int(n.nvmlDeviceGetUtilizationRates(h).gpu)
        except Exception:
            pass
        self.report.push(now, sm_mhz=out["sm_mhz"], sm_max_mhz=out["sm_max_mhz"], power_w=out["power_w"], temp_c=out["temp_c"], util_pct=util,
                         reasons=active)
        return out

    def summary(self, windows=(60, 600, 7200)) -> dict:
        """The newest reading plus window summaries (what `/v1/thermal` serves and a bench attaches to a measured phase)."""
        now = time.time()
        return {"now": self.sample(), "windows": {f"{w}s": self.report.window(now - w) for w in windows}}

    def start(self, hz: float = 1.0):
        """Background sampler (reads only); `stop()` ends it."""
        import threading
        if self._thread is not None or self.nvml is None:
            return self
        self._stop = threading.Event()

        def loop():
            while not self._stop.wait(1.0 / hz):
                try:
                    self.sample()
                except Exception:
                    pass
        self._thread = threading.Thread(target=loop, name="thermal-sampler", daemon=True)
        self._thread.start()
        return self

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            self._thread = None


def fabric_snapshot(nvml=None) -> dict:
    """Read-only view of the NVLink fabric for `/v1/fabric`: GPUs, which pairs can reach each other's memory, and the
    NVLink link states NVML reports.  Nothing is changed on any GPU.  (Reference: `/v1/fabric` reports port traffic of the
    RDMA fabric, cuteafd-api/src/openai.rs:340-347; on an NVSwitch node the fabric is NVLink.)"""
    out: dict = {"available": False}
    try:
        import torch
        n = torch.cuda.device_count()
    except Exception:
        return out
    if n == 0:
        return out
    out = {"available": True, "gpus": n,
           "peer_access": [[bool(i == j or torch.cuda.can_device_access_peer(i, j)) for j in range(n)] for i in range(n)]}
    try:
        if nvml is None:
            import pynvml as nvml
            nvml.nvmlInit()
        links = []
        for i in range(n):
            h = nvml.nvmlDeviceGetHandleByIndex(i)
            up = 0
            for l in range(18):
                try:
                    up += 1 if nvml.nvmlDeviceGetNvLinkState(h, l) else 0
                except Exception:
                    break
            links.append(up)
        out["nvlink_links_up"] = links
    except Exception:
        pass
    return out
