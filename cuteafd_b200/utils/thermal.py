"""Read-only GPU telemetry (clocks, power, throttle reasons) through NVML for `/v1/thermal` and the bench harness.
Nothing here changes a GPU setting.  A fake NVML can be injected for tests.
Reference: shared/thermal.rs:1-21 (throttle seconds by cause)."""
from __future__ import annotations

import time

REASONS = {0x0000000000000004: "sw_power_cap", 0x0000000000000008: "hw_slowdown", 0x0000000000000020: "sw_thermal_slowdown",
           0x0000000000000040: "hw_thermal_slowdown", 0x0000000000000080: "hw_power_brake"}


class ThermalMonitor:
    def __init__(self, nvml=None, index: int = 0):
        self.nvml, self.index = nvml, index
        self.throttle_s: dict = {}
        self._last = None
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
        return {"available": True, "sm_mhz": int(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)),
                "sm_max_mhz": int(n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM)),
                "power_w": n.nvmlDeviceGetPowerUsage(h) / 1000.0, "temp_c": int(n.nvmlDeviceGetTemperature(h, n.NVML_TEMPERATURE_GPU)),
                "reasons": active, "throttle_seconds": dict(self.throttle_s)}


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
