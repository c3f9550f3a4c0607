"""Clock and throttle-reason sampling for the benchmarks (read-only NVML queries)."""
from __future__ import annotations

import statistics
import threading
import time


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU through NVML (read-only queries) from a
    thread of this process, every few milliseconds, while a region runs."""

    PERIOD_S = 0.004

    def __init__(self, index: int):
        self.index, self.samples, self.handle, self.nv = index, [], None, None
        self._stop = threading.Event()
        self.thread = None

    def start(self) -> None:
        try:
            import pynvml as nv
            nv.nvmlInit()
            try:
                import torch
                uuid = str(torch.cuda.get_device_properties(self.index).uuid)
                self.handle = nv.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self.handle = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.nv = nv
        except Exception:
            self.nv = None
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _sample(self) -> None:
        nv = self.nv
        try:
            sm = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
            reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle) if hasattr(
                nv, "nvmlDeviceGetCurrentClocksEventReasons") else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
            try:
                watts = nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
            except Exception:
                watts = None
            self.samples.append((time.monotonic(), sm, int(reasons), watts))
        except Exception:
            pass

    def _run(self) -> None:
        while not self._stop.is_set():
            self._sample()
            time.sleep(self.PERIOD_S)

    def mark_begin(self) -> None:
        self.t0 = time.monotonic()

    def mark_end(self) -> None:
        self.t1 = time.monotonic()

    def window(self, t0: float, t1: float) -> dict:
        """Median SM clock and the throttle reasons seen between two time.monotonic() stamps (the nearest sample
        when the window is shorter than the sampling period). The sampler keeps running."""
        if self.nv is None or not self.samples:
            return {"sm_mhz": None, "reasons": ["nvml unavailable"]}
        masks = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        inside = [s for s in list(self.samples) if t0 <= s[0] <= t1]
        if not inside:
            inside = [min(list(self.samples), key=lambda s: abs(s[0] - (t0 + t1) / 2))]
        reasons = sorted({name for _, _, bits, _ in inside for name, m in masks.items() if bits & m})
        return {"sm_mhz": statistics.median(s[1] for s in inside), "reasons": reasons}

    def stop(self) -> dict:
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        self._stop.set()
        self.thread.join(timeout=2)
        nv = self.nv
        try:
            smax = nv.nvmlDeviceGetMaxClockInfo(self.handle, nv.NVML_CLOCK_SM)
        except Exception:
            smax = None
        masks = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        t0, t1 = getattr(self, "t0", 0.0), getattr(self, "t1", float("inf"))
        sm, reasons, watts = [], set(), []
        for ts, mhz, bits, w in self.samples:
            if ts < t0 or ts > t1:
                continue
            sm.append(mhz)
            if w is not None:
                watts.append(w)
            for name, m in masks.items():
                if bits & m:
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                "sm_max_mhz": smax, "samples": len(sm), "power_w": statistics.median(watts) if watts else None,
                "reasons": sorted(reasons)}
