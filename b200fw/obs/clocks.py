"""SM-clock and throttle-reason sampling with ``nvidia-smi`` while a timed region runs.

Every benchmark line of this repository carries the median SM clock seen under load and the throttle reasons
that were active, so that a number taken on a power-capped or clock-limited GPU can be told from a clean one
(time x median MHz compares cycles instead of seconds).  Only *reads* the GPU's state."""
from __future__ import annotations

import subprocess
import threading


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc, self._reader = index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._reader = threading.Thread(target=self._read, daemon=True)
            self._reader.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()   # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self._reader is not None:
            self._reader.join(timeout=2)        # lines still in the pipe when the sampler ended count too
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in list(self.samples):
            parts = [p.strip() for p in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


class clocks_during:
    """``with clocks_during(gpu_index) as c: ...`` then ``c.summary`` is the sampler's result dict."""

    def __init__(self, index: int = 0):
        self.sampler, self.summary = ClockSampler(index), None

    def __enter__(self):
        self.sampler.start()
        return self

    def __exit__(self, *exc):
        self.summary = self.sampler.stop()
        return False
