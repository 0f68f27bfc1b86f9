"""Named timers and scalar series with summaries and TensorBoard export
(surface of the reference's MetricsCollector, src/utils/metrics.py:30-203)."""
from __future__ import annotations

import contextlib
import time
from collections import defaultdict
from typing import Dict, List, Optional


class MetricsCollector:
    def __init__(self):
        self.series: Dict[str, List[float]] = defaultdict(list)
        self.steps: Dict[str, List[int]] = defaultdict(list)
        self.timers: Dict[str, List[float]] = defaultdict(list)
        self._open: Dict[str, float] = {}

    def record(self, name: str, value: float, step: Optional[int] = None):
        self.series[name].append(float(value))
        self.steps[name].append(len(self.series[name]) - 1 if step is None else int(step))

    def start_timer(self, name: str):
        self._open[name] = time.perf_counter()

    def stop_timer(self, name: str) -> float:
        t0 = self._open.pop(name, None)
        if t0 is None:
            return 0.0
        dt = time.perf_counter() - t0
        self.timers[name].append(dt)
        return dt

    @contextlib.contextmanager
    def timer(self, name: str):
        self.start_timer(name)
        try:
            yield
        finally:
            self.stop_timer(name)

    def get_latest(self, name: str, default: float = 0.0) -> float:
        s = self.series.get(name)
        return s[-1] if s else default

    def get_average(self, name: str, last_n: Optional[int] = None) -> float:
        s = self.series.get(name) or self.timers.get(name)
        if not s:
            return 0.0
        s = s[-last_n:] if last_n else s
        return sum(s) / len(s)

    def summary(self) -> Dict[str, Dict[str, float]]:
        out = {}
        for group in (self.series, self.timers):
            for k, v in group.items():
                if v:
                    out[k] = {"count": len(v), "mean": sum(v) / len(v), "min": min(v), "max": max(v),
                              "last": v[-1], "total": sum(v)}
        return out

    def export_tensorboard(self, writer, prefix: str = ""):
        for k, v in self.series.items():
            for step, val in zip(self.steps[k], v):
                writer.add_scalar(f"{prefix}{k}", val, step)

    def reset(self):
        self.series.clear()
        self.steps.clear()
        self.timers.clear()
        self._open.clear()
