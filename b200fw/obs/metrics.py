"""Named timers and scalar series with summaries and TensorBoard export
(surface of the reference's MetricsCollector, src/utils/metrics.py:30-203)."""
from __future__ import annotations

import contextlib
import time
from ..compat import kwarg_aliases
from dataclasses import dataclass
from collections import defaultdict
from typing import Dict, List, Optional


@dataclass
class TimerRecord:
    """One finished timer interval (src/utils/metrics.py:15-27); ``MetricsCollector.timer_records`` lists them."""
    name: str
    start_time: float
    end_time: float

    @property
    def duration(self) -> float:
        return self.end_time - self.start_time


class MetricsCollector:
    def __init__(self):
        self.series: Dict[str, List[float]] = defaultdict(list)
        self.steps: Dict[str, List[int]] = defaultdict(list)
        self.timers: Dict[str, List[float]] = defaultdict(list)
        self._open: Dict[str, float] = {}
        self.timer_records: List[TimerRecord] = []
        self._start_time = time.time()

    @kwarg_aliases(key="name")
    def record(self, name: str, value: float, step: Optional[int] = None):
        self.series[name].append(float(value))
        self.steps[name].append(len(self.series[name]) - 1 if step is None else int(step))

    def start_timer(self, name: str):
        self._open[name] = time.perf_counter()

    def stop_timer(self, name: str) -> float:
        t0 = self._open.pop(name, None)
        if t0 is None:
            return 0.0
        now = time.perf_counter()
        dt = now - t0
        self.timers[name].append(dt)
        self.timer_records.append(TimerRecord(name, t0, now))
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

    # ---- the reference's method names (src/utils/metrics.py:103-203) ------------------------------------------
    def record_step(self, comm_time_ms: Optional[float] = None, grad_norm: Optional[float] = None,
                    peak_memory_gb: Optional[float] = None, learning_rate: Optional[float] = None):
        """Record whichever per-step figures are given under their usual names."""
        for k, v in (("comm_time_ms", comm_time_ms), ("grad_norm", grad_norm), ("peak_memory_gb", peak_memory_gb),
                     ("learning_rate", learning_rate)):
            if v is not None:
                self.record(k, v)

    def get_summary(self) -> Dict:
        """``{"total_elapsed_s", "timers": {name: count/total_s/mean_s/min_s/max_s}, "metrics": {key:
        count/mean/min/max/last}, "throughput"}`` (``throughput`` when an ``iteration`` timer was used)."""
        total = self.elapsed_time
        out: Dict = {"total_elapsed_s": total, "timers": {}, "metrics": {}}
        for k, v in self.timers.items():
            if v:
                out["timers"][k] = {"count": len(v), "total_s": sum(v), "mean_s": sum(v) / len(v), "min_s": min(v),
                                    "max_s": max(v)}
        for k, v in self.series.items():
            if v:
                out["metrics"][k] = {"count": len(v), "mean": sum(v) / len(v), "min": min(v), "max": max(v), "last": v[-1]}
        n = len(self.timers.get("iteration", []))
        if n and total > 0:
            out["throughput"] = {"iterations_total": n, "iterations_per_hour": n / total * 3600}
        return out

    def to_tensorboard(self, writer, step: int):
        """Latest value of every series (``metrics/<key>``) and timer (``timers/<name>_duration_s``) at ``step``."""
        for k, v in self.series.items():
            if v:
                writer.add_scalar(f"metrics/{k}", v[-1], step)
        for k, v in self.timers.items():
            if v:
                writer.add_scalar(f"timers/{k}_duration_s", v[-1], step)

    @property
    def elapsed_time(self) -> float:
        return time.time() - self._start_time

    def export_tensorboard(self, writer, prefix: str = ""):
        for k, v in self.series.items():
            for step, val in zip(self.steps[k], v):
                writer.add_scalar(f"{prefix}{k}", val, step)

    def reset(self):
        self.series.clear()
        self.steps.clear()
        self.timers.clear()
        self._open.clear()
        self.timer_records.clear()
        self._start_time = time.time()
