"""Schedule timeline: event tracking, ASCII Gantt chart, Chrome-trace JSON, utilisation statistics and
a two-run comparison (src/profiling/schedule_visualizer.py:79-467)."""
from __future__ import annotations

import contextlib
import json
import time
from dataclasses import dataclass, asdict
from typing import Dict, List, Optional


@dataclass
class TimelineEvent:
    name: str
    category: str   # e.g. forward / backward / comm / optimizer / rollout / sync
    lane: str       # row of the chart: "rank0/compute", "stage1", ...
    start_ms: float
    end_ms: float
    meta: Optional[Dict] = None

    @property
    def duration_ms(self) -> float:
        return self.end_ms - self.start_ms

    # the reference's field names (src/profiling/schedule_visualizer.py:50-76): seconds, a device label, a dict
    @property
    def duration_s(self) -> float:
        return self.duration_ms * 1e-3

    @property
    def start_time(self) -> float:
        return self.start_ms * 1e-3

    @property
    def end_time(self) -> float:
        return self.end_ms * 1e-3

    @property
    def device(self) -> str:
        return self.lane

    @property
    def metadata(self) -> Dict:
        return self.meta or {}


ScheduleEvent = TimelineEvent      # the reference's name for an event record


class ScheduleVisualizer:
    SYMBOLS = {"forward": "F", "backward": "B", "comm": "c", "optimizer": "O", "rollout": "R", "sync": "s", "idle": "."}

    def __init__(self):
        self.events: List[TimelineEvent] = []
        self._open: Dict = {}
        self._t0 = time.perf_counter()

    def now_ms(self) -> float:
        return (time.perf_counter() - self._t0) * 1e3

    def add_event(self, name, category, lane="GPU:0", start_ms=None, end_ms=None, meta=None, device=None, **metadata):
        """``add_event(name, category, lane, start_ms, end_ms, meta)``; the reference's form is
        ``add_event(name, start_time, end_time, device="GPU:0", **metadata)`` in seconds
        (src/profiling/schedule_visualizer.py:171-188): numbers in second and third place select it."""
        if isinstance(category, (int, float)) and not isinstance(category, bool):
            start_s, end_s = float(category), float(lane)
            dev = device if device is not None else (start_ms if isinstance(start_ms, str) else "GPU:0")
            self.events.append(TimelineEvent(name, self._STAGE_CATEGORY.get(name, name), dev, start_s * 1e3, end_s * 1e3,
                                             metadata or meta))
            return
        self.events.append(TimelineEvent(name, category, device if device is not None else lane, start_ms, end_ms,
                                         meta if meta is not None else (metadata or None)))

    @contextlib.contextmanager
    def track(self, name: str, category: Optional[str] = None, lane: Optional[str] = None, meta=None, device=None,
              **metadata):
        """``with viz.track(name, category, lane)``; or the reference's ``track(name, device="GPU:0", **metadata)``
        (src/profiling/schedule_visualizer.py:141-169): without a known category in second place the stage name decides
        the category and the second argument (or ``device=``) is the lane."""
        if category is not None and category not in self.SYMBOLS and category not in self._STAGE_CATEGORY.values() \
                and lane is None and device is None:
            device, category = category, None              # track("training", "GPU:1")
        if category is None:
            category = self._STAGE_CATEGORY.get(name, name)
            lane = device if device is not None else (lane if lane is not None else "GPU:0")
        else:
            lane = device if device is not None else (lane if lane is not None else "main")
        s = self.now_ms()
        try:
            yield
        finally:
            self.add_event(name, category, lane, s, self.now_ms(), meta if meta is not None else (metadata or None))

    def lanes(self) -> List[str]:
        seen = []
        for e in self.events:
            if e.lane not in seen:
                seen.append(e.lane)
        return seen

    def ascii_gantt(self, width: int = 100) -> str:
        if not self.events:
            return "(no events)"
        t0 = min(e.start_ms for e in self.events)
        t1 = max(e.end_ms for e in self.events)
        span = max(t1 - t0, 1e-9)
        rows = []
        label_w = max(len(l) for l in self.lanes())
        for lane in self.lanes():
            row = [self.SYMBOLS["idle"]] * width
            for e in (x for x in self.events if x.lane == lane):
                a = int((e.start_ms - t0) / span * (width - 1))
                b = max(a, int((e.end_ms - t0) / span * (width - 1)))
                sym = self.SYMBOLS.get(e.category, e.category[:1].upper() or "?")
                for i in range(a, b + 1):
                    row[i] = sym
            rows.append(f"{lane.ljust(label_w)} |{''.join(row)}|")
        rows.append(f"{' ' * label_w}  0 ms{' ' * (width - 14)}{span:8.2f} ms")
        return "\n".join(rows)

    def chrome_trace(self) -> Dict:
        lanes = {l: i for i, l in enumerate(self.lanes())}
        ev = [{"name": e.name, "cat": e.category, "ph": "X", "ts": e.start_ms * 1e3, "dur": e.duration_ms * 1e3,
               "pid": 0, "tid": lanes[e.lane], "args": e.meta or {}} for e in self.events]
        ev += [{"name": "thread_name", "ph": "M", "pid": 0, "tid": i, "args": {"name": l}} for l, i in lanes.items()]
        return {"traceEvents": ev, "displayTimeUnit": "ms"}

    def save_chrome_trace(self, path: str):
        with open(path, "w") as f:
            json.dump(self.chrome_trace(), f)

    def utilisation(self) -> Dict[str, Dict[str, float]]:
        if not self.events:
            return {}
        t0 = min(e.start_ms for e in self.events)
        t1 = max(e.end_ms for e in self.events)
        span = max(t1 - t0, 1e-9)
        out = {}
        for lane in self.lanes():
            by_cat: Dict[str, float] = {}
            busy = 0.0
            for e in (x for x in self.events if x.lane == lane):
                by_cat[e.category] = by_cat.get(e.category, 0.0) + e.duration_ms
                busy += e.duration_ms
            out[lane] = {"busy_ms": busy, "span_ms": span, "utilisation": min(1.0, busy / span),
                         "bubble_ratio": max(0.0, 1.0 - busy / span), **{f"{k}_ms": v for k, v in by_cat.items()}}
        return out

    def compare(a: "ScheduleVisualizer", b: "ScheduleVisualizer", names=("a", "b")) -> Dict:     # noqa: N805
        """``ScheduleVisualizer.compare(a, b)`` or, as the reference calls it, ``a.compare(b)``."""
        ua, ub = a.utilisation(), b.utilisation()
        span = lambda u: max((v["span_ms"] for v in u.values()), default=0.0)
        mean_u = lambda u: sum(v["utilisation"] for v in u.values()) / max(1, len(u))
        return {names[0]: {"span_ms": span(ua), "mean_utilisation": mean_u(ua)},
                names[1]: {"span_ms": span(ub), "mean_utilisation": mean_u(ub)},
                "speedup": span(ua) / span(ub) if span(ub) > 0 else 0.0}

    def to_rows(self) -> List[Dict]:
        return [asdict(e) for e in self.events]

    # ---- the reference's method names (src/profiling/schedule_visualizer.py:103-467): events are named after the
    # orchestrator stage ("training", "inference", "sync", ...) and live on a device lane ("GPU:0") ----------------
    _STAGE_CATEGORY = {"training": "backward", "inference": "rollout", "inferring": "rollout", "sync": "sync",
                       "syncing": "sync", "sleep": "idle", "wake": "idle", "idle": "idle", "forward": "forward",
                       "backward": "backward", "comm": "comm", "optimizer": "optimizer", "rewarding": "optimizer"}

    def begin_event(self, name: str, device: str = "GPU:0", **metadata):
        self._open[(name, device)] = (self.now_ms(), metadata or None)

    def end_event(self, name: str, device: str = "GPU:0"):
        """Close the matching ``begin_event`` (ignored when there is none)."""
        start = self._open.pop((name, device), None)
        if start is not None:
            self.add_event(name, self._STAGE_CATEGORY.get(name, name), device, start[0], self.now_ms(), start[1])

    def render_ascii(self, width: int = 80) -> str:
        return self.ascii_gantt(width)

    def render_json(self) -> str:
        """Chrome-trace JSON text (load in chrome://tracing or Perfetto)."""
        return json.dumps(self.chrome_trace())

    def get_utilization_stats(self) -> dict:
        u = self.utilisation()
        busy = sum(v["busy_ms"] for v in u.values())
        span = max((v["span_ms"] for v in u.values()), default=0.0)
        by_name: Dict[str, float] = {}
        for e in self.events:
            by_name[e.name] = by_name.get(e.name, 0.0) + e.duration_ms
        return {"total_time_ms": span, "busy_time_ms": busy, "devices": u,
                "utilization": busy / (span * len(u)) if span > 0 and u else 0.0,
                "stage_time_ms": by_name, "stage_ratio": {k: v / busy for k, v in by_name.items()} if busy > 0 else {}}

    def report(self) -> str:
        st = self.get_utilization_stats()
        lines = ["== schedule ==", self.ascii_gantt(80),
                 f"span {st['total_time_ms']:.2f} ms, mean utilisation {100 * st['utilization']:.1f} %"]
        lines += [f"  {k:16s} {v:10.2f} ms  {100 * st['stage_ratio'].get(k, 0.0):5.1f} %"
                  for k, v in sorted(st["stage_time_ms"].items(), key=lambda kv: -kv[1])]
        return "\n".join(lines)

    def reset(self):
        self.events.clear()
        self._open.clear()
        self._t0 = time.perf_counter()

