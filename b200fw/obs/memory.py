"""Memory snapshots, static estimates, per-layer peaks and reports; utilisation-threshold manager.

Surface of the reference's MemoryProfiler / MemoryBreakdown / MemoryReport
(src/utils/memory_profiler.py:16-712) and MemoryManager (src/utils/memory_manager.py:9-100).
Everything degrades to zeros on a CPU-only machine.
"""
from __future__ import annotations

import json
import time
from dataclasses import dataclass, field, asdict
from typing import Any, Dict, List, Optional

import torch

GB = 1024 ** 3


@dataclass
class MemorySnapshot:
    tag: str
    timestamp: float
    allocated_gb: float
    reserved_gb: float
    peak_allocated_gb: float
    peak_reserved_gb: float
    free_gb: float = 0.0
    total_gb: float = 0.0


@dataclass
class MemoryBreakdown:
    """Static estimate of one rank's training memory (GB)."""
    params_gb: float = 0.0
    grads_gb: float = 0.0
    optimizer_gb: float = 0.0
    activations_gb: float = 0.0
    logits_gb: float = 0.0
    total_gb: float = 0.0

    @classmethod
    def estimate(cls, num_params: int, trainable_params: Optional[int] = None, param_bytes: int = 2,
                 tp: int = 1, pp: int = 1, dp: int = 1, zero_stage: int = 1, batch_tokens: int = 0,
                 hidden: int = 0, layers: int = 0, vocab: int = 0, intermediate: int = 0,
                 grad_checkpoint: bool = False, fused_loss: bool = True) -> "MemoryBreakdown":
        trainable = num_params if trainable_params is None else trainable_params
        per_rank = num_params / (tp * pp)
        tr_rank = trainable / (tp * pp)
        params = per_rank * param_bytes / (dp if zero_stage >= 3 else 1)
        grads = tr_rank * param_bytes / (dp if zero_stage >= 2 else 1)
        opt = tr_rank * 12 / (dp if zero_stage >= 1 else 1)
        per_layer = batch_tokens * (hidden * (2 if grad_checkpoint else 10) + (0 if grad_checkpoint else 3 * intermediate / tp)) * 2
        acts = per_layer * layers / pp
        logits = (min(batch_tokens, 4096) if fused_loss else batch_tokens) * vocab * (2 if fused_loss else 6)
        b = cls(params / GB, grads / GB, opt / GB, acts / GB, logits / GB)
        b.total_gb = b.params_gb + b.grads_gb + b.optimizer_gb + b.activations_gb + b.logits_gb
        return b


class MemoryProfiler:
    def __init__(self, device: Optional[torch.device] = None, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self.device = device
        self.snapshots: List[MemorySnapshot] = []
        self.layer_peaks: Dict[str, float] = {}
        self._hooks = []
        self.phase_peaks: Dict[str, float] = {}

    def snapshot(self, tag: str) -> MemorySnapshot:
        if self.enabled:
            free, total = torch.cuda.mem_get_info(self.device)
            s = MemorySnapshot(tag, time.time(), torch.cuda.memory_allocated(self.device) / GB,
                               torch.cuda.memory_reserved(self.device) / GB,
                               torch.cuda.max_memory_allocated(self.device) / GB,
                               torch.cuda.max_memory_reserved(self.device) / GB, free / GB, total / GB)
        else:
            s = MemorySnapshot(tag, time.time(), 0.0, 0.0, 0.0, 0.0)
        self.snapshots.append(s)
        return s

    def reset_peak(self):
        if self.enabled:
            torch.cuda.reset_peak_memory_stats(self.device)

    def mark_phase(self, name: str):
        """Record the peak since the last reset under ``name`` (forward / backward / step)."""
        if self.enabled:
            self.phase_peaks[name] = torch.cuda.max_memory_allocated(self.device) / GB
            torch.cuda.reset_peak_memory_stats(self.device)
        else:
            self.phase_peaks[name] = 0.0

    def attach_layer_hooks(self, model: torch.nn.Module, depth_filter=lambda n: n.count(".") <= 1):
        def make(name):
            def hook(_m, _i, _o):
                if self.enabled:
                    cur = torch.cuda.memory_allocated(self.device) / GB
                    self.layer_peaks[name] = max(self.layer_peaks.get(name, 0.0), cur)
            return hook
        for name, mod in model.named_modules():
            if name and depth_filter(name):
                self._hooks.append(mod.register_forward_hook(make(name)))

    def detach_hooks(self):
        for h in self._hooks:
            h.remove()
        self._hooks.clear()

    def timeline(self) -> List[Dict[str, Any]]:
        return [asdict(s) for s in self.snapshots]


@dataclass
class MemoryReport:
    breakdown: Optional[MemoryBreakdown] = None
    snapshots: List[Dict[str, Any]] = field(default_factory=list)
    phase_peaks: Dict[str, float] = field(default_factory=dict)
    layer_peaks: Dict[str, float] = field(default_factory=dict)
    optimizer_bytes: Dict[str, int] = field(default_factory=dict)
    notes: List[str] = field(default_factory=list)

    @classmethod
    def from_profiler(cls, prof: MemoryProfiler, breakdown: Optional[MemoryBreakdown] = None,
                      optimizer_bytes: Optional[Dict[str, int]] = None) -> "MemoryReport":
        return cls(breakdown, prof.timeline(), dict(prof.phase_peaks), dict(prof.layer_peaks),
                   dict(optimizer_bytes or {}))

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        return d

    def save(self, path: str):
        with open(path, "w") as f:
            json.dump(self.to_dict(), f, indent=2)

    def to_text(self) -> str:
        lines = ["== memory report =="]
        if self.breakdown:
            b = self.breakdown
            lines.append(f"static estimate: params {b.params_gb:.2f} grads {b.grads_gb:.2f} optimizer {b.optimizer_gb:.2f} "
                         f"activations {b.activations_gb:.2f} logits {b.logits_gb:.2f} total {b.total_gb:.2f} GB")
        for k, v in self.phase_peaks.items():
            lines.append(f"peak[{k}] = {v:.2f} GB")
        for s in self.snapshots[-5:]:
            lines.append(f"{s['tag']}: allocated {s['allocated_gb']:.2f} reserved {s['reserved_gb']:.2f} peak {s['peak_allocated_gb']:.2f} GB")
        return "\n".join(lines)


class MemoryManager:
    """Watches utilisation; above ``warn`` it logs, above ``critical`` it empties the caching
    allocator; can hold back a reserve block that is released when an OOM is being handled."""

    def __init__(self, warn: float = 0.85, critical: float = 0.95, reserve_mb: int = 0,
                 device: Optional[torch.device] = None):
        self.warn, self.critical, self.device = warn, critical, device
        self.enabled = torch.cuda.is_available()
        self._reserve = None
        self.events: List[str] = []
        if self.enabled and reserve_mb > 0:
            self._reserve = torch.empty(reserve_mb * 1024 * 1024, dtype=torch.uint8, device=device or "cuda")

    def utilisation(self) -> float:
        if not self.enabled:
            return 0.0
        free, total = torch.cuda.mem_get_info(self.device)
        return 1.0 - free / total

    def check(self) -> str:
        u = self.utilisation()
        if u >= self.critical:
            self.defragment()
            self.events.append(f"critical {u:.3f}")
            return "critical"
        if u >= self.warn:
            self.events.append(f"warn {u:.3f}")
            return "warn"
        return "ok"

    def defragment(self):
        if self.enabled:
            torch.cuda.empty_cache()

    def release_reserve(self) -> bool:
        had = self._reserve is not None
        self._reserve = None
        self.defragment()
        return had
