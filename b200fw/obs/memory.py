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
    device_id: int = -1

    # the reference's field names (src/utils/memory_profiler.py:16-24), in MB
    @property
    def stage(self) -> str:
        return self.tag

    @property
    def allocated_mb(self) -> float:
        return self.allocated_gb * 1024

    @property
    def reserved_mb(self) -> float:
        return self.reserved_gb * 1024

    @property
    def peak_mb(self) -> float:
        return self.peak_allocated_gb * 1024


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


    @staticmethod
    def analyze(model: Optional[torch.nn.Module] = None, optimizer=None) -> Dict[str, float]:
        """Measured bytes held right now by a model's parameters, their gradients and an optimizer's state, in
        MB (the reference's ``MemoryBreakdown(model, optimizer).analyze()``: src/utils/memory_profiler.py:196-251)."""
        mb = 1024 ** 2
        out = {"model_params_mb": 0.0, "gradients_mb": 0.0, "optimizer_states_mb": 0.0}
        if model is not None:
            for p in model.parameters():
                out["model_params_mb"] += p.numel() * p.element_size() / mb
                g = getattr(p, "main_grad", None)
                g = p.grad if g is None else g
                if g is not None:
                    out["gradients_mb"] += g.numel() * g.element_size() / mb
        if optimizer is not None:
            if hasattr(optimizer, "memory_bytes"):
                b = optimizer.memory_bytes()
                out["optimizer_states_mb"] = (sum(v for k, v in b.items() if k != "params") if isinstance(b, dict) else b) / mb
            else:
                for st in getattr(optimizer, "state", {}).values():
                    out["optimizer_states_mb"] += sum(v.numel() * v.element_size() for v in st.values()
                                                      if torch.is_tensor(v)) / mb
        out["total_mb"] = sum(out.values())
        return out

    def report(self) -> str:
        rows = [("params", self.params_gb), ("gradients", self.grads_gb), ("optimizer", self.optimizer_gb),
                ("activations", self.activations_gb), ("logits", self.logits_gb), ("total", self.total_gb)]
        return "\n".join(["== memory estimate (GB per rank) =="] + [f"  {k:12s} {v:8.2f}" for k, v in rows])


class MemoryProfiler:
    def __init__(self, device: Optional[torch.device] = None, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self.device = device
        self.snapshots: List[MemorySnapshot] = []
        self.layer_peaks: Dict[str, float] = {}
        self._hooks = []
        self.phase_peaks: Dict[str, float] = {}

    def snapshot(self, tag: Optional[str] = None, stage: Optional[str] = None) -> MemorySnapshot:
        tag = tag if tag is not None else (stage or "")            # `stage`: the reference's parameter name
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

    # ---- the reference's method names (src/utils/memory_profiler.py:90-160) ------------------------------------
    def get_timeline(self) -> List[MemorySnapshot]:
        return list(self.snapshots)

    @property
    def peak_memory_mb(self) -> float:
        return max((s.peak_mb for s in self.snapshots), default=0.0)

    def delta(self, stage_a: str, stage_b: str) -> float:
        """Allocated-memory change in MB from the first snapshot tagged ``stage_a`` to the first tagged
        ``stage_b`` (0 when either is missing)."""
        a = next((s for s in self.snapshots if s.tag == stage_a), None)
        b = next((s for s in self.snapshots if s.tag == stage_b), None)
        return 0.0 if a is None or b is None else b.allocated_mb - a.allocated_mb

    def report(self) -> str:
        lines = ["== memory timeline ==", f"{'stage':24s} {'allocated MB':>14s} {'reserved MB':>14s} {'peak MB':>12s}"]
        lines += [f"{s.tag:24s} {s.allocated_mb:14.1f} {s.reserved_mb:14.1f} {s.peak_mb:12.1f}" for s in self.snapshots]
        return "\n".join(lines)

    def reset(self):
        self.snapshots.clear()
        self.layer_peaks.clear()
        self.phase_peaks.clear()
        self.reset_peak()


class StepMemoryReporter:
    """The reference's way of using its ``MemoryReport``: an object built as ``MemoryReport(model, optimizer, config)``
    whose ``profile_step(input_ids, labels, train_step_fn)`` / ``generate_report_without_step()`` return a plain dict
    with the sections ``model_spec``, ``static_memory``, ``dynamic_memory``, ``framework_overhead`` and
    ``peak_moments`` (src/utils/memory_profiler.py:409-546; ``scripts/profile_memory.py`` prints from them).
    ``MemoryReport(model, ...)`` returns one of these; the dataclass form is for reports assembled from a
    :class:`MemoryProfiler`.  Byte counts come from the tensors themselves, peaks from the CUDA allocator (zero on a
    CPU)."""

    def __init__(self, model: torch.nn.Module, optimizer=None, config: Optional[Dict[str, Any]] = None):
        self.model, self.optimizer, self.config = model, optimizer, dict(config or {})

    # ---- sections -----------------------------------------------------------------------------------------------
    @staticmethod
    def _readable(n: int) -> str:
        for unit, div in (("B", 1e9), ("M", 1e6), ("K", 1e3)):
            if n >= div:
                return f"{n / div:.2f}{unit}"
        return str(n)

    def _model_spec(self) -> Dict[str, Any]:
        params = list(self.model.parameters())
        total = sum(p.numel() for p in params)
        trainable = sum(p.numel() for p in params if p.requires_grad)
        by_dtype: Dict[str, int] = {}
        for p in params:
            by_dtype[str(p.dtype).replace("torch.", "")] = by_dtype.get(str(p.dtype).replace("torch.", ""), 0) + p.numel()
        return {"total_params": total, "trainable_params": trainable, "frozen_params": total - trainable,
                "total_params_readable": self._readable(total), "trainable_params_readable": self._readable(trainable),
                "trainable_ratio": trainable / total if total else 0.0, "precision_distribution": by_dtype}

    def _static_memory(self) -> Dict[str, float]:
        gb = 1e9
        frozen16 = frozen32 = train = grads = 0
        for p in self.model.parameters():
            b = p.numel() * p.element_size()
            if p.requires_grad:
                train += b
                mg = getattr(p, "main_grad", None)
                g = p.grad if p.grad is not None else mg
                grads += g.numel() * g.element_size() if g is not None else b
            elif p.element_size() <= 2:
                frozen16 += b
            else:
                frozen32 += b
        opt = 0
        o = self.optimizer
        if o is not None and hasattr(o, "memory_bytes"):
            mb = o.memory_bytes()
            opt = sum(mb.values()) if isinstance(mb, dict) else int(mb)
        elif o is not None and hasattr(o, "state"):
            opt = sum(t.numel() * t.element_size() for st in o.state.values() for t in st.values() if torch.is_tensor(t))
        out = {"frozen_weights_bf16_gb": frozen16 / gb, "frozen_weights_fp32_gb": frozen32 / gb,
               "trainable_weights_gb": train / gb, "gradients_gb": grads / gb, "optimizer_states_gb": opt / gb}
        out["static_total_gb"] = sum(out.values())
        return out

    def _overhead(self, device) -> Dict[str, float]:
        if device.type != "cuda":
            return {"pytorch_caching_gb": 0.0, "cuda_context_estimated_gb": 0.0}
        free, total = torch.cuda.mem_get_info(device)
        return {"pytorch_caching_gb": (torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)) / 1e9,
                # what the device reports in use beyond this process's allocator: context, libraries, other tenants
                "cuda_context_estimated_gb": max(0.0, (total - free - torch.cuda.memory_reserved(device)) / 1e9),
                "device_total_memory_gb": total / 1e9}

    def generate_report_without_step(self) -> Dict[str, Any]:
        device = next(self.model.parameters()).device
        return {"model_spec": self._model_spec(), "static_memory": self._static_memory(), "dynamic_memory": {},
                "framework_overhead": self._overhead(device), "peak_moments": {}, "config": self.config}

    def profile_step(self, input_ids, labels=None, train_step_fn=None) -> Dict[str, Any]:
        """One measured step.  With ``train_step_fn`` that callable is the step; without one the step is a forward
        pass, the shifted next-token loss over ``labels`` (``-100`` ignored) and a backward pass."""
        device = next(self.model.parameters()).device
        cuda = device.type == "cuda"
        report = self.generate_report_without_step()
        prof = MemoryProfiler(device)
        prof.attach_layer_hooks(self.model)

        def peak_gb():
            if not cuda:
                return 0.0
            torch.cuda.synchronize(device)
            return torch.cuda.max_memory_allocated(device) / 1e9

        try:
            before = torch.cuda.memory_allocated(device) if cuda else 0
            prof.reset_peak()
            with torch.no_grad():
                self.model(input_ids)
            report["peak_moments"]["forward_peak_gb"] = peak_gb()
            report["peak_moments"]["forward_activation_gb"] = \
                ((torch.cuda.memory_allocated(device) - before) / 1e9) if cuda else 0.0
            prof.reset_peak()
            self.model.train()
            if train_step_fn is not None:
                train_step_fn(input_ids, labels)
            else:
                logits = self.model(input_ids)
                if labels is not None:
                    loss = torch.nn.functional.cross_entropy(
                        logits[:, :-1, :].reshape(-1, logits.shape[-1]).float(), labels[:, 1:].reshape(-1),
                        ignore_index=-100)
                    loss.backward()
            report["peak_moments"]["backward_peak_gb"] = peak_gb()
            if train_step_fn is None and self.optimizer is not None and hasattr(self.optimizer, "step"):
                prof.reset_peak()
                try:
                    self.optimizer.step()
                    self.optimizer.zero_grad()
                except Exception as e:  # noqa: BLE001 - the report is still useful without the optimizer phase
                    report["peak_moments"]["optimizer_step_error"] = f"{type(e).__name__}: {e}"
            report["peak_moments"]["step_peak_gb"] = max(peak_gb(), report["peak_moments"]["backward_peak_gb"])
        finally:
            prof.detach_hooks()
        report["dynamic_memory"] = {"per_layer_peak_mb": dict(prof.layer_peaks)}
        report["static_memory"] = self._static_memory()      # gradients and optimizer state exist now
        report["framework_overhead"] = self._overhead(device)
        return report


@dataclass
class MemoryReport:
    breakdown: Optional[MemoryBreakdown] = None
    snapshots: List[Dict[str, Any]] = field(default_factory=list)
    phase_peaks: Dict[str, float] = field(default_factory=dict)
    layer_peaks: Dict[str, float] = field(default_factory=dict)
    optimizer_bytes: Dict[str, int] = field(default_factory=dict)
    notes: List[str] = field(default_factory=list)

    def __new__(cls, *args, **kwargs):
        # the reference's form ``MemoryReport(model, optimizer, config)``: a reporter object (see StepMemoryReporter)
        if args and isinstance(args[0], torch.nn.Module):
            return StepMemoryReporter(*args, **kwargs)
        return super().__new__(cls)

    @classmethod
    def from_profiler(cls, prof: MemoryProfiler, breakdown: Optional[MemoryBreakdown] = None,
                      optimizer_bytes: Optional[Dict[str, int]] = None) -> "MemoryReport":
        return cls(breakdown, prof.timeline(), dict(prof.phase_peaks), dict(prof.layer_peaks),
                   dict(optimizer_bytes or {}))

    # ---- the reference's entry points (src/utils/memory_profiler.py:454-546): there ``MemoryReport(model,
    # optimizer, config)`` is an object with these two methods; here they are constructors of the report ---------
    @classmethod
    def profile_step(cls, input_ids, labels, train_step_fn, model: Optional[torch.nn.Module] = None, optimizer=None,
                     breakdown: Optional[MemoryBreakdown] = None) -> "MemoryReport":
        """Run ``train_step_fn(input_ids, labels)`` once with snapshots around it, the step's peak and (with a
        ``model``) per-layer peaks from forward hooks."""
        prof = MemoryProfiler()
        if model is not None:
            prof.attach_layer_hooks(model)
        prof.snapshot("before_step")
        prof.reset_peak()
        try:
            train_step_fn(input_ids, labels)
        finally:
            prof.detach_hooks()
        prof.mark_phase("step")
        prof.snapshot("after_step")
        rep = cls.from_profiler(prof, breakdown, cls._optimizer_bytes(optimizer))
        if model is not None:
            rep.notes.append("measured MB: " + json.dumps(MemoryBreakdown.analyze(model, optimizer)))
        return rep

    @classmethod
    def generate_report_without_step(cls, model: Optional[torch.nn.Module] = None, optimizer=None,
                                     breakdown: Optional[MemoryBreakdown] = None) -> "MemoryReport":
        """Static part only: what the model and optimizer hold now, no training step."""
        prof = MemoryProfiler()
        prof.snapshot("static")
        rep = cls.from_profiler(prof, breakdown, cls._optimizer_bytes(optimizer))
        rep.notes.append("measured MB: " + json.dumps(MemoryBreakdown.analyze(model, optimizer)))
        return rep

    @staticmethod
    def _optimizer_bytes(optimizer) -> Dict[str, int]:
        if optimizer is None or not hasattr(optimizer, "memory_bytes"):
            return {}
        b = optimizer.memory_bytes()
        return dict(b) if isinstance(b, dict) else {"total": int(b)}

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

    def __init__(self, *args, warn: float = 0.85, critical: float = 0.95, reserve_mb: int = 0,
                 device: Optional[torch.device] = None, warning_threshold: Optional[float] = None,
                 critical_threshold: Optional[float] = None):
        """``MemoryManager(warn, critical, reserve_mb, device)``; or, in the reference's order
        (src/utils/memory_manager.py:22-40), ``MemoryManager(device, warning_threshold, critical_threshold)``: a device
        (index, name or ``torch.device``) in first place selects that form."""
        if args and (isinstance(args[0], (str, torch.device)) or (isinstance(args[0], int) and not isinstance(args[0], bool))):
            names = ("device", "warn", "critical")
        else:
            names = ("warn", "critical", "reserve_mb", "device")
        given = dict(warn=warn, critical=critical, reserve_mb=reserve_mb, device=device)
        for name, value in zip(names, args):
            given[name] = value
        warn, critical, reserve_mb, device = given["warn"], given["critical"], given["reserve_mb"], given["device"]
        warn = warning_threshold if warning_threshold is not None else warn
        critical = critical_threshold if critical_threshold is not None else critical
        if isinstance(device, int):
            device = torch.device("cuda", device)
        self.warn, self.critical, self.device = float(warn), float(critical), device
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

    # ---- the reference's method names (src/utils/memory_manager.py:25-100) ---------------------------------------
    def get_stats(self) -> Dict[str, float]:
        """Allocated / reserved / peak / total GB of the device, without side effects (``{}`` without CUDA)."""
        if not self.enabled:
            return {}
        return {"allocated_gb": torch.cuda.memory_allocated(self.device) / 1e9,
                "reserved_gb": torch.cuda.memory_reserved(self.device) / 1e9,
                "peak_gb": torch.cuda.max_memory_allocated(self.device) / 1e9,
                "total_gb": torch.cuda.get_device_properties(self.device or 0).total_memory / 1e9}

    def check_memory_pressure(self) -> Dict[str, float]:
        """Current figures plus ``utilization`` (allocated / total) and ``fragmentation_gb``; records a warn /
        critical event when a threshold is crossed."""
        if not self.enabled:
            return {"allocated_gb": 0, "reserved_gb": 0, "total_gb": 0, "utilization": 0}
        st = self.get_stats()
        st["utilization"] = st["allocated_gb"] / st["total_gb"] if st["total_gb"] else 0.0
        st["fragmentation_gb"] = st["reserved_gb"] - st["allocated_gb"]
        if st["utilization"] >= self.critical:
            self.events.append(f"critical {st['utilization']:.3f}")
        elif st["utilization"] >= self.warn:
            self.events.append(f"warn {st['utilization']:.3f}")
        return st

    def reserve_buffer(self, size_mb: int = 512):
        """Hold back ``size_mb`` of device memory to hand out when an out-of-memory error is being handled."""
        if self.enabled and self._reserve is None:
            self._reserve = torch.empty(size_mb * 1024 * 1024, dtype=torch.uint8, device=self.device or "cuda")

    def release_buffer(self):
        self.release_reserve()

