"""Communication and compute profilers.

* :class:`CommProfiler` — CUDA-event timing per collective, bus-bandwidth formulas, P50/95/99,
  communication ratio (src/profiling/comm_profiler.py:34-276); adds NVLink 5 peaks and a roofline
  fraction for fused compute+collective paths.
* :class:`ComputeProfiler` — FLOP estimator, MFU against a peak table, per-layer timing
  (src/profiling/compute_profiler.py:53-388); adds the B200 peak (measured when available) and reports
  both the reference-formula MFU (src/orchestrator/colocate_orchestrator.py:1197-1217) and an exact
  count including attention and GQA projection sizes.
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from collections import defaultdict
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

DEVICE_BANDWIDTH_GBS = {  # per direction per GPU
    "B200": 900.0, "H100": 450.0, "H20": 450.0, "A100": 300.0, "V100": 150.0, "PCIe4": 32.0,
}
MEASURED_NVLINK_GBS = {"B200_peer_copy": 770.0, "B200_allreduce_bus_8x": 725.0}
PEAK_TFLOPS_BF16 = {"B200": 2250.0, "H100": 989.0, "H20": 148.0, "A100": 312.0, "V100": 125.0, "L40S": 362.0}


def measured_peaks(path: Optional[str] = None) -> Dict[str, float]:
    """Measured roofline denominators for this machine if a ``MEASURED_PEAKS.json`` is present next to
    the package (hbm_gbs, bf16_tflops, bf16_tflops_sustained); otherwise an earlier measurement on the
    same kind of GPU, flagged ``source = fallback``."""
    cand = [path] if path else []
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    cand.append(os.path.join(here, "MEASURED_PEAKS.json"))
    for c in cand:
        if c and os.path.exists(c):
            with open(c) as f:
                d = json.load(f)
            d["source"] = "measured"
            return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def _pct(v: List[float], q: float) -> float:
    if not v:
        return 0.0
    s = sorted(v)
    i = min(len(s) - 1, max(0, int(round(q * (len(s) - 1)))))
    return s[i]


@dataclass
class CommRecord:
    """One timed collective (src/profiling/comm_profiler.py:22-31)."""
    op_type: str
    data_size_bytes: int
    latency_ms: float
    bandwidth_gbps: float
    overlap_hidden_ms: float = 0.0
    timestamp: float = 0.0
    world_size: int = 1


@dataclass
class LayerProfile:
    """Per-layer timing (src/profiling/compute_profiler.py:26-50)."""
    layer_name: str
    forward_ms: float
    backward_ms: float = 0.0
    flops: int = 0
    params: int = 0

    @property
    def total_ms(self) -> float:
        return self.forward_ms + self.backward_ms

    @property
    def tflops(self) -> float:
        """TFLOP/s from the forward time."""
        return (self.flops / 1e12) / (self.forward_ms / 1e3) if self.forward_ms > 0 and self.flops > 0 else 0.0


class CommProfiler:
    def __init__(self, device_name: str = "B200", enabled: bool = True):
        self.enabled = enabled
        self.device_name = device_name
        self.records: Dict[str, List[Dict[str, float]]] = defaultdict(list)
        self.total_step_ms = 0.0         # whole step (set_step_time), or ...
        self.compute_ms = 0.0            # ... compute outside the collectives (record_compute_time)

    @contextlib.contextmanager
    def profile_op(self, op: Optional[str] = None, nbytes=0, world_size: int = 1, op_type: Optional[str] = None,
                   tensor: Optional[torch.Tensor] = None):
        """``profile_op(op, nbytes, world_size)``; the reference passes the tensor itself
        (``profile_op(op_type, tensor, world_size)``: src/profiling/comm_profiler.py:96-150), whose size is then used."""
        op = op if op is not None else op_type
        if torch.is_tensor(nbytes):
            tensor = nbytes
        if tensor is not None:
            nbytes = tensor.numel() * tensor.element_size()
        if not self.enabled:
            yield
            return
        cuda = torch.cuda.is_available()
        if cuda:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
        t0 = time.perf_counter()
        yield
        if cuda:
            e.record()
            e.synchronize()
            ms = s.elapsed_time(e)
        else:
            ms = (time.perf_counter() - t0) * 1e3
        self.add(op, nbytes, world_size, ms)

    def add(self, op: str, nbytes: int, world_size: int, ms: float):
        self.records[op].append({"bytes": nbytes, "world": world_size, "ms": ms,
                                 "bus_gbs": self.bus_bandwidth(op, nbytes, world_size, ms)})

    @staticmethod
    def bus_bandwidth(op: str, nbytes: int, n: int, ms: float) -> float:
        """Ring-equivalent bus bandwidth in GB/s: all_reduce 2(n-1)/n, all_gather / reduce_scatter
        (n-1)/n of the full tensor, broadcast / p2p 1."""
        if ms <= 0 or n <= 0:
            return 0.0
        factor = {"all_reduce": 2.0 * (n - 1) / n, "all_gather": (n - 1) / n, "reduce_scatter": (n - 1) / n}.get(op, 1.0)
        return nbytes * factor / (ms * 1e-3) / 1e9

    @staticmethod
    def fused_roofline(flops: float, wire_bytes: float, ms: float, peak_tflops: float,
                       link_gbs: float = MEASURED_NVLINK_GBS["B200_peer_copy"]) -> Dict[str, float]:
        """Target time of a fused compute+collective kernel = max(compute at peak, bytes over the link);
        returns the target, the bound and achieved/target."""
        t_c = flops / (peak_tflops * 1e12) * 1e3
        t_w = wire_bytes / (link_gbs * 1e9) * 1e3
        tgt = max(t_c, t_w)
        return {"t_compute_ms": t_c, "t_wire_ms": t_w, "target_ms": tgt,
                "bound": "compute" if t_c >= t_w else "wire", "fraction": tgt / ms if ms > 0 else 0.0}

    def set_step_time(self, ms: float):
        self.total_step_ms += ms

    # ---- the reference's method names (src/profiling/comm_profiler.py:101-276) -------------------------------
    def record_compute_time(self, compute_ms: float):
        """Compute time outside the collectives; the communication ratio is then comm / (comm + compute)."""
        self.compute_ms += compute_ms

    def compute_bandwidth(self, data_size: int, latency_ms: float, op_type: str = "all_reduce",
                          world_size: int = 1) -> float:
        """Ring-algorithm bus bandwidth in GB/s.  As in the reference, ``data_size`` of an all-gather is the
        per-rank shard ((N-1) x shard bytes move) while ``bus_bandwidth`` takes the full gathered tensor."""
        n = max(world_size, 2)
        full = data_size * n if op_type == "all_gather" else data_size
        return self.bus_bandwidth(op_type, full, n, latency_ms)

    def get_theoretical_bandwidth(self, device: Optional[str] = None) -> float:
        """Interconnect bandwidth per direction per GPU in GB/s (the NVLink 5 figure for B200)."""
        table = dict(DEVICE_BANDWIDTH_GBS, A100_NVLINK=300.0, A100_PCIE=32.0, H100_NVLINK=450.0, B200_NVLINK=900.0,
                     **{"4090": 32.0, "3090": 16.0})
        return table.get((device or self.device_name).upper().replace("PCIE4", "PCIe4"), table.get(device or "", 32.0))

    @property
    def comm_records(self) -> List[CommRecord]:
        return [CommRecord(op, int(r["bytes"]), r["ms"], r["bus_gbs"], world_size=int(r["world"]))
                for op, recs in self.records.items() for r in recs]

    def report(self) -> str:
        s = self.get_summary()
        lines = ["== communication profile ==",
                 f"total {s['total_comm_ms']:.3f} ms, ratio of step {100 * s['comm_ratio']:.1f} %"]
        for op, d in s["ops"].items():
            lines.append(f"  {op:16s} n={d['count']:<5d} mean {d['mean_ms']:.3f} ms  p95 {d['p95_ms']:.3f} ms  "
                         f"bus {d['mean_bus_gbs']:.1f} GB/s ({100 * d['peak_fraction']:.0f} % of {self.device_name} link)")
        return "\n".join(lines)

    def reset(self):
        self.records.clear()
        self.total_step_ms = 0.0
        self.compute_ms = 0.0

    def get_summary(self) -> Dict:
        out: Dict = {"ops": {}}
        total = 0.0
        for op, recs in self.records.items():
            ms = [r["ms"] for r in recs]
            bw = [r["bus_gbs"] for r in recs]
            total += sum(ms)
            out["ops"][op] = {"count": len(recs), "total_ms": sum(ms), "mean_ms": sum(ms) / len(ms),
                              "p50_ms": _pct(ms, 0.5), "p95_ms": _pct(ms, 0.95), "p99_ms": _pct(ms, 0.99),
                              "mean_bus_gbs": sum(bw) / len(bw),
                              "peak_fraction": (sum(bw) / len(bw)) / DEVICE_BANDWIDTH_GBS.get(self.device_name, 900.0)}
        out["total_comm_ms"] = total
        step = self.total_step_ms if self.total_step_ms > 0 else total + self.compute_ms
        out["comm_ratio"] = total / step if step > 0 else 0.0
        return out


class ComputeProfiler:
    def __init__(self, device_name: str = "B200", peak_tflops: Optional[float] = None, enabled: bool = True):
        self.enabled = enabled
        self.device_name = device_name
        mp = measured_peaks()
        self.peak_tflops = peak_tflops or (mp["bf16_tflops_sustained"] if device_name == "B200"
                                           else PEAK_TFLOPS_BF16.get(device_name, 1000.0))
        self.layer_ms: Dict[str, List[float]] = defaultdict(list)

    # ---- FLOPs -----------------------------------------------------------------------------------
    @staticmethod
    def reference_formula_flops(L, B, S, H, I, V, full: bool = True) -> float:
        """The reference's estimate: fwd = L*2*B*S*(4H^2+3HI) + 2*B*S*H*V; x3 full / x2 LoRA."""
        fwd = L * 2.0 * B * S * (4 * H * H + 3 * H * I) + 2.0 * B * S * H * V
        return fwd * (3 if full else 2)

    @staticmethod
    def exact_flops(cfg, B: int, S: int, full: bool = True, causal: bool = True,
                    grad_checkpoint: bool = False, supervised_fraction: float = 1.0,
                    count_recompute: bool = False) -> float:
        """Matmul FLOPs of one training step's forward+backward as the kernels execute them: GQA-sized
        projections, SwiGLU FFN, causal attention (S^2 terms halved), and the LM head on the supervised rows
        only (``supervised_fraction`` of the tokens: rows whose label is ignored never reach the LM head).
        The forward pass that gradient checkpointing repeats is hardware work, not model work: it is added
        only with ``count_recompute`` (use that figure for HFU, the default for MFU)."""
        T = B * S
        D = cfg.head_dim
        proj = cfg.hidden_size * D * (2 * cfg.num_heads + 2 * cfg.num_kv_heads)
        ffn = 3 * cfg.hidden_size * cfg.intermediate_size
        attn = 2 * S * cfg.num_heads * D * (0.5 if causal else 1.0)  # per token: QK^T and PV, MACs
        body = 2.0 * T * cfg.num_layers * (proj + ffn + attn)
        head = 2.0 * T * supervised_fraction * cfg.hidden_size * cfg.vocab_size
        mult = 3 if full else 2
        total = (body + head) * mult
        if grad_checkpoint and count_recompute:
            total += body                                  # the layers' forward runs a second time
        return total

    def compute_mfu(self, *args, flops: Optional[float] = None, step_s: Optional[float] = None,
                    n_gpus: Optional[int] = None, actual_time_s: Optional[float] = None,
                    device: Optional[str] = None, num_devices: Optional[int] = None) -> float:
        """``compute_mfu(flops, step_s, n_gpus=1)``: whole-job FLOPs over ``n_gpus`` devices.

        The reference's form ``compute_mfu(actual_time_s, flops, device="A100", num_devices=1)``
        (src/profiling/compute_profiler.py:183-223) is accepted as well: there ``flops`` is already per GPU, the
        device count does not enter, and ``device`` names the peak to divide by.  Positionally the two are told apart
        by magnitude (a step's FLOPs exceed its seconds by many orders) and by a device name in third place."""
        reference_form = actual_time_s is not None or device is not None or num_devices is not None
        f, t = flops, (actual_time_s if actual_time_s is not None else step_s)
        if len(args) >= 3:
            if isinstance(args[2], str):                    # (seconds, FLOPs, device name[, count])
                device, reference_form = args[2], True
            else:                                           # (FLOPs, seconds, n_gpus)
                n_gpus = args[2]
        if len(args) >= 2:
            t, f = sorted(args[:2])
            reference_form = reference_form or args[0] < args[1]        # seconds first: the reference's order
        elif len(args) == 1:
            if t is not None:                               # compute_mfu(flops, step_s=...)
                f = args[0]
            else:                                           # compute_mfu(seconds, flops=...)
                t, reference_form = args[0], True
        if f is None or t is None or t <= 0:
            return 0.0
        if reference_form:
            return float(f) / (float(t) * self.get_peak_tflops(device) * 1e12)
        return float(f) / (float(t) * (n_gpus or 1) * self.peak_tflops * 1e12)

    # ---- per-layer timing --------------------------------------------------------------------------
    @contextlib.contextmanager
    def profile_layer(self, name: str):
        if not self.enabled:
            yield
            return
        cuda = torch.cuda.is_available()
        if cuda:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
        t0 = time.perf_counter()
        yield
        if cuda:
            e.record()
            e.synchronize()
            self.layer_ms[name].append(s.elapsed_time(e))
        else:
            self.layer_ms[name].append((time.perf_counter() - t0) * 1e3)

    def profile_model(self, model, run, warmup: int = 1, iters: int = 3) -> Dict[str, float]:
        """Time every top-level layer of ``model`` with forward hooks while ``run()`` executes."""
        starts: Dict[str, float] = {}
        hooks = []
        cuda = torch.cuda.is_available()

        def pre(name):
            def f(_m, _i):
                if cuda:
                    torch.cuda.synchronize()
                starts[name] = time.perf_counter()
            return f

        def post(name):
            def f(_m, _i, _o):
                if cuda:
                    torch.cuda.synchronize()
                self.layer_ms[name].append((time.perf_counter() - starts[name]) * 1e3)
            return f

        for name, mod in model.named_modules():
            if name and name.count(".") <= 1:
                hooks.append(mod.register_forward_pre_hook(pre(name)))
                hooks.append(mod.register_forward_hook(post(name)))
        try:
            for i in range(warmup + iters):
                if i == warmup:
                    self.layer_ms.clear()
                run()
        finally:
            for h in hooks:
                h.remove()
        return {k: sum(v) / len(v) for k, v in self.layer_ms.items()}

    # ---- the reference's method names (src/profiling/compute_profiler.py:83-388) -----------------------------
    def estimate_flops(self, batch_size: int, seq_len: int, hidden_size: int, num_layers: int, intermediate_size: int,
                       vocab_size: int, num_heads: int = 32, head_dim: int = 128, is_training: bool = True,
                       num_kv_heads: Optional[int] = None, causal: bool = False) -> Dict[str, float]:
        """Per-component forward FLOPs of a SwiGLU transformer and the total (x3 when training).  With the
        defaults (full-size K/V projections, non-causal S^2 terms) this is the reference's estimate; pass
        ``num_kv_heads`` / ``causal=True`` for the GQA, causal count the kernels actually execute."""
        B, S, H, I = batch_size, seq_len, hidden_size, intermediate_size
        kv = num_heads if num_kv_heads is None else num_kv_heads
        qkv = 2.0 * B * S * H * head_dim * (num_heads + 2 * kv)
        att = 2 * 2.0 * B * num_heads * S * S * head_dim * (0.5 if causal else 1.0)
        out = 2.0 * B * S * num_heads * head_dim * H
        mlp = 3 * 2.0 * B * S * H * I
        head = 2.0 * B * S * H * vocab_size
        fwd = num_layers * (qkv + att + out + mlp) + head
        return {"attention_per_layer": qkv + att + out, "mlp_per_layer": mlp, "per_layer": qkv + att + out + mlp,
                "lm_head": head, "forward_total": fwd, "backward_total": 2 * fwd if is_training else 0.0,
                "total": fwd * (3 if is_training else 1)}

    def get_peak_tflops(self, device: Optional[str] = None) -> float:
        """Dense bf16 tensor peak in TFLOP/s; for B200 the measured sustained cuBLAS figure this profiler uses."""
        if device is None or device.upper() == self.device_name.upper():
            return self.peak_tflops
        return PEAK_TFLOPS_BF16.get(device.upper(), PEAK_TFLOPS_BF16.get(device, 312.0))

    @property
    def layer_profiles(self) -> List[LayerProfile]:
        return [LayerProfile(k, sum(v) / len(v)) for k, v in self.layer_ms.items() if v]

    def report(self) -> str:
        lines = ["== compute profile ==", f"peak {self.peak_tflops:.0f} TFLOP/s ({self.device_name})"]
        total = sum(p.forward_ms for p in self.layer_profiles) or 1.0
        for p in sorted(self.layer_profiles, key=lambda x: -x.forward_ms):
            lines.append(f"  {p.layer_name:40s} {p.forward_ms:9.3f} ms  {100 * p.forward_ms / total:5.1f} %")
        return "\n".join(lines)

    def reset(self):
        self.layer_ms.clear()

    def get_summary(self) -> Dict:
        return {"peak_tflops": self.peak_tflops,
                "layers": {k: {"count": len(v), "mean_ms": sum(v) / len(v)} for k, v in self.layer_ms.items() if v}}
