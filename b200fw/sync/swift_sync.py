"""SwiftSync: ship LoRA *deltas* instead of full weights, with a periodic full sync.

Roles of the reference module (src/transfer/swift_sync.py:36-596): ``DeltaComputer`` (GPU subtraction
against the previous snapshot; full sync when ``step > 0 and step % N == 0``), ``SwiftSyncTransfer``
(apply the delta to the shadow buffer -> notify the worker with ``update_weights(state, mode)`` ->
swap -> stats).  A worker without ``update_weights`` raises and leaves the version untouched.
"""
from __future__ import annotations

import inspect
import time
from dataclasses import dataclass, field
from collections.abc import Coroutine
from typing import Dict, List, Optional

import torch

from .double_buffer import DoubleBufferedLoRA, FlatState
from ..compat import kwarg_aliases


@dataclass
class SwiftSyncConfig:
    enabled: bool = False
    fallback_full_every: int = 10
    double_buffer: bool = True
    # further fields of the reference's config (src/transfer/swift_sync.py:36-52)
    delta_threshold: float = 1e-8        # reserved there for sparse deltas; not used by either implementation
    async_transfer: bool = True          # the orchestrator picks sync_*_async when it runs inside an event loop
    enable_double_buffer: Optional[bool] = None   # the reference's name for ``double_buffer``; wins when given

    def __post_init__(self):
        if self.enable_double_buffer is not None:
            self.double_buffer = bool(self.enable_double_buffer)
        self.enable_double_buffer = self.double_buffer


@dataclass
class DeltaVersion:
    """What one delta sync carried (src/transfer/swift_sync.py:55-68)."""
    version: int
    timestamp: float
    num_params: int
    delta_bytes: int


@dataclass
class SwiftSyncStats:
    delta_syncs: int = 0
    full_syncs: int = 0
    bytes_sent: int = 0
    total_time_s: float = 0.0
    last_mode: str = ""
    last_bytes: int = 0
    last_time_s: float = 0.0
    history: List[Dict] = field(default_factory=list)

    def record(self, mode: str, nbytes: int, dt: float):
        if mode == "delta":
            self.delta_syncs += 1
        else:
            self.full_syncs += 1
        self.bytes_sent += nbytes
        self.total_time_s += dt
        self.last_mode, self.last_bytes, self.last_time_s = mode, nbytes, dt
        self.history.append({"mode": mode, "bytes": nbytes, "time_s": dt,
                             "gbps": nbytes / dt / 1e9 if dt > 0 else 0.0})


    # the reference's counter names (SyncStats, src/transfer/swift_sync.py:71-83)
    @property
    def total_delta_syncs(self) -> int:
        return self.delta_syncs

    @property
    def total_full_syncs(self) -> int:
        return self.full_syncs

    @property
    def total_delta_bytes(self) -> int:
        return sum(h["bytes"] for h in self.history if h["mode"] == "delta")

    @property
    def total_full_bytes(self) -> int:
        return sum(h["bytes"] for h in self.history if h["mode"] != "delta")

    @property
    def last_sync_time(self) -> float:
        return self.last_time_s

    @property
    def last_sync_type(self) -> str:
        return self.last_mode

    @property
    def cumulative_time(self) -> float:
        return self.total_time_s


SyncStats = SwiftSyncStats


class SyncResult(int, Coroutine):
    """What ``sync_delta`` / ``sync_full`` return: the new version as an ``int`` that can also be awaited.

    The reference declares these two methods ``async`` (src/transfer/swift_sync.py:352-470), so code written
    against it says ``await transfer.sync_delta(delta, worker)`` or ``asyncio.run(transfer.sync_full(...))``;
    here the work is done by the time the call returns, and awaiting the result yields the
    :class:`DeltaVersion` record at once."""

    def __new__(cls, version: int, info: "DeltaVersion"):
        obj = int.__new__(cls, version)
        obj.info = info
        return obj

    def __await__(self):
        if False:
            yield
        return self.info

    def send(self, value):
        raise StopIteration(self.info)

    def throw(self, typ, val=None, tb=None):
        raise val if val is not None else (typ() if isinstance(typ, type) else typ)

    def close(self):
        pass


class DeltaComputer:
    def __init__(self, fallback_full_every=10):
        """``fallback_full_every``: the period, or a :class:`SwiftSyncConfig` carrying it (the reference passes
        its config: src/transfer/swift_sync.py:90-110)."""
        if isinstance(fallback_full_every, SwiftSyncConfig):
            fallback_full_every = fallback_full_every.fallback_full_every
        self.fallback_full_every = int(fallback_full_every)
        self.prev: Optional[Dict[str, torch.Tensor]] = None
        self._step_count = 0

    def should_full_sync(self, step: int) -> bool:
        return step > 0 and self.fallback_full_every > 0 and step % self.fallback_full_every == 0

    @torch.no_grad()
    @kwarg_aliases(current_lora="current", prev_lora="prev")
    def compute_delta(self, current: Dict[str, torch.Tensor],
                      prev: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
        """current - previous snapshot (first call: the full state), then remember ``current``.  With an explicit
        ``prev`` the call is stateless: ``current - prev`` per key, a key missing from ``prev`` yields itself."""
        self._step_count += 1
        if prev is not None:
            return {k: v.detach() - prev[k].to(v.device) if k in prev else v.detach().clone() for k, v in current.items()}
        if isinstance(current, FlatState):
            # one subtraction for all adapters; ``current.flat`` is the caller's fresh copy and becomes the snapshot
            if isinstance(self.prev, FlatState) and self.prev.same_layout(current):
                delta = FlatState(current.layout, current.flat - self.prev.flat)
            else:
                delta = current.clone()
            self.prev = current
            return delta
        keys = list(current)
        cur = [current[k].detach() for k in keys]
        if self.prev is not None and list(self.prev) == keys and all(
                p.shape == c.shape and p.device == c.device and p.dtype == c.dtype
                for p, c in zip(self.prev.values(), cur)):
            # same tensors as last time: two multi-tensor launches instead of two small kernels per tensor
            old = list(self.prev.values())
            delta = dict(zip(keys, torch._foreach_sub(cur, old)))
            torch._foreach_copy_(old, cur)                 # the snapshot is updated in place
            return delta
        if self.prev is None:
            delta = {k: v.clone() for k, v in zip(keys, cur)}
        else:
            delta = {k: v - self.prev[k] if k in self.prev else v.clone() for k, v in zip(keys, cur)}
        self.prev = {k: v.clone() for k, v in zip(keys, cur)}
        return delta

    def reset(self):
        self.prev = None

    @staticmethod
    def compute_delta_bytes(delta: Dict[str, torch.Tensor]) -> int:
        return _nbytes(delta)


def _nbytes(state: Dict[str, torch.Tensor]) -> int:
    if isinstance(state, FlatState):
        return state.flat.numel() * state.flat.element_size()
    return sum(v.numel() * v.element_size() for v in state.values())


class SwiftSyncTransfer:
    def __init__(self, infer_worker=None, config: Optional[SwiftSyncConfig] = None,
                 buffer: Optional[DoubleBufferedLoRA] = None):
        if isinstance(infer_worker, SwiftSyncConfig):      # the reference's constructor takes the config first
            infer_worker, config = None, infer_worker
        self.worker = infer_worker
        self.config = config or SwiftSyncConfig(enabled=True)
        self.buffer = buffer or DoubleBufferedLoRA()
        self.delta_computer = DeltaComputer(self.config.fallback_full_every)
        self.stats = SwiftSyncStats()

    def _commit(self, payload: Dict[str, torch.Tensor], mode: str) -> int:
        """Update the local copy after the worker accepted the payload: shadow + swap with double buffering, in
        place without.  Returns the new version."""
        if not self.config.double_buffer:
            return self.buffer.update_in_place(payload, add=mode == "delta")
        if mode == "delta":
            self.buffer.apply_delta_to_shadow(payload)
            return self.buffer.swap_buffers()
        return self.buffer.set_full_state(payload, swap=True)

    def _notify(self, state: Dict[str, torch.Tensor], mode: str):
        if self.worker is None:
            return
        fn = getattr(self.worker, "update_weights", None)
        if fn is None:
            raise AttributeError("inference worker has no update_weights(state, mode)")
        remote = getattr(fn, "remote", None)
        res = remote(state, mode=mode) if remote is not None else fn(state, mode=mode)
        if inspect.isawaitable(res):
            import asyncio
            try:
                loop = asyncio.get_running_loop()
            except RuntimeError:
                loop = None
            if loop is None:
                asyncio.run(_await(res))
            else:   # already inside a loop: the caller should use the async variants
                raise RuntimeError("use sync_delta_async / sync_full_async inside an event loop")

    def sync_delta(self, delta: Dict[str, torch.Tensor], infer_worker=None) -> int:
        """Apply a delta: notify first (a worker that cannot take it must not see a version bump),
        then update the local double buffer and swap.  ``infer_worker`` replaces the worker given at construction."""
        if infer_worker is not None:
            self.worker = infer_worker
        t0 = time.perf_counter()
        self._notify(delta, "delta")
        v = self._commit(delta, "delta")
        self.stats.record("delta", _nbytes(delta), time.perf_counter() - t0)
        return SyncResult(v, DeltaVersion(v, time.time(), len(delta), _nbytes(delta)))

    def sync_full(self, state: Optional[Dict[str, torch.Tensor]] = None, infer_worker=None, *,
                  full_state: Optional[Dict[str, torch.Tensor]] = None) -> int:
        state = state if state is not None else full_state          # ``full_state``: the reference's keyword
        if infer_worker is not None:
            self.worker = infer_worker
        t0 = time.perf_counter()
        self._notify(state, "full")
        v = self._commit(state, "full")
        self.delta_computer.prev = state.clone() if isinstance(state, FlatState) else \
            {k: t.detach().clone() for k, t in state.items()}
        self.stats.record("full", _nbytes(state), time.perf_counter() - t0)
        return SyncResult(v, DeltaVersion(v, time.time(), len(state), _nbytes(state)))

    async def sync_delta_async(self, delta: Dict[str, torch.Tensor], infer_worker=None) -> int:
        if infer_worker is not None:
            self.worker = infer_worker
        t0 = time.perf_counter()
        await self._notify_async(delta, "delta")
        v = self._commit(delta, "delta")
        self.stats.record("delta", _nbytes(delta), time.perf_counter() - t0)
        return v

    async def sync_full_async(self, state: Dict[str, torch.Tensor], infer_worker=None) -> int:
        if infer_worker is not None:
            self.worker = infer_worker
        t0 = time.perf_counter()
        await self._notify_async(state, "full")
        v = self._commit(state, "full")
        self.delta_computer.prev = state.clone() if isinstance(state, FlatState) else \
            {k: t.detach().clone() for k, t in state.items()}   # next delta is relative to this
        self.stats.record("full", _nbytes(state), time.perf_counter() - t0)
        return v

    async def _notify_async(self, state, mode):
        if self.worker is None:
            return
        fn = getattr(self.worker, "update_weights", None)
        if fn is None:
            raise AttributeError("inference worker has no update_weights(state, mode)")
        res = fn(state, mode=mode)
        if inspect.isawaitable(res):
            await res

    def sync(self, step: int, lora_state: Dict[str, torch.Tensor]) -> int:
        """Policy wrapper: periodic full sync, deltas otherwise."""
        if self.delta_computer.prev is None or self.delta_computer.should_full_sync(step):
            return self.sync_full(lora_state)
        delta = self.delta_computer.compute_delta(lora_state)       # also moves the snapshot to ``lora_state``
        try:
            return self.sync_delta(delta)
        except Exception:
            # the worker never saw this delta but the snapshot already contains it: the next delta would silently skip
            # it.  Forget the snapshot instead, so that the next sync is a full one.
            self.delta_computer.reset()
            raise

    # ---- the reference's names (src/transfer/swift_sync.py:340-596) -------------------------------------------
    def initialize(self, initial_lora_state: Dict[str, torch.Tensor]) -> None:
        """Seed the previous-state snapshot and both buffers with the adapters' initial state, so that the first
        ``sync`` already sends a delta.  Without it the first ``sync`` is a full one."""
        self.delta_computer.prev = initial_lora_state.clone() if isinstance(initial_lora_state, FlatState) else \
            {k: v.detach().clone() for k, v in initial_lora_state.items()}
        self.buffer = DoubleBufferedLoRA(initial_lora_state)         # version 0: nothing has been synced yet

    @property
    def initialized(self) -> bool:
        return self.delta_computer.prev is not None

    @property
    def prev_snapshot(self) -> Optional[Dict[str, torch.Tensor]]:
        return self.delta_computer.prev

    @property
    def double_buffer(self) -> Optional[DoubleBufferedLoRA]:
        """The local double buffer (``None`` when the config turns double buffering off: the state is then kept
        in a single buffer that is updated in place)."""
        return self.buffer if self.config.double_buffer else None

    @property
    def version(self) -> int:
        return self.buffer.version

    @property
    def last_delta_version(self) -> Optional[DeltaVersion]:
        h = next((x for x in reversed(self.stats.history) if x["mode"] == "delta"), None)
        return None if h is None else DeltaVersion(self.version, time.time(), len(self.buffer.get_active_state()), h["bytes"])

    def get_stats_summary(self) -> Dict:
        s = self.stats
        return {"version": self.version, "initialized": self.initialized, "total_delta_syncs": s.total_delta_syncs,
                "total_full_syncs": s.total_full_syncs, "total_delta_bytes": s.total_delta_bytes,
                "total_full_bytes": s.total_full_bytes, "last_sync_time": s.last_sync_time,
                "last_sync_type": s.last_sync_type, "cumulative_time": s.cumulative_time,
                "config": {"enabled": self.config.enabled, "fallback_full_every": self.config.fallback_full_every,
                           "enable_double_buffer": self.config.double_buffer, "async_transfer": self.config.async_transfer}}

    def get_stats(self) -> Dict:
        s = self.stats
        return {"delta_syncs": s.delta_syncs, "full_syncs": s.full_syncs, "bytes_sent": s.bytes_sent,
                "total_time_s": s.total_time_s, "version": self.buffer.version, "last_mode": s.last_mode,
                "last_bytes": s.last_bytes, "last_time_s": s.last_time_s}


async def _await(x):
    return await x
