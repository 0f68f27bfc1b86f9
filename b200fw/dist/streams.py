"""Compute / communication / transfer CUDA streams with event-based hand-offs.

Same surface as the reference's StreamManager (src/distributed/stream_manager.py:17-171): a default
priority compute stream, a high-priority communication stream and a transfer stream, plus counters.
On a CPU-only machine every method is a no-op so the callers need no branches.
"""
from __future__ import annotations

import contextlib
from typing import Dict, Optional

import torch


class StreamManager:
    def __init__(self, device: Optional[torch.device] = None):
        self.enabled = torch.cuda.is_available() and (device is None or device.type == "cuda")
        self.device = device
        self.stats: Dict[str, int] = {"comm_ops": 0, "transfer_ops": 0, "syncs": 0}
        if self.enabled:
            self.compute_stream = torch.cuda.current_stream(device)
            self.comm_stream = torch.cuda.Stream(device=device, priority=-1)
            self.transfer_stream = torch.cuda.Stream(device=device, priority=0)
        else:
            self.compute_stream = self.comm_stream = self.transfer_stream = None

    def _ctx(self, stream):
        return torch.cuda.stream(stream) if self.enabled else contextlib.nullcontext()

    def comm_context(self):
        self.stats["comm_ops"] += 1
        return self._ctx(self.comm_stream)

    def transfer_context(self):
        self.stats["transfer_ops"] += 1
        return self._ctx(self.transfer_stream)

    def _sync(self, waiter, signaller):
        if not self.enabled:
            return None
        ev = torch.cuda.Event()
        ev.record(signaller)
        waiter.wait_event(ev)
        self.stats["syncs"] += 1
        return ev

    def sync_compute_to_comm(self):
        """Communication stream waits for everything queued so far on the compute stream."""
        return self._sync(self.comm_stream, torch.cuda.current_stream() if self.enabled else None)

    def sync_comm_to_compute(self):
        return self._sync(torch.cuda.current_stream() if self.enabled else None, self.comm_stream)

    def sync_compute_to_transfer(self):
        return self._sync(self.transfer_stream, torch.cuda.current_stream() if self.enabled else None)

    def sync_transfer_to_compute(self):
        return self._sync(torch.cuda.current_stream() if self.enabled else None, self.transfer_stream)

    def synchronize_all(self):
        if self.enabled:
            torch.cuda.synchronize(self.device)

    def get_stats(self) -> Dict[str, int]:
        return dict(self.stats)

    # ---- the reference's method names (src/distributed/stream_manager.py:60-171) -----------------------------
    def compute_scope(self):
        return self._ctx(self.compute_stream)

    def comm_scope(self):
        return self.comm_context()

    def transfer_scope(self):
        return self.transfer_context()

    def sync_all(self):
        self.synchronize_all()

    def get_stream_stats(self) -> Dict[str, int]:
        return self.get_stats()

    def reset_stats(self):
        for k in self.stats:
            self.stats[k] = 0

    @property
    def _enabled(self) -> bool:
        return self.enabled

