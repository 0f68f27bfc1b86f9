"""Double-buffered LoRA state on the inference side (src/transfer/swift_sync.py:181-292).

``active`` is what the engine reads; deltas are applied to ``shadow`` in place; ``swap_buffers`` flips
the two under a lock and bumps the version.  After a swap the new shadow is brought level with the new
active so that the next delta applies to current weights.
"""
from __future__ import annotations

import threading
from typing import Dict, Optional

import torch


class DoubleBufferedLoRA:
    def __init__(self, initial_state: Optional[Dict[str, torch.Tensor]] = None,
                 initial_lora_state: Optional[Dict[str, torch.Tensor]] = None):
        initial_state = initial_state if initial_state is not None else initial_lora_state
        self._lock = threading.Lock()
        self.active: Dict[str, torch.Tensor] = {}
        self.shadow: Dict[str, torch.Tensor] = {}
        self.version = 0
        self.swap_count = 0
        if initial_state:
            self.set_full_state(initial_state, swap=False)
            self.active = {k: v.clone() for k, v in self.shadow.items()}

    def set_full_state(self, state: Dict[str, torch.Tensor], swap: bool = True) -> int:
        with self._lock:
            self.shadow = {k: v.detach().clone() for k, v in state.items()}
        return self.swap_buffers() if swap else self.version

    def apply_delta_to_shadow(self, delta: Dict[str, torch.Tensor]) -> int:
        """``shadow[k] += delta[k]`` in place (unknown keys start from zero).  Returns the count applied."""
        n = 0
        with self._lock:
            if delta and all(k in self.shadow and self.shadow[k].shape == d.shape and self.shadow[k].dtype == d.dtype
                             and self.shadow[k].device == d.device for k, d in delta.items()):
                torch._foreach_add_([self.shadow[k] for k in delta], [d.detach() for d in delta.values()])
                return len(delta)
            for k, d in delta.items():
                cur = self.shadow.get(k)
                if cur is None:
                    self.shadow[k] = d.detach().clone()
                else:
                    cur.add_(d.to(cur.dtype).to(cur.device))
                n += 1
        return n

    def update_in_place(self, payload: Dict[str, torch.Tensor], add: bool) -> int:
        """Single-buffer mode: add ``payload`` to (or overwrite) the active tensors directly, keep the shadow
        level with them, bump the version."""
        with self._lock:
            for k, t in payload.items():
                cur = self.active.get(k)
                if cur is None or cur.shape != t.shape:
                    self.active[k] = t.detach().clone()
                elif add:
                    cur.add_(t.to(cur.dtype).to(cur.device))
                else:
                    cur.copy_(t)
                self.shadow[k] = self.active[k].clone()
            self.version += 1
            return self.version

    def swap_buffers(self) -> int:
        with self._lock:
            self.active, self.shadow = self.shadow, self.active
            # level the new shadow with the new active
            if self.active and list(self.active) == list(self.shadow) and all(
                    s.shape == v.shape and s.dtype == v.dtype and s.device == v.device
                    for s, v in zip(self.shadow.values(), self.active.values())):
                torch._foreach_copy_(list(self.shadow.values()), list(self.active.values()))
                self.version += 1
                self.swap_count += 1
                return self.version
            for k, v in self.active.items():
                s = self.shadow.get(k)
                if s is None or s.shape != v.shape:
                    self.shadow[k] = v.clone()
                else:
                    s.copy_(v)
            for k in [k for k in self.shadow if k not in self.active]:
                del self.shadow[k]
            self.version += 1
            self.swap_count += 1
            return self.version

    def get_active_state(self) -> Dict[str, torch.Tensor]:
        with self._lock:
            return dict(self.active)

    def get_version(self) -> int:
        return self.version
