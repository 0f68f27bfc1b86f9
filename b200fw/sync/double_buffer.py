"""Double-buffered LoRA state on the inference side (src/transfer/swift_sync.py:181-292).

``active`` is what the engine reads; deltas are applied to ``shadow`` in place; ``swap_buffers`` flips
the two under a lock and bumps the version.  After a swap the new shadow is brought level with the new
active so that the next delta applies to current weights.
"""
from __future__ import annotations

import threading
from collections.abc import Mapping
from typing import Dict, Optional

import torch


class FlatLayout:
    """Keys, shapes and offsets of a set of tensors packed back to back in one 1-D tensor."""

    def __init__(self, keys, shapes):
        self.keys = tuple(keys)
        self.shapes = tuple(tuple(int(d) for d in sh) for sh in shapes)
        self.offsets, n = [], 0
        for sh in self.shapes:
            self.offsets.append(n)
            m = 1
            for d in sh:
                m *= d
            n += m
        self.numel = n
        self.index = {k: i for i, k in enumerate(self.keys)}


class FlatState(Mapping):
    """A read-only ``{name: tensor}`` mapping whose tensors are views of ONE flat tensor (``flat``), created when they
    are asked for.  The SwiftSync stages recognise two flat states of the same layout and work on ``flat`` directly:
    a delta, a snapshot or a buffer swap over ~400 adapter tensors is then one tensor op instead of ~400 (or two
    multi-tensor launches plus as many Python-side tensor handles)."""

    def __init__(self, layout: FlatLayout, flat: torch.Tensor):
        assert flat.dim() == 1 and flat.numel() == layout.numel
        self.layout, self.flat = layout, flat

    def __getitem__(self, key):
        i = self.layout.index[key]
        sh, o = self.layout.shapes[i], self.layout.offsets[i]
        n = 1
        for d in sh:
            n *= d
        return self.flat[o:o + n].view(sh)

    def __contains__(self, key):
        return key in self.layout.index

    def __iter__(self):
        return iter(self.layout.keys)

    def __len__(self):
        return len(self.layout.keys)

    def clone(self) -> "FlatState":
        return FlatState(self.layout, self.flat.detach().clone())

    def same_layout(self, other) -> bool:
        return isinstance(other, FlatState) and other.layout is self.layout and other.flat.dtype == self.flat.dtype \
            and other.flat.device == self.flat.device


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
            self.active = self.shadow.clone() if isinstance(self.shadow, FlatState) else \
                {k: v.clone() for k, v in self.shadow.items()}

    def set_full_state(self, state: Dict[str, torch.Tensor], swap: bool = True) -> int:
        with self._lock:
            self.shadow = state.clone() if isinstance(state, FlatState) else {k: v.detach().clone() for k, v in state.items()}
        return self.swap_buffers() if swap else self.version

    def apply_delta_to_shadow(self, delta: Dict[str, torch.Tensor]) -> int:
        """``shadow[k] += delta[k]`` in place (unknown keys start from zero).  Returns the count applied."""
        n = 0
        with self._lock:
            if isinstance(self.shadow, FlatState):
                if self.shadow.same_layout(delta):
                    self.shadow.flat.add_(delta.flat)
                    return len(delta)
                self.shadow = dict(self.shadow)          # views of the flat tensor: the general path below edits them
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
            if isinstance(self.active, FlatState):
                self.active = dict(self.active)
            if isinstance(self.shadow, FlatState):
                self.shadow = dict(self.shadow)
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
            if isinstance(self.active, FlatState):
                if self.active.same_layout(self.shadow):
                    self.shadow.flat.copy_(self.active.flat)
                else:
                    self.shadow = self.active.clone()
                self.version += 1
                self.swap_count += 1
                return self.version
            if isinstance(self.shadow, FlatState):
                self.shadow = dict(self.shadow)
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
