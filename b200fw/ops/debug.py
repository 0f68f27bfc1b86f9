"""Guard bands around kernel outputs: a host-side out-of-bounds write detector.

``compute-sanitizer`` style tools are not always available where the kernels run, and a stray store from a
tile-edge predicate usually lands in a neighbouring tensor where nothing notices.  Inside
``with canary_arena() as arena:`` every tensor that the Python side of an op allocates with ``torch.empty`` /
``torch.zeros`` / ``torch.empty_like`` / ``torch.zeros_like`` on the watched device type is carved out of a
larger byte buffer that is pre-filled with a pattern:

    [ 4096 guard bytes | payload | slack to the next 256 bytes | 4096 guard bytes ]

The payload keeps its 512-byte allocator alignment (TMA and 16-byte vector accesses still work).  On exit the
device is synchronised and every guard byte is compared with the pattern; a mismatch raises ``CanaryError``
naming the allocation (shape, dtype, call site) and the first corrupted offset relative to the payload.  Nothing
traps or faults on the device: the check is a host-side comparison after the kernels have finished.

The reference has no race or bounds detection at all (its only concurrency test is the double-buffer swap
stress in tests/test_swift_sync.py:154-173); this is the bounds half of the replacement, the numerics tests
against fp32 references at tile-edge shapes are the other half.
"""
from __future__ import annotations

import contextlib
import traceback
from typing import Iterable, List, Tuple

import torch

__all__ = ["CanaryArena", "CanaryError", "canary_arena", "GUARD_BYTES"]

GUARD_BYTES = 4096
_PATTERN = 0xA5
_PATCHED = ("empty", "zeros", "empty_like", "zeros_like")


class CanaryError(RuntimeError):
    pass


class CanaryArena:
    def __init__(self):
        self.records: List[Tuple[torch.Tensor, int, str]] = []      # (raw bytes, payload bytes, label)

    def alloc(self, shape, dtype: torch.dtype, device, zero: bool = False, label: str = "") -> torch.Tensor:
        shape = tuple(int(s) for s in shape)
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        padded = (nbytes + 255) // 256 * 256
        raw = _ORIG["empty"](GUARD_BYTES + padded + GUARD_BYTES, dtype=torch.uint8, device=device)
        raw.fill_(_PATTERN)
        view = raw[GUARD_BYTES:GUARD_BYTES + nbytes].view(dtype).view(shape)
        if zero:
            view.zero_()
        self.records.append((raw, nbytes, label or f"{shape} {dtype}"))
        return view

    def violations(self) -> List[str]:
        """One line per corrupted guard region (empty when every canary is intact)."""
        out = []
        for raw, nbytes, label in self.records:
            if raw.is_cuda:
                torch.cuda.synchronize(raw.device)
            front, back = raw[:GUARD_BYTES], raw[GUARD_BYTES + nbytes:]
            bad = (front != _PATTERN).nonzero()
            if bad.numel():
                first = int(bad.max()) - GUARD_BYTES             # closest to the payload
                out.append(f"{label}: {bad.numel()} bytes written BEFORE the tensor (nearest at offset {first})")
            bad = (back != _PATTERN).nonzero()
            if bad.numel():
                out.append(f"{label}: {bad.numel()} bytes written AFTER the tensor (first at offset "
                           f"{nbytes + int(bad.min())} of a {nbytes}-byte payload)")
        return out

    def check(self):
        v = self.violations()
        if v:
            raise CanaryError("out-of-bounds writes detected:\n  " + "\n  ".join(v))


_ORIG = {name: getattr(torch, name) for name in _PATCHED}


def _call_site() -> str:
    for fr in reversed(traceback.extract_stack(limit=8)):
        if not fr.filename.endswith("ops/debug.py"):
            return f"{fr.filename.rsplit('/', 1)[-1]}:{fr.lineno}"
    return "?"


@contextlib.contextmanager
def canary_arena(device_types: Iterable[str] = ("cuda",), check: bool = True):
    """Route this thread's (and, the patch being process-wide, every thread's) ``torch.empty``-family
    allocations on ``device_types`` through a :class:`CanaryArena`; verify the guard bands on exit."""
    arena = CanaryArena()
    kinds = tuple(device_types)

    def watched(device) -> bool:
        return device is not None and torch.device(device).type in kinds

    def make_new(name, zero):
        orig = _ORIG[name]

        def fn(*size, dtype=None, device=None, **kw):
            if kw or not watched(device):
                return orig(*size, dtype=dtype, device=device, **kw)
            shape = size[0] if len(size) == 1 and isinstance(size[0], (tuple, list, torch.Size)) else size
            return arena.alloc(shape, dtype or torch.get_default_dtype(), device, zero,
                               f"{name}{tuple(shape)} {dtype} at {_call_site()}")
        return fn

    def make_like(name, zero):
        orig = _ORIG[name]

        def fn(t, dtype=None, device=None, **kw):
            dev = device if device is not None else t.device
            if kw or not watched(dev) or not t.is_contiguous():
                return orig(t, dtype=dtype, device=device, **kw)
            return arena.alloc(t.shape, dtype or t.dtype, dev, zero,
                               f"{name}{tuple(t.shape)} {dtype or t.dtype} at {_call_site()}")
        return fn

    patches = {"empty": make_new("empty", False), "zeros": make_new("zeros", True),
               "empty_like": make_like("empty_like", False), "zeros_like": make_like("zeros_like", True)}
    for name, fn in patches.items():
        setattr(torch, name, fn)
    try:
        yield arena
    finally:
        for name in _PATCHED:
            setattr(torch, name, _ORIG[name])
    if check:
        arena.check()
