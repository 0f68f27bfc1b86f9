"""NVTX ranges around the phases of a training step, an inference step and a weight sync.

Off by default (a disabled range is one attribute test and a shared null context).  Enable with
``B200FW_NVTX=1`` in the environment or ``nvtx.enable()``; the ranges then show up in Nsight Systems /
Nsight Compute (``ncu --nvtx --nvtx-include "train/micro_step/"`` limits a capture to one phase).  The
reference has no NVTX or profiler integration (its timers are CUDA-event context managers:
src/profiling/comm_profiler.py:53-99, src/profiling/compute_profiler.py:254-284).
"""
from __future__ import annotations

import contextlib
import functools
import os

import torch

__all__ = ["enable", "enabled", "range", "annotate"]

_state = {"on": os.environ.get("B200FW_NVTX", "0") == "1", "pushed": 0}
_NULL = contextlib.nullcontext()


def enable(on: bool = True):
    _state["on"] = bool(on)


def enabled() -> bool:
    return _state["on"]


class _Range:
    __slots__ = ("name",)

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        _state["pushed"] += 1
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()
        return False


def range(name: str):  # noqa: A001 - mirrors torch.cuda.nvtx.range
    """Context manager: an NVTX range when enabled, a shared no-op otherwise."""
    return _Range(name) if _state["on"] else _NULL


def annotate(name: str):
    """Decorator form of :func:`range`."""
    def deco(fn):
        @functools.wraps(fn)
        def wrapped(*a, **k):
            if not _state["on"]:
                return fn(*a, **k)
            with _Range(name):
                return fn(*a, **k)
        return wrapped
    return deco
