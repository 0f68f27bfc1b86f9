"""ctypes binding of the in-tree sm_100a kernel library (``b200fw/_lib/libb200fw.so``).

The library is loaded on first use.  On a machine with a CUDA device a missing or unloadable library
is an error (the CUDA ops never fall back silently to PyTorch); on a CPU-only machine the ops layer
never calls into it.
"""
from __future__ import annotations

import ctypes  # noqa: F401  (re-exported: ops use nv.ctypes)
import threading
from typing import Optional

import torch

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


class NativeError(RuntimeError):
    """A launcher rejected its arguments, a launch failed, or a kernel recorded an error status."""


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            from . import _build

            path = _build.LIB_PATH
            if not path.exists():
                path = _build.build()
            handle = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
            handle.b2_last_error.restype = ctypes.c_char_p
            handle.b2_status_read_and_clear.restype = ctypes.c_int
            if torch.cuda.is_available():
                handle.b2_set_device(int(torch.cuda.current_device()))
            _lib = handle
    return _lib


def available() -> bool:
    """True when kernels can run here: a CUDA device is present (the library is then mandatory)."""
    return torch.cuda.is_available()


def last_error() -> str:
    return lib().b2_last_error().decode(errors="replace")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what} failed (rc={rc}): {last_error()}")


def read_status() -> int:
    """Synchronise and return the device status word (0 = ok), clearing it."""
    return int(lib().b2_status_read_and_clear())


def assert_ok(what: str = "kernel") -> None:
    st = read_status()
    if st != 0:
        raise NativeError(f"{what}: device status {st} (a bounded wait ran out or an argument was rejected)")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = -1


def stream_ptr() -> ctypes.c_void_p:
    """The current CUDA stream of this process's device as a raw handle.  Called once per kernel launch:
    the raw-handle query is ~50x cheaper than building a ``torch.cuda.Stream`` object each time."""
    global _device_index
    if _raw_stream is not None:
        if _device_index < 0:
            _device_index = torch.cuda.current_device()
        return ctypes.c_void_p(_raw_stream(_device_index))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


# number of kernel launches issued through this binding (bench.py reports it)
launch_count = 0


def count_launch(n: int = 1) -> None:
    global launch_count
    launch_count += n


def set_device(index: int) -> None:
    """Tell the kernel library which device this process drives (call after torch.cuda.set_device)."""
    global _device_index
    if torch.cuda.is_available():
        lib().b2_set_device(int(index))
        _device_index = int(index)
