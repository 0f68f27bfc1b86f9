"""Symmetric (peer-mapped) device memory and cross-GPU flags for the in-kernel communication paths.

Every rank of a group allocates a buffer of the same size; after the rendezvous each rank knows the
device pointer of every peer's buffer and the kernels in ``csrc/comm.cu`` and the fused GEMMs read and
write them directly over NVLink.  Allocation and handle exchange use PyTorch's symmetric-memory
allocator (CUDA VMM handles exchanged through the process group's store); the reference has no
counterpart — its collectives are NCCL calls (src/distributed/comm.py:35-120).  Where the platform binds
the allocation to an NVLink multicast object (NVSwitch with NVLS), ``mc_ptr`` is its multicast address:
``multimem.ld_reduce`` on it returns the sum over all ranks' buffers, ``multimem.st`` writes all of them.
``B200FW_NVLS=0`` makes every path use plain peer loads and stores instead.

Cross-GPU ordering uses ``FlagBarrier``: a small int32 flag buffer per rank, one slot per (source rank,
channel).  Two forms: ``signal`` / ``wait`` take the epoch from the host (one kernel each); ``barrier_dev``
is one launch whose epoch counter lives on the device, so it can be captured in a CUDA graph and replayed.
A channel is used with one form only.  Every wait is bounded in time and records a failure in the device
status word (and clears ``ok``) instead of trapping or spinning forever.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _native as nv


def nvls_enabled() -> bool:
    return os.environ.get("B200FW_NVLS", "1") != "0"


class SymmetricBuffer:
    def __init__(self, numel: int, dtype: torch.dtype, group, device: Optional[torch.device] = None):
        import torch.distributed._symmetric_memory as symm
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.tensor = symm.empty(numel, dtype=dtype, device=self.device)
        self.handle = symm.rendezvous(self.tensor, group=group)
        bases = [int(p) for p in self.handle.buffer_ptrs]
        # the tensor may sit at an offset inside the allocation the handle describes
        off = int(self.tensor.data_ptr()) - bases[self.rank]
        if off < 0 or off >= (1 << 40):
            off = 0
        self.peer_ptrs: List[int] = [b + off for b in bases]
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.mc_ptr: int = (mc + off) if (mc and nvls_enabled()) else 0
        self.tensor.zero_()
        self._arr = (ctypes.c_void_p * self.world)(*self.peer_ptrs)

    @property
    def ptr_array(self):
        """``void* const*`` argument for the launchers (host array of peer pointers)."""
        return self._arr

    def offset_ptr_array(self, byte_offset: int):
        return (ctypes.c_void_p * self.world)(*[p + byte_offset for p in self.peer_ptrs])


class FlagBarrier:
    CHANNELS = 8

    def __init__(self, group, device: Optional[torch.device] = None, limit_ms: int = 2000, channels: int = 0):
        self.channels = int(channels) if channels else self.CHANNELS
        self.buf = SymmetricBuffer(8 * self.channels, torch.int32, group, device)
        self.world, self.rank = self.buf.world, self.buf.rank
        self.limit_ms = limit_ms
        self.epoch = [0] * self.channels
        self.result = torch.ones(1, dtype=torch.int32, device=self.buf.device)
        # device-side epochs of the one-launch barrier, and its sticky "every wait so far succeeded" word
        self.epochs_dev = torch.zeros(self.channels, dtype=torch.int32, device=self.buf.device)
        self.ok_dev = torch.ones(1, dtype=torch.int32, device=self.buf.device)
        dist.barrier(group=group)     # everyone's flags are zeroed before anyone signals

    def signal(self, channel: int = 0) -> int:
        self.epoch[channel] += 1
        nv.check(nv.lib().b2_flag_signal_all(self.buf.ptr_array, self.world, self.rank, self.channels, channel,
                                             self.epoch[channel], nv.stream_ptr()), "flag_signal_all")
        nv.count_launch()
        return self.epoch[channel]

    def wait(self, channel: int = 0, epoch: Optional[int] = None) -> None:
        nv.check(nv.lib().b2_flag_wait_all(nv.ptr(self.buf.tensor), self.world, self.channels, channel,
                                           self.epoch[channel] if epoch is None else epoch, self.limit_ms,
                                           nv.ptr(self.result), nv.stream_ptr()), "flag_wait_all")
        nv.count_launch()

    def barrier(self, channel: int = 0) -> None:
        """Stream-ordered barrier over the group: work queued before it on every rank is complete (and
        visible) before work queued after it starts on any rank."""
        self.signal(channel)
        self.wait(channel)

    def barrier_dev(self, channel: int) -> None:
        """The same barrier as one launch with the epoch kept on the device (CUDA-graph capturable).  Every rank
        must issue the same sequence of calls per channel.  A wait that runs out clears ``ok_dev``."""
        nv.check(nv.lib().b2_flag_barrier(self.buf.ptr_array, nv.ptr(self.buf.tensor), nv.ptr(self.epochs_dev),
                                          self.world, self.rank, self.channels, channel, self.limit_ms,
                                          nv.ptr(self.ok_dev), nv.stream_ptr()), "flag_barrier")
        nv.count_launch()

    def ok(self) -> bool:
        """Host check (synchronises): did every wait so far succeed?"""
        return bool(int(self.result.item())) and bool(int(self.ok_dev.item()))

    def reset_ok(self) -> None:
        self.result.fill_(1)
        self.ok_dev.fill_(1)


class NormAllReduce:
    """Sum of two fp32 scalars over the group in one kernel (slots in peer memory + the device-epoch barrier of
    ``flags`` on ``channel``); writes the total and its square root (``-1`` when not finite)."""

    def __init__(self, flags: FlagBarrier, group, channel: int, device: Optional[torch.device] = None):
        self.flags, self.channel = flags, channel
        self.slots = SymmetricBuffer(32, torch.float32, group, device)

    def __call__(self, parts: torch.Tensor, norm_sq: torch.Tensor, grad_norm: torch.Tensor) -> None:
        f = self.flags
        nv.check(nv.lib().b2_norm_allreduce(self.slots.ptr_array, nv.ptr(self.slots.tensor), f.buf.ptr_array,
                                            nv.ptr(f.buf.tensor), nv.ptr(f.epochs_dev), f.world, f.rank, f.channels,
                                            self.channel, nv.ptr(parts), nv.ptr(norm_sq), nv.ptr(grad_norm),
                                            f.limit_ms, nv.ptr(f.ok_dev), nv.stream_ptr()), "norm_allreduce")
        nv.count_launch()
