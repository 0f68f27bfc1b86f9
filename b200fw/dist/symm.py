"""Symmetric (peer-mapped) device memory and cross-GPU flags for the in-kernel communication paths.

Every rank of a group allocates a buffer of the same size; after the rendezvous each rank knows the
device pointer of every peer's buffer and the kernels in ``csrc/comm.cu`` and the fused GEMMs read and
write them directly over NVLink.  Allocation and handle exchange use PyTorch's symmetric-memory
allocator (CUDA VMM handles exchanged through the process group's store); the reference has no
counterpart — its collectives are NCCL calls (src/distributed/comm.py:35-120).

Cross-GPU ordering uses ``FlagBarrier``: a small int32 flag buffer per rank, one slot per (source rank,
channel).  ``signal`` writes a monotonically increasing epoch into every peer's slot with a
system-scope release; ``wait`` spins with a time limit on this rank's own slots and records a failure in
the device status word instead of trapping or spinning forever.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _native as nv


class SymmetricBuffer:
    def __init__(self, numel: int, dtype: torch.dtype, group, device: Optional[torch.device] = None):
        import torch.distributed._symmetric_memory as symm
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.tensor = symm.empty(numel, dtype=dtype, device=self.device)
        self.handle = symm.rendezvous(self.tensor, group=group)
        self.peer_ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
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

    def __init__(self, group, device: Optional[torch.device] = None, limit_ms: int = 2000):
        self.buf = SymmetricBuffer(8 * self.CHANNELS, torch.int32, group, device)
        self.world, self.rank = self.buf.world, self.buf.rank
        self.limit_ms = limit_ms
        self.epoch = [0] * self.CHANNELS
        self.result = torch.ones(1, dtype=torch.int32, device=self.buf.device)
        dist.barrier(group=group)     # everyone's flags are zeroed before anyone signals

    def signal(self, channel: int = 0) -> int:
        self.epoch[channel] += 1
        nv.check(nv.lib().b2_flag_signal_all(self.buf.ptr_array, self.world, self.rank, self.CHANNELS, channel,
                                             self.epoch[channel], nv.stream_ptr()), "flag_signal_all")
        nv.count_launch()
        return self.epoch[channel]

    def wait(self, channel: int = 0, epoch: Optional[int] = None) -> None:
        nv.check(nv.lib().b2_flag_wait_all(nv.ptr(self.buf.tensor), self.world, self.CHANNELS, channel,
                                           self.epoch[channel] if epoch is None else epoch, self.limit_ms,
                                           nv.ptr(self.result), nv.stream_ptr()), "flag_wait_all")
        nv.count_launch()

    def barrier(self, channel: int = 0) -> None:
        """Stream-ordered barrier over the group: work queued before it on every rank is complete (and
        visible) before work queued after it starts on any rank."""
        self.signal(channel)
        self.wait(channel)

    def ok(self) -> bool:
        """Host check (synchronises): did the last wait succeed?"""
        return bool(int(self.result.item()))
