"""Collectives, tensor-parallel autograd regions, async all-reduce with a bounded host wait, and
pipeline p2p primitives.

These wrap ``torch.distributed`` (NCCL on GPUs, gloo on CPUs) and are the control plane and the
measured baseline; the fused compute+collective kernels live in :mod:`b200fw.ops.fused_tp` and
:mod:`b200fw.optim`.  ``group=None`` makes every collective a no-op, as in the reference
(src/distributed/comm.py:35-120).
"""
from __future__ import annotations

import time
from typing import List, Optional

import torch
import torch.distributed as dist

from .streams import StreamManager


def _size(group) -> int:
    return 1 if group is None else dist.get_world_size(group)


def all_reduce(t: torch.Tensor, group=None, op=dist.ReduceOp.SUM) -> torch.Tensor:
    if group is not None and _size(group) > 1:
        dist.all_reduce(t, op=op, group=group)
    return t


def all_gather(t: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenate along dim 0."""
    n = _size(group)
    if n == 1:
        return t
    out = torch.empty((n * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, t.contiguous(), group=group)
    return out


def all_gather_last_dim(t: torch.Tensor, group=None) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return t
    parts = [torch.empty_like(t) for _ in range(n)]
    dist.all_gather(parts, t.contiguous(), group=group)
    return torch.cat(parts, dim=-1)


def reduce_scatter(t: torch.Tensor, group=None, op=None) -> torch.Tensor:
    """Reduce over ranks (sum unless ``op`` says otherwise), keep this rank's dim-0 slice."""
    n = _size(group)
    if n == 1:
        return t
    assert t.shape[0] % n == 0
    out = torch.empty((t.shape[0] // n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    dist.reduce_scatter_tensor(out, t.contiguous(), op=op if op is not None else dist.ReduceOp.SUM, group=group)
    return out


def broadcast(t: torch.Tensor, src: int, group=None) -> torch.Tensor:
    if group is not None and _size(group) > 1:
        dist.broadcast(t, src=src, group=group)
    return t


# ---- tensor-parallel autograd regions (Megatron f / g operators) -------------------------------
class _CopyToParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        return all_reduce(g.contiguous().clone(), ctx.group), None


class _ReduceFromParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        return all_reduce(x.contiguous().clone(), group)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherFromParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather_last_dim(x, group)

    @staticmethod
    def backward(ctx, g):
        n = _size(ctx.group)
        if n == 1:
            return g, None
        r = dist.get_rank(ctx.group)
        return g.chunk(n, dim=-1)[r].contiguous(), None


class _GatherSeq(torch.autograd.Function):
    """Sequence-parallel all-gather along dim 0 (forward) / reduce-scatter (backward)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather(x, group)

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter(g.contiguous(), ctx.group), None


class _ScatterSeq(torch.autograd.Function):
    """Sequence-parallel reduce-scatter along dim 0 (forward) / all-gather (backward)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return reduce_scatter(x.contiguous(), group)

    @staticmethod
    def backward(ctx, g):
        return all_gather(g.contiguous(), ctx.group), None


class _ScatterToSeq(torch.autograd.Function):
    """Keep this rank's dim-0 slice of a replicated tensor (forward) / all-gather the gradient slices
    (backward), so that the producer of the replicated tensor sees its complete gradient."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n, r = _size(group), dist.get_rank(group)
        rows = x.shape[0] // n
        return x[r * rows:(r + 1) * rows]

    @staticmethod
    def backward(ctx, g):
        return all_gather(g.contiguous(), ctx.group), None


class _GatherSeqReplicated(torch.autograd.Function):
    """All-gather along dim 0 (forward) into a tensor that every rank then consumes identically;
    each rank's gradient of the gathered tensor is already complete, so backward keeps the local
    slice instead of reduce-scattering."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather(x, group)

    @staticmethod
    def backward(ctx, g):
        n, r = _size(ctx.group), dist.get_rank(ctx.group)
        rows = g.shape[0] // n
        return g[r * rows:(r + 1) * rows].contiguous(), None


def scatter_to_sequence_region(x, group=None):
    return x if group is None else _ScatterToSeq.apply(x, group)


def gather_sequence_replicated(x, group=None):
    return x if group is None else _GatherSeqReplicated.apply(x, group)


def copy_to_parallel_region(x, group=None):
    return x if group is None else _CopyToParallelRegion.apply(x, group)


def reduce_from_parallel_region(x, group=None):
    return x if group is None else _ReduceFromParallelRegion.apply(x, group)


def gather_from_parallel_region(x, group=None):
    return x if group is None else _GatherFromParallelRegion.apply(x, group)


class _ScatterToParallelRegion(torch.autograd.Function):
    """Keep this rank's slice of the last dim (forward) / all-gather the gradient slices along it (backward)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.chunk(_size(group), dim=-1)[dist.get_rank(group)].contiguous()

    @staticmethod
    def backward(ctx, g):
        return all_gather_last_dim(g.contiguous(), ctx.group), None


def scatter_to_parallel_region(x, group=None):
    return x if group is None else _ScatterToParallelRegion.apply(x, group)


def gather_sequence(x, group=None):
    return x if group is None else _GatherSeq.apply(x, group)


def reduce_scatter_sequence(x, group=None):
    return x if group is None else _ScatterSeq.apply(x, group)


# ---- async all-reduce with bounded host wait --------------------------------------------------
class AsyncHandle:
    """Completion handle whose ``wait`` polls instead of blocking forever.

    The reference polls a CUDA event every 10 ms and raises after 300 s
    (src/distributed/comm.py:313-352); the same host-side hang detection is kept here and works for
    both NCCL work objects and CUDA events.
    """

    def __init__(self, work=None, event=None, stream_manager: Optional[StreamManager] = None):
        self.work, self.event, self.sm = work, event, stream_manager
        self.done = work is None and event is None

    def is_completed(self) -> bool:
        if self.done:
            return True
        if self.event is not None:
            return self.event.query()
        return self.work.is_completed()

    def is_done(self) -> bool:
        """Non-blocking completion query (the reference's name: src/distributed/comm.py:355-359)."""
        return self.is_completed()

    def wait(self, timeout_sec: float = 300.0, poll_s: float = 0.01):
        if self.done:
            return
        t0 = time.time()
        if self.event is not None:
            while not self.event.query():
                if time.time() - t0 > timeout_sec:
                    raise RuntimeError(f"async collective did not complete within {timeout_sec}s")
                time.sleep(poll_s)
            if self.sm is not None:
                self.sm.sync_comm_to_compute()
        else:
            while not self.work.is_completed():
                if time.time() - t0 > timeout_sec:
                    raise RuntimeError(f"async collective did not complete within {timeout_sec}s")
                time.sleep(poll_s)
            self.work.wait()
        self.done = True


class AsyncAllReduce:
    """All-reduce issued on the communication stream; the caller overlaps compute and then waits."""

    def __init__(self, stream_manager: Optional[StreamManager] = None, group=None, timeout_sec: float = 300.0):
        # the reference's argument order is (group, stream_manager, timeout_sec): accept either
        if isinstance(group, StreamManager) or (stream_manager is not None and not isinstance(stream_manager, StreamManager)):
            stream_manager, group = (group if isinstance(group, StreamManager) else None), stream_manager
        self.sm, self.group, self.timeout_sec = stream_manager, group, timeout_sec

    @property
    def stream_manager(self):
        return self.sm

    def start(self, tensor: torch.Tensor) -> "AsyncHandle":
        """All-reduce ``tensor`` in place over the group given at construction; ``handle.wait()`` before use
        (src/distributed/comm.py:260-300)."""
        return self.launch(tensor, self.group)

    def launch(self, t: torch.Tensor, group=None) -> AsyncHandle:
        if group is None or _size(group) == 1:
            return AsyncHandle()
        if self.sm is not None and self.sm.enabled and t.is_cuda:
            self.sm.sync_compute_to_comm()
            with self.sm.comm_context():
                dist.all_reduce(t, group=group)
                ev = torch.cuda.Event()
                ev.record()
            return AsyncHandle(event=ev, stream_manager=self.sm)
        work = dist.all_reduce(t, group=group, async_op=True)
        return AsyncHandle(work=work)


def all_reduce_async(tensor: torch.Tensor, group, stream_manager: Optional[StreamManager] = None,
                     timeout_sec: float = 300.0) -> AsyncHandle:
    """``handle = all_reduce_async(t, group, sm)``; compute that does not need ``t``; ``handle.wait()``
    (src/distributed/comm.py:362-385)."""
    return AsyncAllReduce(stream_manager, group, timeout_sec).start(tensor)


# ---- pipeline p2p -------------------------------------------------------------------------------
def _batch(ops: List[dist.P2POp]):
    if not ops:
        return
    for w in dist.batch_isend_irecv(ops):
        w.wait()


def send_forward(t: torch.Tensor, dst: Optional[int], group=None):
    if dst is not None:
        _batch([dist.P2POp(dist.isend, t.contiguous(), dst, group)])


def recv_forward(shape, dtype, device, src: Optional[int], group=None) -> Optional[torch.Tensor]:
    if src is None:
        return None
    buf = torch.empty(tuple(shape), dtype=dtype, device=device)
    _batch([dist.P2POp(dist.irecv, buf, src, group)])
    return buf


def send_backward(t: torch.Tensor, dst: Optional[int], group=None):
    if dst is not None:
        _batch([dist.P2POp(dist.isend, t.contiguous(), dst, group)])


def recv_backward(shape, dtype, device, src: Optional[int], group=None) -> Optional[torch.Tensor]:
    if src is None:
        return None
    buf = torch.empty(tuple(shape), dtype=dtype, device=device)
    _batch([dist.P2POp(dist.irecv, buf, src, group)])
    return buf


def send_forward_recv_backward(out: torch.Tensor, shape, dtype, device, peer: Optional[int], group=None):
    """Send activations to the next stage and receive the gradient for an earlier micro-batch from
    it in one batched call, which cannot deadlock in the 1F1B steady state."""
    if peer is None:
        return None
    buf = torch.empty(tuple(shape), dtype=dtype, device=device)
    _batch([dist.P2POp(dist.isend, out.contiguous(), peer, group), dist.P2POp(dist.irecv, buf, peer, group)])
    return buf


def send_backward_recv_forward(grad: torch.Tensor, shape, dtype, device, peer: Optional[int], group=None):
    if peer is None:
        return None
    buf = torch.empty(tuple(shape), dtype=dtype, device=device)
    _batch([dist.P2POp(dist.isend, grad.contiguous(), peer, group), dist.P2POp(dist.irecv, buf, peer, group)])
    return buf


class PipeChannel:
    """One direction of one pipeline-stage boundary: an ordered stream of equally shaped tensors to ``peer`` (a
    sender) or from it (a receiver), on a communicator and a CUDA stream of its own.

    The reference's stage-to-stage primitives (src/distributed/comm.py:404-558) post a send / receive pair and wait
    for it on the compute stream, with a fresh receive buffer per call.  Here activations (downstream) and
    gradients (upstream) travel on separate communicators and a send never holds the compute stream:

    * ``post_recv()`` enqueues the receive into the next buffer of a persistent ring on the communication stream
      (which first waits for the compute work queued so far: the buffer's previous use is over) and returns a handle;
      ``wait(handle)`` makes the compute stream wait for it and returns the buffer.  Post a receive where its data
      is used: an NCCL receive occupies the GPU until its sender arrives, and left pending ahead of unrelated compute
      it can stall that compute when streams outnumber the hardware queues.
    * ``send(t)`` enqueues the send on the communication stream after the compute work that produced ``t``; the
      compute stream does not wait for it.

    On CPU (gloo) the same calls are plain ``irecv`` / ``isend`` with ``wait`` at the matching point."""

    def __init__(self, group, peer: Optional[int], shape, dtype, device, depth: int = 4):
        self.group, self.peer = group, peer
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.ring = [torch.empty(tuple(shape), dtype=dtype, device=device) for _ in range(depth)] if peer is not None else []
        self.next = 0
        self.stream = torch.cuda.Stream(device=self.device) if (self.cuda and peer is not None) else None
        self._sends: List = []

    def post_recv(self):
        if self.peer is None:
            return None
        buf = self.ring[self.next % len(self.ring)]
        self.next += 1
        if self.cuda:
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                work = dist.irecv(buf, src=self.peer, group=self.group)
        else:
            work = dist.irecv(buf, src=self.peer, group=self.group)
        return buf, work

    def wait(self, handle) -> Optional[torch.Tensor]:
        if handle is None:
            return None
        buf, work = handle
        work.wait()          # NCCL: the current (compute) stream waits for the transfer; gloo: the host does
        return buf

    def send(self, t: torch.Tensor):
        if self.peer is None:
            return
        t = t.contiguous()
        if self.cuda:
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                work = dist.isend(t, dst=self.peer, group=self.group)
            t.record_stream(self.stream)
        else:
            work = dist.isend(t, dst=self.peer, group=self.group)
        self._sends = [(w, x) for w, x in self._sends if not w.is_completed()] + [(work, t)]

    def flush(self):
        """End of a schedule: every send has left (gloo needs the explicit wait; on NCCL this orders the
        communication stream before whatever the compute stream does next with the sent tensors' memory)."""
        for w, _ in self._sends:
            w.wait()
        self._sends = []
