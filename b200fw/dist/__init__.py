"""Distributed runtime: 3-D process groups, collectives, PP p2p, streams, symmetric memory."""
from .context import ParallelContext
from .comm import (
    all_reduce, all_gather, all_gather_last_dim, reduce_scatter, broadcast,
    copy_to_parallel_region, reduce_from_parallel_region, gather_from_parallel_region,
    AsyncAllReduce, AsyncHandle,
    send_forward, recv_forward, send_backward, recv_backward,
    send_forward_recv_backward, send_backward_recv_forward,
)
from .streams import StreamManager
from .heartbeat import PeerLostError, RankHeartbeat

__all__ = [
    "ParallelContext", "all_reduce", "all_gather", "all_gather_last_dim", "reduce_scatter",
    "broadcast", "copy_to_parallel_region", "reduce_from_parallel_region",
    "gather_from_parallel_region", "AsyncAllReduce", "AsyncHandle", "send_forward", "recv_forward",
    "send_backward", "recv_backward", "send_forward_recv_backward", "send_backward_recv_forward",
    "StreamManager", "PeerLostError", "RankHeartbeat",
]
