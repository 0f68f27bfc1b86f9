"""CUDA-graph decode: one captured graph per batch size with static input buffers.

Same behaviour as the reference's CUDAGraphRunner (src/inference/cuda_graph.py:30-233): capture sizes
1, 2, 4, ... up to a maximum, three warm-up runs before each capture, a shared memory pool, ``replay``
pads the batch to the next captured size and returns a clone of the static output, ``invalidate``
drops every graph.  Because weight updates are written in place, graphs stay valid across weight
syncs; only shape changes (block-table width) force a re-capture.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch


class CUDAGraphRunner:
    def __init__(self, max_batch_size: int = 256, warmups: int = 3):
        self.sizes = [s for s in (1, 2, 4, 8, 16, 32, 64, 128, 256, 512) if s <= max_batch_size]
        if not self.sizes or self.sizes[-1] < max_batch_size:
            self.sizes.append(max_batch_size)
        self.warmups = warmups
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.static_in: Dict[int, Dict[str, torch.Tensor]] = {}
        self.static_out: Dict[int, torch.Tensor] = {}
        self.pool = None
        self.replays = 0
        self.captures = 0

    def padded_size(self, n: int) -> Optional[int]:
        for s in self.sizes:
            if s >= n:
                return s
        return None

    def has(self, size: int) -> bool:
        return size in self.graphs

    def is_captured(self, batch_size: int) -> bool:
        """True when the bucket that ``batch_size`` pads to has a graph (src/inference/cuda_graph.py:207-210)."""
        padded = self.padded_size(batch_size)
        return padded is not None and padded in self.graphs

    def capture(self, size: int, make_inputs: Callable[[int], Dict[str, torch.Tensor]],
                fn: Callable[[Dict[str, torch.Tensor]], torch.Tensor]):
        """``make_inputs(size)`` returns the static input tensors; ``fn(inputs)`` is the step."""
        inputs = make_inputs(size)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(self.warmups):
                fn(inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
        with torch.cuda.graph(g, pool=self.pool):
            out = fn(inputs)
        self.graphs[size], self.static_in[size], self.static_out[size] = g, inputs, out
        self.captures += 1

    def replay(self, size: int, inputs: Dict[str, torch.Tensor]):
        """Copy ``inputs`` (same keys, leading dim <= size) into the static buffers and replay."""
        static = self.static_in[size]
        for k, v in inputs.items():
            dst = static[k]
            if v.shape == dst.shape:
                dst.copy_(v, non_blocking=True)
            else:
                idx = tuple(slice(0, s) for s in v.shape)
                dst[idx].copy_(v, non_blocking=True)
        self.graphs[size].replay()
        self.replays += 1
        out = self.static_out[size]
        return tuple(o.clone() for o in out) if isinstance(out, tuple) else out.clone()

    def invalidate(self):
        self.graphs.clear()
        self.static_in.clear()
        self.static_out.clear()

    def get_stats(self) -> dict:
        return {"captured_sizes": sorted(self.graphs), "captures": self.captures, "replays": self.replays}
