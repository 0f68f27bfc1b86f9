"""Tensor-parallel linear layers whose collective runs INSIDE the tcgen05 GEMM kernel.

* :func:`allgather_gemm`   — column-parallel forward (and the input-gradient GEMM of a row-parallel
  layer): extra warps of the GEMM kernel push this rank's sequence-parallel activation shard into every
  rank's gather buffer (one ``multimem.st`` through the switch per 16 bytes where NVLS is available, else one
  store per peer) while the MMA pipeline already works on the row blocks whose pieces have all arrived.
* :func:`gemm_reduce_scatter` — row-parallel forward (and the input-gradient GEMM of a column-parallel
  layer): every output tile goes straight to the rank that owns those rows; each rank sums its rows
  over the source ranks (and adds the residual) as soon as the tiles land.

Replaces ``all_gather`` / ``all_reduce`` + ``F.linear`` pairs of the reference's parallel layers
(src/distributed/tensor_parallel.py:156-159,236-239; the reference all-reduces replicated activations,
it has no sequence parallelism).  Buffers live in symmetric memory (:mod:`b200fw.dist.symm`); two
parities alternate so that a rank that runs ahead never overwrites data a peer still reads; counters
and flags only grow (epochs), nothing is reset between calls.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native as nv
from ..dist.symm import FlagBarrier, SymmetricBuffer
from .gemm import gemm, grad_into_main


import os as _os

_AG_NVLS = _os.environ.get("B200FW_AG_NVLS", "auto")     # "1" / "0" force multimem stores on / off in all-gather -> GEMM


class _RSState:
    def __init__(self, group, rows, N, bn, device):
        self.world = dist.get_world_size(group)
        nb = (N + bn - 1) // bn
        self.recv = [SymmetricBuffer(self.world * rows * N, torch.bfloat16, group, device) for _ in range(2)]
        self.cnt = [SymmetricBuffer((rows // 128) * nb, torch.int32, group, device) for _ in range(2)]
        self.epoch = [0, 0]
        self.calls = 0


class _AGSlot:
    """The gather buffers of one call site ("slot"): two parities of a symmetric ``[M, K]`` buffer with their
    arrival counters.  The gathered activations a call returns ARE the buffer (no copy): a slot must not be used
    again twice before the tensor returned earlier has been consumed (``generation`` lets the consumer check)."""

    def __init__(self, group, rows, K, device):
        self.world = dist.get_world_size(group)
        M = rows * self.world
        self.buf = [SymmetricBuffer(M * K, torch.bfloat16, group, device) for _ in range(2)]
        self.flags = [SymmetricBuffer(M // 128, torch.int32, group, device) for _ in range(2)]
        self.uses = [0, 0]
        self.calls = 0


class FusedTPContext:
    """Per-TP-group workspace cache and the flag barrier that orders buffer reuse across ranks."""

    _by_group: Dict[int, "FusedTPContext"] = {}

    def __init__(self, group):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.rs: Dict[Tuple[int, int, int], _RSState] = {}
        self.ag: Dict[tuple, _AGSlot] = {}
        self.barrier = FlagBarrier(group, self.device)
        # "rank p has entered fused all-gather call number c": written by the peers, read by the push warps
        self.ag_ready = SymmetricBuffer(8, torch.int32, group, self.device)
        self.ag_calls = 0

    @classmethod
    def get(cls, group) -> "FusedTPContext":
        key = id(group)
        if key not in cls._by_group:
            cls._by_group[key] = cls(group)
        return cls._by_group[key]


def _bn_for(M: int, N: int) -> int:
    return 256 if (N % 256 == 0 and ((M + 127) // 128) * (N // 256) >= 148) else 128


def gemm_reduce_scatter(x: torch.Tensor, w: torch.Tensor, group, *, b_mn: bool = False,
                        residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``reduce_scatter_rows(x @ w^T) (+ residual)``: ``x [M, K_local]``, ``w [N, K_local]`` (or
    ``[K_local, N]`` with ``b_mn``); returns this rank's ``[M/world, N]`` rows."""
    ctx = FusedTPContext.get(group)
    M, K = x.shape
    N = w.shape[1] if b_mn else w.shape[0]
    rows = M // ctx.world
    assert M % ctx.world == 0 and rows % 128 == 0 and x.is_contiguous() and w.stride(-1) == 1
    bn = _bn_for(M, N)
    key = (rows, N, bn)
    st = ctx.rs.get(key)
    if st is None:
        st = ctx.rs[key] = _RSState(group, rows, N, bn, ctx.device)
        ctx.barrier.barrier(2)       # everyone's buffers exist and are zeroed before the first tile lands
    par = st.calls & 1
    st.calls += 1
    st.epoch[par] += 1
    out = torch.empty((rows, N), device=x.device, dtype=torch.bfloat16)
    if residual is not None:
        assert residual.shape == (rows, N) and residual.is_contiguous()
    nv.check(nv.lib().b2_gemm_bf16_comm(
        1, nv.ptr(x), nv.ptr(w), nv.ptr(None), M, N, K, w.stride(0), int(b_mn), bn, st.recv[par].ptr_array,
        st.cnt[par].ptr_array, nv.ptr(out), nv.ptr(residual), None, nv.ptr(None), None, None, 0, ctx.world, ctx.rank,
        rows, st.epoch[par], nv.stream_ptr()), "gemm_reduce_scatter")
    nv.count_launch()
    return out


def allgather_gemm(x_shard: torch.Tensor, w: torch.Tensor, group, *, b_mn: bool = False, slot=None
                   ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``all_gather_rows(x_shard) @ w^T``: ``x_shard [M/world, K]``; returns ``(y [M, N], gathered x
    [M, K])`` — the gathered activations are kept for the weight-gradient GEMM.

    ``slot`` names the call site whose (double-buffered) symmetric gather buffers are used; the returned
    ``gathered`` is then a view of the buffer and stays valid until the slot's second next call.  Callers whose
    gathered activations live longer (saved for a backward pass that runs after other calls of the same shape) pass
    a slot of their own; without a slot the buffers are shared per shape and ``gathered`` is a private copy whenever
    autograd is recording."""
    ctx = FusedTPContext.get(group)
    rows, K = x_shard.shape
    N = w.shape[1] if b_mn else w.shape[0]
    M = rows * ctx.world
    assert rows % 128 == 0 and w.stride(-1) == 1 and x_shard.is_contiguous()
    key = ("slot", slot, rows, K) if slot is not None else ("shape", rows, K)
    st = ctx.ag.get(key)
    if st is None:
        st = ctx.ag[key] = _AGSlot(group, rows, K, ctx.device)
        ctx.barrier.barrier(3)       # everyone's buffers and counters exist (zeroed) before the first piece lands
    par = st.calls & 1
    st.calls += 1
    st.uses[par] += 1
    ctx.ag_calls += 1
    buf, flags = st.buf[par], st.flags[par]
    y = torch.empty((M, N), device=x_shard.device, dtype=torch.bfloat16)
    bn = _bn_for(M, N)
    # one multimem.st per 16 bytes reaches every rank; with two ranks there is nothing to save and plain stores
    # measured faster (F1 0.246 vs 0.322 ms), with four the switch wins on the long GEMM (F2 0.809 vs 0.873 ms)
    mc = buf.mc_ptr if (ctx.world > 2 or _AG_NVLS == "1") and _AG_NVLS != "0" else 0
    nv.check(nv.lib().b2_gemm_bf16_comm(
        2, nv.ptr(x_shard), nv.ptr(w), nv.ptr(y), M, N, K, w.stride(0), int(b_mn), bn, None, None, nv.ptr(None),
        nv.ptr(None), buf.ptr_array, nv.ctypes.c_void_p(mc), flags.ptr_array, ctx.ag_ready.ptr_array,
        ctx.ag_calls, ctx.world, ctx.rank, rows, st.uses[par], nv.stream_ptr()), "allgather_gemm")
    nv.count_launch()
    gathered = buf.tensor.view(M, K)
    if slot is None and torch.is_grad_enabled():
        gathered = gathered.clone()
    return y, gathered


# Every contraction length takes the fused kernel: with reductions on their own warps, row blocks scheduled so that
# they complete progressively, and one cumulative release per tile, the short-K case (o_proj, K = 1024 per rank at
# TP8: the GEMM is 0.12 ms, the wire 0.11-0.19 ms) runs 0.28 / 0.30 ms at 2 / 4 GPUs against 0.39 / 0.40 ms for the
# plain GEMM followed by NCCL's reduce-scatter.  The threshold stays as a knob (contractions shorter than it use NCCL).
FUSED_RS_MIN_K = 0


def _reduce_scatter_gemm(x: torch.Tensor, w: torch.Tensor, group, *, b_mn: bool = False,
                         residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    K = x.shape[1]
    if K >= FUSED_RS_MIN_K:
        return gemm_reduce_scatter(x, w, group, b_mn=b_mn, residual=residual)
    from ..dist import comm
    y = comm.reduce_scatter(gemm(x, w, b_mn=b_mn), group)
    return y if residual is None else y.add_(residual)


class _ColumnLinearSP(torch.autograd.Function):
    """y = all_gather(x) @ W^T with the gather inside the GEMM; backward: dx = reduce_scatter(dy @ W)
    inside the GEMM, dW = dy^T @ gathered x."""

    @staticmethod
    def forward(ctx, x, w, group, slot):
        y, xg = allgather_gemm(x, w, group, slot=slot)
        ctx.save_for_backward(xg, w)
        ctx.group = group
        return y

    @staticmethod
    def backward(ctx, dy):
        xg, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = _reduce_scatter_gemm(dy, w, ctx.group, b_mn=True)
        dw = grad_into_main(w, lambda out, acc: gemm(dy, xg, a_mn=True, b_mn=True, out=out, accumulate=acc))
        return dx, dw, None, None


class _RowLinearSP(torch.autograd.Function):
    """y = reduce_scatter(x @ W^T) + residual inside the GEMM; backward: dx = all_gather(dy) @ W with
    the gather inside the GEMM, dW = gathered dy^T @ x."""

    @staticmethod
    def forward(ctx, x, w, residual, group):
        ctx.save_for_backward(x, w)
        ctx.group = group
        ctx.has_res = residual is not None
        return _reduce_scatter_gemm(x, w, group, residual=residual)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        # the gathered gradient is consumed by the weight-gradient GEMM right below: one shared slot serves every layer
        dx, dyg = allgather_gemm(dy, w, ctx.group, b_mn=True, slot="backward")
        dw = grad_into_main(w, lambda out, acc: gemm(dyg, x, a_mn=True, b_mn=True, out=out, accumulate=acc))
        return dx, dw, (dy if ctx.has_res else None), None


def column_linear_sp(x: torch.Tensor, w: torch.Tensor, group, slot=None) -> torch.Tensor:
    """``slot``: see :func:`allgather_gemm` (the gathered input is saved for the weight gradient)."""
    return _ColumnLinearSP.apply(x.contiguous(), w, group, slot)


def row_linear_sp(x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor], group) -> torch.Tensor:
    return _RowLinearSP.apply(x.contiguous(), w, residual, group)


def supported(x_rows_local_or_total: int, world: int, sharded_rows: bool) -> bool:
    rows = x_rows_local_or_total if sharded_rows else x_rows_local_or_total // max(world, 1)
    return rows > 0 and rows % 128 == 0 and world <= 8
