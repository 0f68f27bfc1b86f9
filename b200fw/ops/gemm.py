"""bf16 GEMM on the tcgen05 kernel and the autograd ``linear`` built on it.

Reference call sites this replaces: ``F.linear`` in ColumnParallelLinear / RowParallelLinear
(src/distributed/tensor_parallel.py:159,236).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as nv

OUT_FP32, ACCUMULATE, RESIDUAL = 1, 2, 4


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, accumulate: bool = False,
         residual: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
         bn: int = 0, max_ctas: int = 0) -> torch.Tensor:
    """``C[M,N] (+)= A @ B^T (+ residual)``.

    ``a`` is ``[M,K]`` (or ``[K,M]`` when ``a_mn``); ``b`` is ``[N,K]`` (or ``[K,N]`` when ``b_mn``).
    Rows may be strided (last dim contiguous).  CUDA bf16 inputs run the tcgen05 kernel; CPU inputs
    run ``torch.matmul`` in the input dtype.
    """
    if not a.is_cuda:
        A = a.t() if a_mn else a
        Bm = b.t() if b_mn else b
        r = A.float() @ Bm.float().t()
        if residual is not None:
            r = r + residual.float()
        if out is not None:
            if accumulate:
                out.add_(r.to(out.dtype))
            else:
                out.copy_(r.to(out.dtype))
            return out
        return r.to(out_dtype if a.dtype == torch.bfloat16 else a.dtype)
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "gemm: bf16 operands required on CUDA"
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, f"gemm: contraction mismatch {K} vs {Kb}"
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=out_dtype)
    else:
        assert out.shape == (M, N) and out.stride(-1) == 1
    flags = (OUT_FP32 if out.dtype == torch.float32 else 0) | (ACCUMULATE if accumulate else 0)
    if residual is not None:
        assert residual.shape == (M, N) and residual.stride(0) == out.stride(0) and residual.dtype == torch.bfloat16
        flags |= RESIDUAL
    rc = nv.lib().b2_gemm_bf16(nv.ptr(a), nv.ptr(b), nv.ptr(out), nv.ptr(residual), M, N, K,
                               a.stride(0), b.stride(0), out.stride(0), int(a_mn), int(b_mn), flags, bn,
                               max_ctas, nv.stream_ptr())
    nv.check(rc, "gemm")
    nv.count_launch()
    return out


class _NoGradCtx:
    """Stand-in for an autograd context when nothing will be differentiated (inference, evaluation): the ops call
    their ``forward`` with it directly and skip ``Function.apply``, whose bookkeeping costs several microseconds per
    call: a decode step issues about 300 such calls."""

    needs_input_grad = (False,) * 16

    def save_for_backward(self, *tensors):
        pass

    def __setattr__(self, name, value):      # forward() may park tensors on its context: keep none of them alive
        pass


NO_GRAD_CTX = _NoGradCtx()


def no_grad_needed(*tensors) -> bool:
    """True when autograd records nothing for an op over ``tensors``."""
    if not torch.is_grad_enabled():
        return True
    return not any(t is not None and t.requires_grad for t in tensors)


def grad_into_main(param: torch.Tensor, compute) -> Optional[torch.Tensor]:
    """Gradient-accumulation fusion.

    If ``param`` carries a ``main_grad`` buffer (set up by the optimizers in :mod:`b200fw.optim`),
    ``compute(out, accumulate)`` writes the weight gradient straight into it (accumulating from the
    second micro-batch on), the parameter's ``grad_ready`` hook fires, and ``None`` is returned to
    autograd.  Otherwise ``compute(None, False)`` returns a fresh gradient tensor for autograd.
    """
    mg = getattr(param, "main_grad", None)
    if mg is None:
        return compute(None, False)
    compute(mg, bool(getattr(param, "grad_filled", False)))
    param.grad_filled = True
    hook = getattr(param, "grad_ready_hook", None)
    if hook is not None:
        hook(param)
    return None


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, residual):
        ctx.save_for_backward(x, w)
        ctx.has_res = residual is not None
        return gemm(x, w, residual=residual)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy if dy.stride(-1) == 1 else dy.contiguous()
        dx = gemm(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = None
        if w.requires_grad:
            dw = grad_into_main(w, lambda out, acc: gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=acc))
        return dx, dw, (dy if ctx.has_res else None)


def linear(x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y = x @ w^T (+ residual)`` for 2-D ``x``; the residual add is fused in the GEMM epilogue."""
    if not x.is_cuda:
        y = torch.nn.functional.linear(x, w.to(x.dtype))
        return y if residual is None else y + residual
    if no_grad_needed(x, w, residual):
        return gemm(x, w, residual=residual)
    return _Linear.apply(x, w, residual)
