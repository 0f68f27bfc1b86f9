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
         bn: int = 0, max_ctas: int = 0, ext=None) -> torch.Tensor:
    """``C[M,N] (+)= A @ B^T (+ A2 @ B2^T) (+ residual)``.

    ``a`` is ``[M,K]`` (or ``[K,M]`` when ``a_mn``); ``b`` is ``[N,K]`` (or ``[K,N]`` when ``b_mn``).
    Rows may be strided (last dim contiguous).  CUDA bf16 inputs run the tcgen05 kernel; CPU inputs
    run ``torch.matmul`` in the input dtype.  ``ext=(a2, b2)`` appends a second operand pair along the contraction
    (``a2 [M,K2]``; ``b2 [N,K2]``, or ``[K2,N]`` when ``b_mn``; ``K2 % 8 == 0``): both products are accumulated in
    the same pass of the kernel, so a low-rank update costs no second trip over the ``[M,N]`` output.
    """
    if not a.is_cuda:
        A = a.t() if a_mn else a
        Bm = b.t() if b_mn else b
        r = A.float() @ Bm.float().t()
        if ext is not None:
            b2 = ext[1].t() if b_mn else ext[1]
            r = r + ext[0].float() @ b2.float().t()
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
    if ext is not None:
        a2, b2 = ext
        K2 = a2.shape[1]
        assert not a_mn and not accumulate and a2.dtype == torch.bfloat16 and b2.dtype == torch.bfloat16
        assert a2.shape == (M, K2) and b2.shape == ((K2, N) if b_mn else (N, K2)) and K2 % 8 == 0
        assert a2.stride(-1) == 1 and b2.stride(-1) == 1
        rc = nv.lib().b2_gemm_bf16_ext(nv.ptr(a), nv.ptr(b), nv.ptr(out), nv.ptr(residual), M, N, K, a.stride(0),
                                       b.stride(0), out.stride(0), int(b_mn), flags, bn, nv.ptr(a2), nv.ptr(b2), K2,
                                       a2.stride(0), b2.stride(0), nv.stream_ptr())
        nv.check(rc, "gemm_ext")
        nv.count_launch()
        return out
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


class _LoRALinear(torch.autograd.Function):
    """``y = x W^T + (x A^T) Bs^T (+ residual)`` with the low-rank product riding in the base GEMM's accumulator
    (``gemm(..., ext=...)``), forward and input-gradient alike.  ``a_cat [R, K]`` and ``bs [N, R]`` (B already times
    its scaling) are the layer's stacked adapters in the activation dtype; ``w`` is the frozen base weight.

    Two ways to receive the adapter gradients.  ``plan is None``: ``a_cat`` and ``bs`` are differentiable inputs and
    get ``[R, K]`` / ``[N, R]`` gradients.  Otherwise ``a_cat`` / ``bs`` were built without autograd, ``plan`` lists
    ``(rank offset, rank, first row, last row, scaling)`` per adapter and ``params`` are the adapters' own fp32
    ``A_0, B_0, A_1, B_1, ...``: each gets its slice of the stacked gradient, written straight into its
    ``main_grad`` bucket view when the optimizer provides one (no autograd graph through the stacking, and the
    micro-step stays CUDA-graph capturable)."""

    @staticmethod
    def forward(ctx, x, w, a_cat, bs, residual, plan, *params):
        mid = gemm(x, a_cat)                                     # [M, R]
        y = gemm(x, w, residual=residual, ext=(mid, bs))
        ctx.save_for_backward(x, w, a_cat, bs, mid)
        ctx.has_res, ctx.plan, ctx.params = residual is not None, plan, params
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, a_cat, bs, mid = ctx.saved_tensors
        plan, params = ctx.plan, ctx.params
        dy = dy if dy.stride(-1) == 1 else dy.contiguous()
        dmid = gemm(dy, bs, b_mn=True)                           # [M, R] = dy @ Bs
        dx = gemm(dy, w, b_mn=True, ext=(dmid, a_cat)) if ctx.needs_input_grad[0] else None    # dy W + dmid A
        want_ab = plan is not None or ctx.needs_input_grad[2] or ctx.needs_input_grad[3]
        da = gemm(dmid, x, a_mn=True, b_mn=True, out_dtype=torch.float32) if want_ab else None     # [R, K]
        db = gemm(dy, mid, a_mn=True, b_mn=True, out_dtype=torch.float32) if want_ab else None     # [N, R]
        dw = None
        if w.requires_grad:
            dw = grad_into_main(w, lambda out, acc: gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=acc))
        head = (dx, dw, None, None, dy if ctx.has_res else None, None)
        if plan is None:
            return (dx, dw, da.to(a_cat.dtype) if ctx.needs_input_grad[2] else None,
                    db.to(bs.dtype) if ctx.needs_input_grad[3] else None, dy if ctx.has_res else None, None)
        grads = []
        for i, (r0, r, s0, e0, sc) in enumerate(plan):
            pa, pb = params[2 * i], params[2 * i + 1]
            ga, gb = da[r0:r0 + r], db[s0:e0, r0:r0 + r]

            def into_a(out, acc, g=ga):
                if out is None:
                    return g.clone()
                return out.add_(g) if acc else out.copy_(g)

            def into_b(out, acc, g=gb, s_=sc):
                if out is None:
                    return g * s_
                return out.add_(g, alpha=s_) if acc else torch.mul(g, s_, out=out)

            grads.append(grad_into_main(pa, into_a) if pa.requires_grad else None)
            grads.append(grad_into_main(pb, into_b) if pb.requires_grad else None)
        return head + tuple(grads)


def lora_linear(x: torch.Tensor, w: torch.Tensor, a_cat: torch.Tensor, bs: torch.Tensor,
                residual: Optional[torch.Tensor] = None, plan=None, params=()) -> torch.Tensor:
    """LoRA-adapted linear for 2-D ``x``: ``x @ w^T + (x @ a_cat^T) @ bs^T (+ residual)``.  On CUDA the rank-R update
    is accumulated inside the base projection's GEMM (the reference runs three matmuls and an add per adapted layer:
    src/distributed/lora.py:172-177,227-235); R (the stacked rank) must be a multiple of 8 there.  ``plan`` /
    ``params``: see :class:`_LoRALinear`."""
    if not x.is_cuda or a_cat.shape[0] % 8:
        assert plan is None, "the per-adapter gradient plan belongs to the CUDA path"
        y = torch.nn.functional.linear(x, w.to(x.dtype))
        y = y + torch.nn.functional.linear(torch.nn.functional.linear(x, a_cat.to(x.dtype)), bs.to(x.dtype))
        return y if residual is None else y + residual
    if no_grad_needed(x, w, a_cat, bs, residual, *params):
        return gemm(x, w, residual=residual, ext=(gemm(x, a_cat), bs))
    return _LoRALinear.apply(x, w, a_cat, bs, residual, plan, *params)
