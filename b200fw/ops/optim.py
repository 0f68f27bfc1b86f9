"""Flat-buffer optimizer kernels: sum of squares (doubles as the NaN/Inf scan) and fused AdamW.

They replace the per-parameter ``norm(2).item()`` loop and ``torch.optim.AdamW`` on the ZeRO shard
(src/engines/train_engine.py:1466-1485, src/distributed/zero_optim.py:203-209).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as nv


def sumsq(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[0] += sum(x*x)`` in fp32.  NaN / Inf inputs propagate into the result."""
    if out is None:
        out = torch.zeros(1, device=x.device, dtype=torch.float32)
    if not x.is_cuda:
        out += x.float().pow(2).sum()
        return out
    x = x.reshape(-1)
    assert x.is_contiguous() and x.dtype in (torch.float32, torch.bfloat16)
    nv.check(nv.lib().b2_sumsq(nv.ptr(x), nv.ctypes.c_longlong(x.numel()), int(x.dtype == torch.float32),
                               nv.ptr(out), nv.stream_ptr()), "sumsq")
    nv.count_launch()
    return out


def fused_adamw(master: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, grad: torch.Tensor,
                hyper: torch.Tensor, *, param_out: Optional[torch.Tensor] = None,
                norm_sq: Optional[torch.Tensor] = None, grad_scale: float = 1.0) -> None:
    """One AdamW step on a flat fp32 master buffer.

    ``hyper`` is a device fp32 tensor ``[lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2,
    max_norm]``.  When ``norm_sq`` (device fp32[1], the global squared gradient norm *after*
    ``grad_scale``) is given the step clips to ``max_norm`` and is skipped entirely if the norm is not
    finite.  ``param_out`` receives the updated parameters as bf16.
    """
    n = master.numel()
    if not master.is_cuda:
        lr, b1, b2, eps, wd, bc1, bc2, max_norm = [float(v) for v in hyper.tolist()]
        g = grad.float() * grad_scale
        if norm_sq is not None:
            ns = float(norm_sq)
            if ns != ns or ns in (float("inf"), float("-inf")):
                return
            if max_norm > 0:
                g = g * min(1.0, max_norm / (ns ** 0.5 + 1e-6))
        exp_avg.mul_(b1).add_(g, alpha=1 - b1)
        exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
        master.mul_(1 - lr * wd).addcdiv_(exp_avg / bc1, (exp_avg_sq / bc2).sqrt() + eps, value=-lr)
        if param_out is not None:
            param_out.copy_(master.to(param_out.dtype))
        return
    assert master.dtype == torch.float32 and grad.numel() == n
    assert param_out is None or param_out.dtype == torch.bfloat16
    nv.check(nv.lib().b2_adamw(nv.ptr(master), nv.ptr(exp_avg), nv.ptr(exp_avg_sq), nv.ptr(grad),
                               int(grad.dtype == torch.float32), nv.ptr(param_out), nv.ctypes.c_longlong(n),
                               nv.ptr(hyper), nv.ptr(norm_sq), nv.ctypes.c_float(grad_scale), nv.stream_ptr()),
             "adamw")
    nv.count_launch()
