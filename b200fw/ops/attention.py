"""Causal flash attention (training / prefill over contiguous K,V) on the tcgen05 kernels.

Replaces the reference's three-way backend switch — ``flash_attn_func``, SDPA, manual softmax
(src/distributed/tensor_parallel.py:464-535) — with one native path.  ``fused_qkv_attention`` also
folds the per-head QK-RMSNorm + RoPE in front, so that the backward pass writes dQ/dK/dV straight
into one fused gradient buffer for the QKV projection.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _native as nv
from .elementwise import qknorm_rope
from .gemm import grad_into_main


def _attn_ref(q, k, v, B, S, Hq, Hkv, scale):
    D = q.shape[-1] // Hq
    qf = q.reshape(B, S, Hq, D).transpose(1, 2).float()
    kf = k.reshape(B, S, Hkv, D).transpose(1, 2).float()
    vf = v.reshape(B, S, Hkv, D).transpose(1, 2).float()
    g = Hq // Hkv
    kf = kf.repeat_interleave(g, dim=1)
    vf = vf.repeat_interleave(g, dim=1)
    att = (qf @ kf.transpose(-1, -2)) * scale
    mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
    att = att.masked_fill(~mask, float("-inf")).softmax(-1)
    return (att @ vf).transpose(1, 2).reshape(B * S, Hq * D).to(q.dtype)


def _fwd(q, k, v, B, S, Hq, Hkv, scale):
    T = B * S
    out = torch.empty((T, Hq * 128), device=q.device, dtype=q.dtype)
    lse = torch.empty((Hq, T), device=q.device, dtype=torch.float32)
    nv.check(nv.lib().b2_attn_fwd(nv.ptr(q), nv.ptr(k), nv.ptr(v), nv.ptr(out), nv.ptr(lse), B, S, Hq, Hkv,
                                  128, v.stride(0), nv.ctypes.c_float(scale), nv.stream_ptr()), "attn_fwd")
    nv.count_launch()
    return out, lse


def _bwd(q, k, v, out, dout, lse, dq, dk, dv, B, S, Hq, Hkv, scale):
    T = B * S
    dsum = torch.empty((Hq, T), device=q.device, dtype=torch.float32)
    nv.check(nv.lib().b2_attn_bwd(nv.ptr(q), nv.ptr(k), nv.ptr(v), nv.ptr(out), nv.ptr(dout), nv.ptr(lse),
                                  nv.ptr(dsum), nv.ptr(dq), nv.ptr(dk), nv.ptr(dv), B, S, Hq, Hkv, 128,
                                  v.stride(0), dk.stride(0), dv.stride(0), nv.ctypes.c_float(scale),
                                  nv.stream_ptr()), "attn_bwd")
    nv.count_launch(3)


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, B, S, Hq, Hkv, scale):
        q, k = q.contiguous(), k.contiguous()
        out, lse = _fwd(q, k, v, B, S, Hq, Hkv, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.dims = (B, S, Hq, Hkv, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        B, S, Hq, Hkv, scale = ctx.dims
        dq = torch.empty_like(q)
        dk = torch.empty_like(k)
        dv = torch.empty((B * S, Hkv * 128), device=q.device, dtype=q.dtype)
        _bwd(q, k, v, out, dout.contiguous(), lse, dq, dk, dv, B, S, Hq, Hkv, scale)
        return dq, dk, dv, None, None, None, None, None


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, B: int, S: int, Hq: int, Hkv: int,
                    scale: Optional[float] = None) -> torch.Tensor:
    """Causal GQA attention over ``B`` sequences of ``S`` tokens.

    ``q [B*S, Hq*D]``, ``k [B*S, Hkv*D]`` contiguous; ``v [B*S, Hkv*D]`` may be a column slice of a
    wider buffer (row stride is passed to the kernel).  Returns ``[B*S, Hq*D]``.
    """
    D = q.shape[-1] // Hq
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        return _attn_ref(q, k, v, B, S, Hq, Hkv, scale)
    assert D == 128, "CUDA attention kernels are specialised for head_dim 128"
    return _FlashAttn.apply(q, k, v, B, S, Hq, Hkv, scale)


class _FusedQKVAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, qw, kw, pos, cos, sin, B, S, Hq, Hkv, eps, scale):
        M = qkv.shape[0]
        L = nv.lib()
        q = torch.empty((M, Hq * 128), device=qkv.device, dtype=qkv.dtype)
        k = torch.empty((M, Hkv * 128), device=qkv.device, dtype=qkv.dtype)
        rstd = torch.empty((M, Hq + Hkv), device=qkv.device, dtype=torch.float32)
        nv.check(L.b2_qknorm_rope_fwd(nv.ptr(qkv), nv.ptr(qw), nv.ptr(kw), nv.ptr(pos), nv.ptr(cos), nv.ptr(sin),
                                      nv.ptr(q), nv.ptr(k), nv.ptr(rstd), M, Hq, Hkv, 128, qkv.stride(0),
                                      nv.ctypes.c_float(eps), nv.stream_ptr()), "qknorm_rope_fwd")
        nv.count_launch()
        v = qkv[:, (Hq + Hkv) * 128:]
        out, lse = _fwd(q, k, v, B, S, Hq, Hkv, scale)
        ctx.save_for_backward(qkv, qw, kw, pos, cos, sin, q, k, rstd, out, lse)
        ctx.dims = (B, S, Hq, Hkv, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, qw, kw, pos, cos, sin, q, k, rstd, out, lse = ctx.saved_tensors
        B, S, Hq, Hkv, scale = ctx.dims
        M = qkv.shape[0]
        L = nv.lib()
        v = qkv[:, (Hq + Hkv) * 128:]
        dqkv = torch.empty_like(qkv)
        dq = torch.empty_like(q)
        dk = torch.empty_like(k)
        dv = dqkv[:, (Hq + Hkv) * 128:]
        _bwd(q, k, v, out, dout.contiguous(), lse, dq, dk, dv, B, S, Hq, Hkv, scale)
        dwq = torch.zeros(128, device=qkv.device, dtype=torch.float32)
        dwk = torch.zeros(128, device=qkv.device, dtype=torch.float32)
        nv.check(L.b2_qknorm_rope_bwd(nv.ptr(dq), nv.ptr(dk), nv.ptr(qkv), nv.ptr(qw), nv.ptr(kw), nv.ptr(pos),
                                      nv.ptr(cos), nv.ptr(sin), nv.ptr(rstd), nv.ptr(dqkv), nv.ptr(dwq),
                                      nv.ptr(dwk), M, Hq, Hkv, 128, qkv.stride(0), nv.stream_ptr()),
                 "qknorm_rope_bwd")
        nv.count_launch()

        def into(param, g):
            def run(o, acc):
                if o is None:
                    return g.to(param.dtype)
                if acc:
                    o.add_(g.to(o.dtype))
                else:
                    o.copy_(g)
                return o
            return grad_into_main(param, run)

        return dqkv, into(qw, dwq), into(kw, dwk), None, None, None, None, None, None, None, None, None


def fused_qkv_attention(qkv, qw, kw, pos, cos, sin, B, S, Hq, Hkv, head_dim, eps=1e-6, scale=None):
    """QK-RMSNorm + RoPE + causal attention on the fused QKV projection ``[B*S, (Hq+2Hkv)*D]``."""
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    if not qkv.is_cuda:
        q, k, v = qknorm_rope(qkv, qw, kw, pos, cos, sin, Hq, Hkv, head_dim, eps)
        return _attn_ref(q, k, v, B, S, Hq, Hkv, scale)
    assert head_dim == 128
    return _FusedQKVAttn.apply(qkv, qw, kw, pos.to(torch.int32), cos, sin, B, S, Hq, Hkv, eps, scale)
