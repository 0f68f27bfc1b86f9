"""RMSNorm, fused QK-RMSNorm + RoPE, SwiGLU and embedding.

Reference call sites: RMSNorm (src/distributed/tensor_parallel.py:78-84), q_norm/k_norm and
``_apply_rotary_emb`` (:373-374,397-421,451-462), SwiGLU (:295-299), ``nn.Embedding`` (:818,885).
"""
from __future__ import annotations

from typing import Tuple

import torch

from .. import _native as nv
from .gemm import NO_GRAD_CTX, grad_into_main, no_grad_needed

_rope_cache = {}


def rope_tables(max_pos: int, head_dim: int, theta: float, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``cos``/``sin`` tables ``[max_pos, head_dim/2]`` (half-rotation convention)."""
    key = (max_pos, head_dim, float(theta), str(device))
    if key not in _rope_cache:
        inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
        ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
        _rope_cache[key] = (ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous())
    return _rope_cache[key]


# ---- RMSNorm ------------------------------------------------------------------------------------
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        M, H = x.shape
        y = torch.empty_like(x)
        rstd = torch.empty(M, device=x.device, dtype=torch.float32)
        nv.check(nv.lib().b2_rmsnorm_fwd(nv.ptr(x), nv.ptr(w), nv.ptr(y), nv.ptr(rstd), M, H,
                                         nv.ctypes.c_float(eps), nv.stream_ptr()), "rmsnorm_fwd")
        nv.count_launch()
        ctx.save_for_backward(x, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        M, H = x.shape
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        L = nv.lib()
        partial = torch.empty(L.b2_rmsnorm_bwd_ctas() * H, device=x.device, dtype=torch.float32)

        def run(out, acc):
            tgt = out if out is not None else torch.empty_like(w)
            nv.check(L.b2_rmsnorm_bwd(nv.ptr(dy), nv.ptr(x), nv.ptr(w), nv.ptr(rstd), nv.ptr(dx),
                                      nv.ptr(tgt), nv.ptr(partial), M, H, 0, int(acc),
                                      int(tgt.dtype == torch.float32), nv.stream_ptr()), "rmsnorm_bwd")
            nv.count_launch(3)
            return tgt

        dw = grad_into_main(w, run)
        return dx, dw, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Row-wise RMSNorm over the last dim of a 2-D tensor, fp32 internally."""
    if not x.is_cuda:
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)
    if no_grad_needed(x, w):
        return _RMSNorm.forward(NO_GRAD_CTX, x.contiguous(), w, eps)
    return _RMSNorm.apply(x.contiguous(), w, eps)


# ---- QK-norm + RoPE -------------------------------------------------------------------------------
class _QKNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, qw, kw, pos, cos, sin, Hq, Hkv, eps):
        M = qkv.shape[0]
        q = torch.empty((M, Hq * 128), device=qkv.device, dtype=qkv.dtype)
        k = torch.empty((M, Hkv * 128), device=qkv.device, dtype=qkv.dtype)
        rstd = torch.empty((M, Hq + Hkv), device=qkv.device, dtype=torch.float32)
        nv.check(nv.lib().b2_qknorm_rope_fwd(nv.ptr(qkv), nv.ptr(qw), nv.ptr(kw), nv.ptr(pos), nv.ptr(cos),
                                             nv.ptr(sin), nv.ptr(q), nv.ptr(k), nv.ptr(rstd), M, Hq, Hkv, 128,
                                             qkv.stride(0), nv.ctypes.c_float(eps), nv.stream_ptr()),
                 "qknorm_rope_fwd")
        nv.count_launch()
        ctx.save_for_backward(qkv, qw, kw, pos, cos, sin, rstd)
        ctx.dims = (Hq, Hkv)
        v = qkv[:, (Hq + Hkv) * 128:]
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        qkv, qw, kw, pos, cos, sin, rstd = ctx.saved_tensors
        Hq, Hkv = ctx.dims
        M = qkv.shape[0]
        buf = torch.empty_like(qkv)
        buf[:, (Hq + Hkv) * 128:].copy_(dv)
        dwq = torch.zeros(128, device=qkv.device, dtype=torch.float32)
        dwk = torch.zeros(128, device=qkv.device, dtype=torch.float32)
        nv.check(nv.lib().b2_qknorm_rope_bwd(nv.ptr(dq.contiguous()), nv.ptr(dk.contiguous()), nv.ptr(qkv),
                                             nv.ptr(qw), nv.ptr(kw), nv.ptr(pos), nv.ptr(cos), nv.ptr(sin),
                                             nv.ptr(rstd), nv.ptr(buf), nv.ptr(dwq), nv.ptr(dwk), M, Hq, Hkv,
                                             128, qkv.stride(0), nv.stream_ptr()), "qknorm_rope_bwd")
        nv.count_launch()

        def into(param, g):
            def run(out, acc):
                if out is None:
                    return g.to(param.dtype)
                if acc:
                    out.add_(g.to(out.dtype))
                else:
                    out.copy_(g)
                return out
            return grad_into_main(param, run)

        return buf, into(qw, dwq), into(kw, dwk), None, None, None, None, None, None


def _rope_ref(x, pos, cos, sin):
    # x [M, H, D]; half-rotation
    c = cos[pos][:, None, :].float()
    s = sin[pos][:, None, :].float()
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def qknorm_rope(qkv: torch.Tensor, qw: torch.Tensor, kw: torch.Tensor, pos: torch.Tensor,
                cos: torch.Tensor, sin: torch.Tensor, Hq: int, Hkv: int, head_dim: int,
                eps: float = 1e-6):
    """Split the fused projection ``[M,(Hq+2Hkv)*D]``; per-head RMSNorm + RoPE on q and k.

    Returns ``q [M,Hq*D]``, ``k [M,Hkv*D]`` and ``v`` (a strided view of ``qkv``).
    """
    if not qkv.is_cuda:
        M = qkv.shape[0]
        D = head_dim
        q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)

        def hn(x, w, H):
            xf = x.reshape(M, H, D).float()
            return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()

        qn = _rope_ref(hn(q, qw, Hq), pos.long(), cos, sin).reshape(M, Hq * D).to(qkv.dtype)
        kn = _rope_ref(hn(k, kw, Hkv), pos.long(), cos, sin).reshape(M, Hkv * D).to(qkv.dtype)
        return qn, kn, v
    assert head_dim == 128, "CUDA qknorm_rope kernel is specialised for head_dim 128"
    if no_grad_needed(qkv, qw, kw):
        return _QKNormRope.forward(NO_GRAD_CTX, qkv, qw, kw, pos if pos.dtype == torch.int32 else pos.to(torch.int32),
                                   cos, sin, Hq, Hkv, eps)
    return _QKNormRope.apply(qkv, qw, kw, pos.to(torch.int32), cos, sin, Hq, Hkv, eps)


def qknorm_rope_store(qkv: torch.Tensor, qw: torch.Tensor, kw: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor,
                      sin: torch.Tensor, Hq: int, Hkv: int, head_dim: int, eps: float, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, slots: torch.Tensor):
    """Inference form of :func:`qknorm_rope`: the same split / norm / rotation, and the new keys and values are
    written into the 16-bit paged cache ``[blocks, block_size, Hkv, D]`` at row ``slots[t]`` (``block * block_size +
    offset``; negative = padding row, nothing stored) by the same kernel.  One launch replaces the reference's
    rotary call plus its ``store_kvcache`` kernel (src/inference/attention.py:32-110).  No gradient."""
    if not qkv.is_cuda:
        q, k, v = qknorm_rope(qkv, qw, kw, pos, cos, sin, Hq, Hkv, head_dim, eps)
        keep = (slots >= 0).nonzero().flatten()
        rows = slots.long().index_select(0, keep)
        k_cache.view(-1, Hkv, head_dim).index_copy_(0, rows, k.reshape(-1, Hkv, head_dim).index_select(0, keep).to(k_cache.dtype))
        v_cache.view(-1, Hkv, head_dim).index_copy_(0, rows, v.reshape(-1, Hkv, head_dim).index_select(0, keep).to(v_cache.dtype))
        return q, k, v
    assert head_dim == 128 and k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
    M = qkv.shape[0]
    # the kernel indexes pos / slots by token and the caches by slot: sizes the host knows are checked here
    assert slots.dtype == torch.int32 and slots.is_cuda and slots.numel() == M and pos.numel() == M
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape == v_cache.shape
    assert k_cache.shape[-2:] == (Hkv, 128) and qkv.shape[1] == (Hq + 2 * Hkv) * 128 and qkv.stride(1) == 1
    q = torch.empty((M, Hq * 128), device=qkv.device, dtype=qkv.dtype)
    k = torch.empty((M, Hkv * 128), device=qkv.device, dtype=qkv.dtype)
    pos = pos if pos.dtype == torch.int32 else pos.to(torch.int32)
    nv.check(nv.lib().b2_qknorm_rope_store(nv.ptr(qkv), nv.ptr(qw), nv.ptr(kw), nv.ptr(pos), nv.ptr(cos), nv.ptr(sin),
                                           nv.ptr(q), nv.ptr(k), M, Hq, Hkv, 128, qkv.stride(0),
                                           nv.ctypes.c_float(eps), nv.ptr(slots), nv.ptr(k_cache), nv.ptr(v_cache),
                                           nv.stream_ptr()), "qknorm_rope_store")
    nv.count_launch()
    return q, k, qkv[:, (Hq + Hkv) * 128:]


# ---- SwiGLU ---------------------------------------------------------------------------------------
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        M, I2 = gu.shape
        out = torch.empty((M, I2 // 2), device=gu.device, dtype=gu.dtype)
        nv.check(nv.lib().b2_swiglu_fwd(nv.ptr(gu), nv.ptr(out), nv.ctypes.c_longlong(M), I2 // 2,
                                        nv.stream_ptr()), "swiglu_fwd")
        nv.count_launch()
        ctx.save_for_backward(gu)
        return out

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        M, I2 = gu.shape
        dgu = torch.empty_like(gu)
        nv.check(nv.lib().b2_swiglu_bwd(nv.ptr(dout.contiguous()), nv.ptr(gu), nv.ptr(dgu),
                                        nv.ctypes.c_longlong(M), I2 // 2, nv.stream_ptr()), "swiglu_bwd")
        nv.count_launch()
        return dgu


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` on the fused ``[M, 2I]`` projection (gate columns first)."""
    if not gu.is_cuda:
        g, u = gu.chunk(2, dim=-1)
        return (torch.nn.functional.silu(g.float()) * u.float()).to(gu.dtype)
    if no_grad_needed(gu):
        return _SwiGLU.forward(NO_GRAD_CTX, gu.contiguous())
    return _SwiGLU.apply(gu.contiguous())


# ---- embedding ------------------------------------------------------------------------------------
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        M, H = ids.numel(), table.shape[1]
        out = torch.empty((M, H), device=table.device, dtype=table.dtype)
        nv.check(nv.lib().b2_embedding_fwd(nv.ptr(ids), nv.ptr(table), nv.ptr(out), M, H, nv.stream_ptr()),
                 "embedding_fwd")
        nv.count_launch()
        ctx.save_for_backward(ids)
        ctx.table = table
        return out

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        table = ctx.table
        M, H = ids.numel(), table.shape[1]
        dout = dout.contiguous()

        def run(out, acc):
            tgt = out
            if tgt is None:
                tgt = torch.zeros_like(table)
            elif not acc:
                tgt.zero_()
            if tgt.dtype == torch.bfloat16:
                nv.check(nv.lib().b2_embedding_bwd(nv.ptr(ids), nv.ptr(dout), nv.ptr(tgt), M, H,
                                                   nv.stream_ptr()), "embedding_bwd")
                nv.count_launch()
            else:
                tgt.index_add_(0, ids, dout.to(tgt.dtype))
            return tgt

        return None, grad_into_main(table, run)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Row gather ``[M] -> [M,H]``; backward is a bf16 atomic scatter-add."""
    ids = ids.reshape(-1)
    if not table.is_cuda:
        return torch.nn.functional.embedding(ids, table)
    if no_grad_needed(table):
        return _Embedding.forward(NO_GRAD_CTX, ids.long().contiguous(), table)
    return _Embedding.apply(ids.long().contiguous(), table)
