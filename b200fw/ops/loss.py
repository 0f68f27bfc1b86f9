"""Fused LM-head losses: the ``[tokens, vocab]`` logits exist only one row-chunk at a time.

* :func:`lm_head_cross_entropy` — masked-mean CE; forward computes the loss *and* the gradients
  (Liger-style): for each chunk, logits = h W^T (tcgen05 GEMM), one row kernel turns them in place
  into ``(softmax - onehot) * scale``, and two more GEMMs produce dh and accumulate dW.  Replaces
  ``lm_head`` + ``F.cross_entropy`` (src/engines/train_engine.py:1376-1385).
* :func:`lm_head_logprob` — per-token log-probability of the label (GRPO / IcePop / rollout scoring);
  backward recomputes the chunk's logits.  Replaces ``log_softmax`` + ``gather`` over ``[B*K,S,V]``
  (src/engines/train_engine.py:1132-1139).
* :func:`grpo_token_loss` — clipped surrogate + KL on token log-probs
  (src/engines/train_engine.py:1387-1449) as one stats kernel and one gradient kernel.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import _native as nv
from .gemm import gemm, grad_into_main

IGNORE = -100
DEFAULT_CHUNK = 4096


def _rows(logits, labels, mode, scale=None, loss_sum=None, lse=None, logp=None, g=None, inv_t=1.0):
    rows, V = logits.shape
    nv.check(nv.lib().b2_vocab_rows(nv.ptr(logits), nv.ptr(labels), rows, V, logits.stride(0), mode,
                                    nv.ptr(scale), nv.ptr(loss_sum), nv.ptr(lse), nv.ptr(logp), nv.ptr(g),
                                    nv.ctypes.c_longlong(IGNORE), nv.ctypes.c_float(inv_t), nv.stream_ptr()),
             "vocab_rows")
    nv.count_launch()


class _LMHeadCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, labels, loss_scale, chunk, n_valid):
        M, H = h.shape
        V = w.shape[0]
        need_grad = h.requires_grad or w.requires_grad
        n_valid_f = n_valid.to(torch.float32).clamp_(min=1.0)
        scale = (loss_scale / n_valid_f).reshape(1).contiguous()
        loss_sum = torch.zeros(1, device=h.device, dtype=torch.float32)
        dh = torch.empty_like(h) if need_grad else None
        first = True
        for s in range(0, M, chunk):
            e = min(M, s + chunk)
            logits = gemm(h[s:e], w)
            _rows(logits, labels[s:e], 0, scale=scale, loss_sum=loss_sum)
            if not need_grad:
                continue  # logits hold gradients nobody wants; only loss_sum matters
            gemm(logits, w, b_mn=True, out=dh[s:e])
            if w.requires_grad:
                hs = h[s:e]
                if first:
                    ctx.dw = grad_into_main(w, lambda out, acc: gemm(logits, hs, a_mn=True, b_mn=True,
                                                                      out=out, accumulate=acc))
                    first = False
                else:
                    tgt = getattr(w, "main_grad", None)
                    gemm(logits, hs, a_mn=True, b_mn=True, out=tgt if tgt is not None else ctx.dw,
                         accumulate=True)
            del logits
        ctx.dh = dh
        ctx.w_needs = w.requires_grad
        if not hasattr(ctx, "dw"):
            ctx.dw = None
        return (loss_sum / n_valid_f).squeeze(0)

    @staticmethod
    def backward(ctx, gout):
        # gradients were computed with loss_scale already applied; gout scales them further (it is
        # 1.0 when the caller passes the accumulation factor through loss_scale).
        dh = ctx.dh
        dw = ctx.dw
        if dh is not None:
            dh = dh * gout.to(dh.dtype)
        if dw is not None:
            dw = dw * gout.to(dw.dtype)
        return dh, dw, None, None, None, None


def lm_head_cross_entropy(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, loss_scale: float = 1.0,
                          chunk: int = DEFAULT_CHUNK, n_valid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Mean CE of ``h @ w^T`` against ``labels`` (``-100`` ignored) without materialising the logits.

    The returned loss is the unscaled mean; the gradients carry ``loss_scale`` (use it for
    ``1/grad_accum`` and call ``backward()`` on the returned value directly — scaling the loss again
    would scale the gradients twice).  ``n_valid`` overrides the normaliser (e.g. a global count).
    """
    labels = labels.reshape(-1)
    if n_valid is None:
        n_valid = (labels != IGNORE).sum()
    if not h.is_cuda:
        logits = torch.nn.functional.linear(h, w.to(h.dtype)).float()
        tot = torch.nn.functional.cross_entropy(logits, labels, ignore_index=IGNORE, reduction="sum")
        loss = tot / n_valid.clamp(min=1).float()
        return _ScaleGrad.apply(loss, loss_scale)
    return _LMHeadCE.apply(h.contiguous(), w, labels.long().contiguous(), float(loss_scale), int(chunk), n_valid)


class _ScaleGrad(torch.autograd.Function):
    """Identity in forward, multiplies the gradient by ``s`` (keeps CPU and CUDA semantics equal)."""

    @staticmethod
    def forward(ctx, x, s):
        ctx.s = s
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g * ctx.s, None


class _LMHeadLogprob(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, labels, inv_t, chunk):
        M = h.shape[0]
        lse = torch.empty(M, device=h.device, dtype=torch.float32)
        logp = torch.empty(M, device=h.device, dtype=torch.float32)
        for s in range(0, M, chunk):
            e = min(M, s + chunk)
            logits = gemm(h[s:e], w)
            _rows(logits, labels[s:e], 1, lse=lse[s:e], logp=logp[s:e], inv_t=inv_t)
            del logits
        ctx.save_for_backward(h, w, labels, lse)
        ctx.args = (inv_t, chunk)
        return logp

    @staticmethod
    def backward(ctx, g):
        h, w, labels, lse = ctx.saved_tensors
        inv_t, chunk = ctx.args
        M = h.shape[0]
        g = g.contiguous().float()
        dh = torch.empty_like(h)
        dw_holder = {"dw": None, "first": True}
        for s in range(0, M, chunk):
            e = min(M, s + chunk)
            logits = gemm(h[s:e], w)
            _rows(logits, labels[s:e], 2, lse=lse[s:e], g=g[s:e], inv_t=inv_t)
            gemm(logits, w, b_mn=True, out=dh[s:e])
            if w.requires_grad:
                hs = h[s:e]
                if dw_holder["first"]:
                    dw_holder["dw"] = grad_into_main(
                        w, lambda out, acc: gemm(logits, hs, a_mn=True, b_mn=True, out=out, accumulate=acc))
                    dw_holder["first"] = False
                else:
                    tgt = getattr(w, "main_grad", None)
                    gemm(logits, hs, a_mn=True, b_mn=True, out=tgt if tgt is not None else dw_holder["dw"],
                         accumulate=True)
            del logits
        return dh, dw_holder["dw"], None, None, None


def lm_head_logprob(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0,
                    chunk: int = DEFAULT_CHUNK) -> torch.Tensor:
    """``log softmax(h @ w^T / temperature)[label]`` per row as fp32 ``[M]`` (0 where label is -100)."""
    labels = labels.reshape(-1)
    if not h.is_cuda:
        logits = torch.nn.functional.linear(h, w.to(h.dtype)).float() / temperature
        lp = torch.log_softmax(logits, dim=-1)
        safe = labels.clamp(min=0)
        out = lp.gather(-1, safe[:, None]).squeeze(-1)
        return torch.where(labels == IGNORE, torch.zeros_like(out), out)
    return _LMHeadLogprob.apply(h.contiguous(), w, labels.long().contiguous(), 1.0 / temperature, int(chunk))


def _grpo_ref(lp, old_lp, ref_lp, mask, adv, clip_eps, beta):
    ratio = torch.exp(lp - old_lp)
    a = adv[:, None]
    surr1 = ratio * a
    surr2 = ratio.clamp(1 - clip_eps, 1 + clip_eps) * a
    denom = mask.sum() + 1e-8
    policy = (-torch.min(surr1, surr2) * mask).sum() / denom
    kl = torch.zeros((), device=lp.device)
    if ref_lp is not None and beta > 0:
        kl = (((lp - ref_lp) * mask).sum() / denom).clamp(min=0.0)
    with torch.no_grad():
        mb = mask.bool()
        info = {
            "policy_loss": policy.detach(), "kl_divergence": kl.detach(),
            "ratio_mean": (ratio * mask).sum() / denom,
            "ratio_max": ratio[mb].max() if mb.any() else torch.ones(()),
            "ratio_min": ratio[mb].min() if mb.any() else torch.ones(()),
            "clipped_fraction": ((ratio - 1).abs() > clip_eps).float()[mb].mean() if mb.any() else torch.zeros(()),
            "valid_token_count": mask.sum(),
        }
    return policy + beta * kl, info


class _GRPOLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, lp, old_lp, ref_lp, mask, adv, clip_eps, beta, loss_scale):
        rows, cols = lp.shape
        stats = torch.zeros(8, device=lp.device, dtype=torch.float32)
        stats[6] = float("inf")
        g = torch.empty_like(lp)
        nv.check(nv.lib().b2_grpo_loss(nv.ptr(lp), nv.ptr(old_lp), nv.ptr(ref_lp), nv.ptr(mask), nv.ptr(adv),
                                       rows, cols, nv.ctypes.c_float(clip_eps), nv.ctypes.c_float(beta),
                                       nv.ctypes.c_float(loss_scale), nv.ptr(stats), nv.ptr(g),
                                       nv.stream_ptr()), "grpo_loss")
        nv.count_launch(2)
        ctx.save_for_backward(g)
        denom = stats[1] + 1e-8
        policy = stats[0] / denom
        kl = (stats[2] / denom).clamp(min=0.0) if (ref_lp is not None and beta > 0) else torch.zeros_like(policy)
        ctx.mark_non_differentiable(stats)
        return policy + beta * kl, stats

    @staticmethod
    def backward(ctx, gout, _gstats):
        (g,) = ctx.saved_tensors
        return g * gout, None, None, None, None, None, None, None


def grpo_token_loss(lp: torch.Tensor, old_lp: torch.Tensor, ref_lp: Optional[torch.Tensor], mask: torch.Tensor,
                    adv: torch.Tensor, clip_eps: float = 0.2, beta: float = 0.0,
                    loss_scale: float = 1.0) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    """GRPO loss on ``[rows, cols]`` token log-probs.  Returns ``(loss, info)``; ``info`` values are
    0-d tensors (no host sync here).  Gradients carry ``loss_scale``."""
    if not lp.is_cuda:
        loss, info = _grpo_ref(lp, old_lp, ref_lp, mask, adv, clip_eps, beta)
        return _ScaleGrad.apply(loss, loss_scale), info
    f = lambda t: None if t is None else t.contiguous().float()
    loss, stats = _GRPOLoss.apply(lp.contiguous(), f(old_lp), f(ref_lp), f(mask), f(adv), float(clip_eps),
                                  float(beta), float(loss_scale))
    denom = stats[1] + 1e-8
    info = {
        "policy_loss": stats[0] / denom,
        "kl_divergence": (stats[2] / denom).clamp(min=0.0) if (ref_lp is not None and beta > 0) else stats[2] * 0,
        "ratio_mean": stats[3] / denom, "ratio_max": stats[5], "ratio_min": stats[6],
        "clipped_fraction": stats[4] / denom.clamp(min=1.0), "valid_token_count": stats[1],
    }
    return loss, info
