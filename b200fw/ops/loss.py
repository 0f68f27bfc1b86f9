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


def _rows(logits, labels, mode, scale=None, loss_sum=None, lse=None, logp=None, g=None, inv_t=1.0,
          vocab_start=0, vocab_total=0, stats=None):
    rows, V = logits.shape
    nv.check(nv.lib().b2_vocab_rows(nv.ptr(logits), nv.ptr(labels), rows, V, logits.stride(0), mode,
                                    nv.ptr(scale), nv.ptr(loss_sum), nv.ptr(lse), nv.ptr(logp), nv.ptr(g),
                                    nv.ctypes.c_longlong(IGNORE), nv.ctypes.c_float(inv_t),
                                    nv.ctypes.c_longlong(vocab_start), nv.ctypes.c_longlong(vocab_total),
                                    nv.ptr(stats), nv.stream_ptr()),
             "vocab_rows")
    nv.count_launch()


_side_stream = {}


def valid_rows(labels: torch.Tensor) -> Optional[torch.Tensor]:
    """Indices of the rows whose label is not ``-100``, or ``None`` when every row counts.

    Rows with an ignored label contribute neither loss nor gradient, so the LM-head GEMMs only need the
    others (in SFT the prompt half of every sequence is masked).  Their number has to reach the host to
    size the GEMMs; the count runs on a side stream that only waits for the labels, so the host does not
    drain the forward pass it has already queued on the main stream."""
    if not labels.is_cuda:
        idx = torch.nonzero(labels != IGNORE).squeeze(-1)
        return None if idx.numel() == labels.numel() else idx
    dev = labels.device
    side = _side_stream.get(dev.index)
    if side is None:
        side = _side_stream[dev.index] = torch.cuda.Stream(device=dev)
    ready = torch.cuda.current_stream(dev).record_event()
    with torch.cuda.stream(side):
        side.wait_event(ready)
        idx = torch.nonzero(labels != IGNORE).squeeze(-1)      # synchronises the side stream only
    labels.record_stream(side)
    idx.record_stream(torch.cuda.current_stream(dev))
    torch.cuda.current_stream(dev).wait_stream(side)
    return None if idx.numel() == labels.numel() else idx


class VocabShard:
    """Which slice of the vocabulary a tensor-parallel rank's LM-head rows cover, and the group to
    combine the per-row softmax statistics over.  ``reduce_dh``: sum the hidden-state gradient over
    the group inside the loss (set it to False when the producer of ``h`` reduce-scatters the
    gradient itself, as the sequence-parallel gather does)."""

    def __init__(self, group, rank: int, world: int, vocab_total: int, reduce_dh: bool = True):
        self.group, self.rank, self.world, self.total = group, rank, world, vocab_total
        if vocab_total % world:
            raise ValueError(f"vocab {vocab_total} is not divisible by the tensor-parallel size {world}")
        self.local = vocab_total // world
        self.start = rank * self.local
        self.reduce_dh = reduce_dh


def _combine_shard_stats(stats: torch.Tensor, shard: VocabShard):
    """``[rows,3]`` local (max, sumexp, label logit) -> global (lse, label_logit), one all-gather."""
    import torch.distributed as dist
    allst = torch.empty((shard.world,) + tuple(stats.shape), device=stats.device, dtype=stats.dtype)
    dist.all_gather_into_tensor(allst, stats, group=shard.group)
    m = allst[..., 0]
    gm = m.max(dim=0).values
    ssum = (allst[..., 1] * torch.exp(m - gm)).sum(dim=0)
    return gm + torch.log(ssum), allst[..., 2].sum(dim=0)


def _dw_step(ctx_holder, w, logits, hs):
    """dW (+)= logits^T hs, written into ``w.main_grad`` when the optimizer provides one."""
    if ctx_holder["first"]:
        ctx_holder["dw"] = grad_into_main(w, lambda out, acc: gemm(logits, hs, a_mn=True, b_mn=True,
                                                                     out=out, accumulate=acc))
        ctx_holder["first"] = False
    else:
        tgt = getattr(w, "main_grad", None)
        gemm(logits, hs, a_mn=True, b_mn=True, out=tgt if tgt is not None else ctx_holder["dw"],
             accumulate=True)


class _LMHeadCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, labels, loss_scale, chunk, n_valid, shard):
        M, H = h.shape
        need_grad = h.requires_grad or w.requires_grad
        n_valid_f = n_valid.to(torch.float32).clamp_(min=1.0)
        scale = (loss_scale / n_valid_f).reshape(1).contiguous()
        loss_sum = torch.zeros(1, device=h.device, dtype=torch.float32)
        dh = torch.empty_like(h) if need_grad else None
        holder = {"dw": None, "first": True}
        for s in range(0, M, chunk):
            e = min(M, s + chunk)
            logits = gemm(h[s:e], w)
            if shard is None:
                _rows(logits, labels[s:e], 0, scale=scale, loss_sum=loss_sum)
            else:
                st = torch.empty(e - s, 3, device=h.device, dtype=torch.float32)
                _rows(logits, labels[s:e], 3, stats=st, vocab_start=shard.start, vocab_total=shard.total)
                lse, label_logit = _combine_shard_stats(st, shard)
                ok = (labels[s:e] != IGNORE) & (labels[s:e] >= 0) & (labels[s:e] < shard.total)
                loss_sum += torch.where(ok, lse - label_logit, torch.zeros_like(lse)).sum()
                if need_grad:
                    _rows(logits, labels[s:e], 4, scale=scale, lse=lse.contiguous(),
                          vocab_start=shard.start, vocab_total=shard.total)
            if not need_grad:
                continue  # logits hold gradients nobody wants; only loss_sum matters
            gemm(logits, w, b_mn=True, out=dh[s:e])
            if w.requires_grad:
                _dw_step(holder, w, logits, h[s:e])
            del logits
        if shard is not None and shard.reduce_dh and dh is not None:
            import torch.distributed as dist
            dist.all_reduce(dh, group=shard.group)
        ctx.dh = dh
        ctx.dw = holder["dw"]
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
        return dh, dw, None, None, None, None, None


def _sharded_logprob_torch(h, w, labels, inv_t, shard: VocabShard):
    """Plain-PyTorch (autograd) form of the vocabulary-sharded log-softmax pick: returns per-row
    ``(logp, lse, label_logit)``; used on CPU and as the oracle of the CUDA path."""
    from ..dist import comm
    if shard.reduce_dh:
        h = comm.copy_to_parallel_region(h, shard.group)
    logits = torch.nn.functional.linear(h, w.to(h.dtype)).float() * inv_t
    gm = comm.all_reduce(logits.detach().max(dim=-1).values, shard.group, op=torch.distributed.ReduceOp.MAX)
    ssum = comm.reduce_from_parallel_region(torch.exp(logits - gm[:, None]).sum(-1), shard.group)
    lse = gm + torch.log(ssum)
    local = labels - shard.start
    mine = (labels != IGNORE) & (local >= 0) & (local < shard.local)
    picked = logits.gather(-1, local.clamp(0, shard.local - 1)[:, None]).squeeze(-1)
    label_logit = comm.reduce_from_parallel_region(torch.where(mine, picked, torch.zeros_like(picked)), shard.group)
    ok = (labels != IGNORE) & (labels >= 0) & (labels < shard.total)
    return torch.where(ok, label_logit - lse, torch.zeros_like(lse)), ok


def lm_head_cross_entropy(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, loss_scale: float = 1.0,
                          chunk: int = DEFAULT_CHUNK, n_valid: Optional[torch.Tensor] = None,
                          shard: Optional[VocabShard] = None) -> torch.Tensor:
    """Mean CE of ``h @ w^T`` against ``labels`` (``-100`` ignored) without materialising the logits.

    The returned loss is the unscaled mean; the gradients carry ``loss_scale`` (use it for
    ``1/grad_accum`` and call ``backward()`` on the returned value directly — scaling the loss again
    would scale the gradients twice).  ``n_valid`` overrides the normaliser (e.g. a global count).
    With ``shard`` the rows of ``w`` are this rank's slice of the vocabulary: every rank computes its
    slice of the logits and the ranks exchange three floats per token (max, sum-exp, label logit).
    The reference keeps the LM head replicated on every TP rank (src/distributed/tensor_parallel.py:845).
    """
    labels = labels.reshape(-1)
    if n_valid is None:
        n_valid = (labels != IGNORE).sum()
    if not h.is_cuda:
        if shard is not None:
            lp, ok = _sharded_logprob_torch(h, w, labels, 1.0, shard)
            loss = -(lp.sum()) / n_valid.clamp(min=1).float()
            return _ScaleGrad.apply(loss, loss_scale)
        logits = torch.nn.functional.linear(h, w.to(h.dtype)).float()
        tot = torch.nn.functional.cross_entropy(logits, labels, ignore_index=IGNORE, reduction="sum")
        loss = tot / n_valid.clamp(min=1).float()
        return _ScaleGrad.apply(loss, loss_scale)
    return _LMHeadCE.apply(h.contiguous(), w, labels.long().contiguous(), float(loss_scale), int(chunk),
                           n_valid, shard)


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
    def forward(ctx, h, w, labels, inv_t, chunk, shard):
        M = h.shape[0]
        lse = torch.empty(M, device=h.device, dtype=torch.float32)
        logp = torch.empty(M, device=h.device, dtype=torch.float32)
        for s in range(0, M, chunk):
            e = min(M, s + chunk)
            logits = gemm(h[s:e], w)
            if shard is None:
                _rows(logits, labels[s:e], 1, lse=lse[s:e], logp=logp[s:e], inv_t=inv_t)
            else:
                st = torch.empty(e - s, 3, device=h.device, dtype=torch.float32)
                _rows(logits, labels[s:e], 3, stats=st, inv_t=inv_t, vocab_start=shard.start,
                      vocab_total=shard.total)
                l, label_logit = _combine_shard_stats(st, shard)
                ok = (labels[s:e] != IGNORE) & (labels[s:e] >= 0) & (labels[s:e] < shard.total)
                lse[s:e] = l
                logp[s:e] = torch.where(ok, label_logit - l, torch.zeros_like(l))
            del logits
        ctx.save_for_backward(h, w, labels, lse)
        ctx.args = (inv_t, chunk, shard)
        return logp

    @staticmethod
    def backward(ctx, g):
        h, w, labels, lse = ctx.saved_tensors
        inv_t, chunk, shard = ctx.args
        M = h.shape[0]
        g = g.contiguous().float()
        dh = torch.empty_like(h)
        dw_holder = {"dw": None, "first": True}
        vs, vt = (0, 0) if shard is None else (shard.start, shard.total)
        for s in range(0, M, chunk):
            e = min(M, s + chunk)
            logits = gemm(h[s:e], w)
            _rows(logits, labels[s:e], 2, lse=lse[s:e], g=g[s:e], inv_t=inv_t, vocab_start=vs, vocab_total=vt)
            gemm(logits, w, b_mn=True, out=dh[s:e])
            if w.requires_grad:
                _dw_step(dw_holder, w, logits, h[s:e])
            del logits
        if shard is not None and shard.reduce_dh:
            import torch.distributed as dist
            dist.all_reduce(dh, group=shard.group)
        return dh, dw_holder["dw"], None, None, None, None


def lm_head_logprob(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0,
                    chunk: int = DEFAULT_CHUNK, shard: Optional[VocabShard] = None) -> torch.Tensor:
    """``log softmax(h @ w^T / temperature)[label]`` per row as fp32 ``[M]`` (0 where label is -100).
    ``shard``: ``w`` holds this rank's slice of the vocabulary (see :func:`lm_head_cross_entropy`)."""
    labels = labels.reshape(-1)
    if not h.is_cuda and shard is not None:
        return _sharded_logprob_torch(h, w, labels, 1.0 / temperature, shard)[0]
    if not h.is_cuda:
        logits = torch.nn.functional.linear(h, w.to(h.dtype)).float() / temperature
        lp = torch.log_softmax(logits, dim=-1)
        safe = labels.clamp(min=0)
        out = lp.gather(-1, safe[:, None]).squeeze(-1)
        return torch.where(labels == IGNORE, torch.zeros_like(out), out)
    return _LMHeadLogprob.apply(h.contiguous(), w, labels.long().contiguous(), 1.0 / temperature, int(chunk),
                                shard)


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
