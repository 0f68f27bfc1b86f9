"""Inference-side ops: paged KV store / gather, paged decode attention (split-KV + LSE merge),
variable-length causal attention over contiguous K/V, batched top-p sampling.

Reference call sites: ``store_kv_cache`` incl. its Triton kernel and fp8 path
(src/inference/attention.py:44-183), ``flash_attn_varlen_func`` / ``flash_attn_with_kvcache`` and the
SDPA fall-backs in ``PagedAttention`` (:188-382), ``PartitionedPagedAttention`` (:387-626), and the
sort-based samplers (src/inference/model_runner.py:590-634, src/inference/engine.py:979-1020).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .. import _native as nv

FP8_MAX = 448.0


# ---- KV store -------------------------------------------------------------------------------------
def kv_store(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
             segments: torch.Tensor, k_scale: Optional[torch.Tensor] = None,
             v_scale: Optional[torch.Tensor] = None) -> None:
    """Write new K/V rows into cache blocks.  ``k [T, Hkv*D]``, ``v [T, Hkv*D]`` (rows may be strided);
    caches ``[blocks, 16, Hkv, D]``; ``segments`` int32 ``[n,4]`` = (block, first row, count, first slot).
    fp8 caches (uint8) carry per-(block, head) scales that only grow; earlier tokens of the block are
    requantised when a new token raises the scale."""
    fp8 = k_cache.dtype == torch.uint8
    nblk, bs, Hkv, D = k_cache.shape
    if not k.is_cuda:
        for blk, t0, cnt, off in segments.tolist():
            if blk < 0 or cnt <= 0:
                continue
            for src, cache, scale in ((k, k_cache, k_scale), (v, v_cache, v_scale)):
                new = src[t0:t0 + cnt].reshape(cnt, Hkv, D).float()
                if not fp8:
                    cache[blk, off:off + cnt] = new.to(cache.dtype)
                    continue
                amax = new.abs().amax(dim=(0, 2))
                old = scale[blk] if off > 0 else torch.zeros(Hkv)
                ns = torch.maximum(old, amax / FP8_MAX)
                ns = torch.where(ns > 0, ns, torch.full_like(ns, 1.0 / FP8_MAX))
                if off > 0:
                    prev = cache[blk, :off].view(torch.float8_e4m3fn).float() * old[None, :, None]
                    cache[blk, :off] = (prev / ns[None, :, None]).to(torch.float8_e4m3fn).view(torch.uint8)
                cache[blk, off:off + cnt] = (new / ns[None, :, None]).to(torch.float8_e4m3fn).view(torch.uint8)
                scale[blk] = ns
        return
    assert D == 128 and bs == 16
    nv.check(nv.lib().b2_kv_store(nv.ptr(k), nv.ptr(v), k.stride(0), v.stride(0), nv.ptr(k_cache), nv.ptr(v_cache),
                                  nv.ptr(k_scale), nv.ptr(v_scale), nv.ptr(segments), segments.shape[0], Hkv, D,
                                  int(fp8), nv.stream_ptr()), "kv_store")
    nv.count_launch()


def kv_gather(k_cache: torch.Tensor, v_cache: torch.Tensor, slots: torch.Tensor, dtype: torch.dtype,
              k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None
              ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Cache rows ``slots`` (= block*16 + offset) as contiguous ``[rows, Hkv*D]`` tensors, dequantised."""
    fp8 = k_cache.dtype == torch.uint8
    nblk, bs, Hkv, D = k_cache.shape
    rows = slots.numel()
    if not k_cache.is_cuda:
        def take(cache, scale):
            flat = cache.reshape(nblk * bs, Hkv, D)[slots.long()]
            if fp8:
                flat = flat.view(torch.float8_e4m3fn).float() * scale[slots.long() // bs][:, :, None]
            return flat.reshape(rows, Hkv * D).to(dtype)
        return take(k_cache, k_scale), take(v_cache, v_scale)
    ko = torch.empty((rows, Hkv * D), device=k_cache.device, dtype=dtype)
    vo = torch.empty_like(ko)
    nv.check(nv.lib().b2_kv_gather(nv.ptr(k_cache), nv.ptr(v_cache), nv.ptr(k_scale), nv.ptr(v_scale),
                                   nv.ptr(slots), nv.ptr(ko), nv.ptr(vo), rows, Hkv, D, int(fp8),
                                   nv.stream_ptr()), "kv_gather")
    nv.count_launch()
    return ko, vo


# ---- paged decode attention --------------------------------------------------------------------------
def paged_decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                           block_tables: torch.Tensor, context_lens: torch.Tensor, Hq: int,
                           scale: Optional[float] = None, k_scale: Optional[torch.Tensor] = None,
                           v_scale: Optional[torch.Tensor] = None, partition: int = 0, nsplit: int = 1,
                           workspace: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
    """One query token per sequence against its paged keys.  ``q [B, Hq*D]``; ``nsplit > 1`` partitions
    every sequence into ``partition``-token ranges that are merged exactly by log-sum-exp."""
    nblk, bs, Hkv, D = k_cache.shape
    B = q.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    fp8 = k_cache.dtype == torch.uint8
    if not q.is_cuda:
        out = torch.zeros((B, Hq * D), dtype=q.dtype)
        ctx = context_lens.tolist()
        for b in range(B):
            n = ctx[b]
            if n <= 0:
                continue
            pos = torch.arange(n)
            slots = (block_tables[b, pos // bs].long() * bs + pos % bs).to(torch.int32)
            K, V = kv_gather(k_cache, v_cache, slots, torch.float32, k_scale, v_scale)
            K, V = K.reshape(n, Hkv, D), V.reshape(n, Hkv, D)
            g = Hq // Hkv
            qb = q[b].float().reshape(Hkv, g, D)
            att = torch.einsum("hgd,nhd->hgn", qb, K) * scale
            out[b] = torch.einsum("hgn,nhd->hgd", att.softmax(-1), V).reshape(Hq * D).to(q.dtype)
        return out
    out = torch.empty((B, Hq * D), device=q.device, dtype=q.dtype)
    if nsplit > 1:
        if workspace is None:
            workspace = (torch.empty((B, Hq, nsplit, D), device=q.device, dtype=torch.float32),
                         torch.empty((B, Hq, nsplit, 2), device=q.device, dtype=torch.float32))
        part_o, part_ml = workspace
    else:
        part_o = part_ml = None
        partition = partition or (1 << 30) // 64 * 64
    nv.check(nv.lib().b2_paged_decode(nv.ptr(q), nv.ptr(k_cache), nv.ptr(v_cache), nv.ptr(k_scale), nv.ptr(v_scale),
                                      nv.ptr(block_tables), nv.ptr(context_lens), block_tables.shape[1],
                                      nv.ptr(out), nv.ptr(part_o), nv.ptr(part_ml), nv.ptr(None), B, Hq, Hkv, D,
                                      int(partition), int(nsplit), nv.ctypes.c_float(scale), int(fp8),
                                      nv.stream_ptr()), "paged_decode")
    nv.count_launch(2 if nsplit > 1 else 1)
    return out


# ---- variable-length causal attention (prefill chunks, speculative verify) ---------------------------
def varlen_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_q: torch.Tensor, cu_k: torch.Tensor,
                     max_q: int, Hq: int, Hkv: int, scale: Optional[float] = None) -> torch.Tensor:
    """Sequence ``b`` owns query rows ``cu_q[b]:cu_q[b+1]`` and key rows ``cu_k[b]:cu_k[b+1]``; its
    queries are the last positions of its keys (query ``i`` sees keys ``0..kv_len-q_len+i``)."""
    D = q.shape[-1] // Hq
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    B = cu_q.numel() - 1
    if not q.is_cuda:
        out = torch.empty_like(q)
        cq, ck = cu_q.tolist(), cu_k.tolist()
        g = Hq // Hkv
        for b in range(B):
            nq, nk = cq[b + 1] - cq[b], ck[b + 1] - ck[b]
            if nq == 0:
                continue
            qb = q[cq[b]:cq[b + 1]].float().reshape(nq, Hkv, g, D)
            kb = k[ck[b]:ck[b + 1]].float().reshape(nk, Hkv, D)
            vb = v[ck[b]:ck[b + 1]].float().reshape(nk, Hkv, D)
            att = torch.einsum("qhgd,khd->hgqk", qb, kb) * scale
            allowed = torch.arange(nk)[None, :] <= (torch.arange(nq)[:, None] + (nk - nq))
            att = att.masked_fill(~allowed, float("-inf")).softmax(-1)
            out[cq[b]:cq[b + 1]] = torch.einsum("hgqk,khd->qhgd", att, vb).reshape(nq, Hq * D).to(q.dtype)
        return out
    assert D == 128
    q, k = q.contiguous(), (k if k.stride(-1) == 1 else k.contiguous())
    out = torch.empty_like(q)
    nv.check(nv.lib().b2_attn_fwd_varlen(nv.ptr(q), nv.ptr(k), nv.ptr(v), nv.ptr(out), nv.ptr(None), B, 0, Hq, Hkv,
                                         D, k.stride(0), v.stride(0), nv.ctypes.c_float(scale), nv.ptr(cu_q),
                                         nv.ptr(cu_k), int(max_q), q.shape[0], k.shape[0], nv.stream_ptr()),
             "attn_fwd_varlen")
    nv.count_launch()
    return out


def paged_prefill_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                            cu_q: torch.Tensor, cu_k: torch.Tensor, max_q: int, Hq: int,
                            scale: Optional[float] = None, k_scale: Optional[torch.Tensor] = None,
                            v_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of prefill chunks straight over the paged cache: sequence ``b`` owns query rows
    ``cu_q[b]:cu_q[b+1]``; its keys / values are the first ``cu_k[b+1] - cu_k[b]`` tokens of the cache blocks
    ``block_tables[b]`` (the chunk's own K / V already stored), its queries the last positions of them.  The kernel's
    TMA producer walks the block table, so the context is never gathered into a contiguous buffer (the reference
    hands ``block_table=`` to ``flash_attn_varlen_func``: src/inference/attention.py:248-257).  bf16 caches only;
    an fp8 cache is dequantised by :func:`kv_gather` and goes through :func:`varlen_attention`."""
    nblk, bs, Hkv, D = k_cache.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    B = cu_q.numel() - 1
    if not q.is_cuda or k_cache.dtype == torch.uint8:
        ck = cu_k.tolist()
        slots = []
        for b in range(B):
            pos = torch.arange(ck[b + 1] - ck[b])
            slots.append((block_tables[b, pos // bs].long() * bs + pos % bs).to(torch.int32))
        slot = torch.cat(slots).to(q.device)
        K, V = kv_gather(k_cache, v_cache, slot, q.dtype if q.is_cuda else torch.float32, k_scale, v_scale)
        return varlen_attention(q, K.to(q.dtype), V.to(q.dtype), cu_q, cu_k, max_q, Hq, Hkv, scale)
    assert D == 128 and bs == 16 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    q = q.contiguous()
    out = torch.empty_like(q)
    nv.check(nv.lib().b2_attn_fwd_paged(nv.ptr(q), nv.ptr(k_cache), nv.ptr(v_cache), nv.ptr(out), nv.ptr(None), B, Hq,
                                        Hkv, D, nblk, nv.ctypes.c_float(scale), nv.ptr(cu_q), nv.ptr(cu_k),
                                        nv.ptr(block_tables), block_tables.shape[1], int(max_q), q.shape[0],
                                        nv.stream_ptr()), "attn_fwd_paged")
    nv.count_launch()
    return out


# ---- sampling ------------------------------------------------------------------------------------------
def topp_sample(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, uniform: torch.Tensor,
                return_logprob: bool = False):
    """Temperature + nucleus sampling for a batch of rows with per-row parameters (device tensors, no
    host sync).  ``temperature <= 0`` is greedy.  ``uniform`` in [0,1) drives the draw, so a fixed
    ``uniform`` makes the result reproducible.  Returns token ids (and the log-prob of each pick under
    the tempered full softmax)."""
    B, V = logits.shape
    if not logits.is_cuda:
        ids = torch.empty(B, dtype=torch.long)
        lps = torch.zeros(B)
        for b in range(B):
            t = float(temperature[b])
            row = logits[b].float()
            if t <= 0:
                ids[b] = int(row.argmax())
                continue
            lp = torch.log_softmax(row / t, -1)
            p = lp.exp()
            sp, si = p.sort(descending=True)
            keep_sorted = (sp.cumsum(0) - sp) < min(max(float(top_p[b]), 0.0), 1.0)
            keep_sorted[0] = True           # top_p <= 0 keeps the most likely token (the kernel's clamp)
            keep = torch.zeros(V, dtype=torch.bool)
            keep[si[keep_sorted]] = True
            kept = torch.where(keep, p, torch.zeros_like(p))
            c = kept.cumsum(0)
            r = min(float(uniform[b]), 0.99999994) * float(c[-1])
            pick = int(torch.searchsorted(c, torch.tensor(r), right=True).clamp(max=V - 1))
            ids[b] = pick
            lps[b] = lp[pick]
        return (ids, lps) if return_logprob else ids
    assert logits.stride(-1) == 1 and logits.dtype in (torch.float32, torch.bfloat16)
    ids = torch.empty(B, device=logits.device, dtype=torch.long)
    lps = torch.empty(B, device=logits.device, dtype=torch.float32) if return_logprob else None
    nv.check(nv.lib().b2_topp_sample(nv.ptr(logits), int(logits.dtype == torch.float32), B, V, logits.stride(0),
                                     nv.ptr(temperature), nv.ptr(top_p), nv.ptr(uniform), nv.ptr(ids), nv.ptr(lps),
                                     nv.stream_ptr()), "topp_sample")
    nv.count_launch()
    return (ids, lps) if return_logprob else ids
