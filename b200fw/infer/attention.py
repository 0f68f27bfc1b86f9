"""Attention modules over the paged KV cache, in the reference's module style.

The engine's ``ModelRunner`` calls the kernels directly (``ops.kv_store``, ``ops.varlen_attention``,
``ops.paged_decode_attention``) with an explicit :class:`InferenceContext`.  The reference instead places a
``PagedAttention`` module in every layer that reads the step's metadata from a module-level context and owns
views of its layer's cache (src/inference/attention.py:44-72, 188-382; the partitioned variant with the exact
log-sum-exp merge: :387-626).  These classes give that shape to the same kernels, for code that builds its own
model around the cache: bind the layer's cache views, publish the context with ``set_context`` and call the
module with ``[tokens, heads, head_dim]`` tensors.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .context import InferenceContext, get_context

# The reference sets this when the flash_attn library imports (src/inference/attention.py:28-32).  Attention here is
# this package's own kernel: available whenever a CUDA device is (the CPU path is the plain softmax formula).
HAS_FLASH_ATTN = torch.cuda.is_available()

__all__ = ["store_kv_cache", "PagedAttention", "PartitionedPagedAttention", "HAS_FLASH_ATTN"]


def _segments_from_slots(slot_mapping: torch.Tensor, block_size: int) -> torch.Tensor:
    """Per-token slot ids (``block * block_size + offset``, ``-1`` = skip) -> the store kernel's segment list
    ``[n, 4]`` = (block, first token row, count, first slot in block), one segment per token."""
    slots = slot_mapping.to(torch.int64).reshape(-1)
    rows = torch.arange(slots.numel(), device=slots.device)
    keep = slots >= 0
    blk = torch.where(keep, slots // block_size, torch.full_like(slots, -1))
    seg = torch.stack([blk, rows, keep.to(torch.int64), torch.where(keep, slots % block_size, torch.zeros_like(slots))], 1)
    return seg.to(torch.int32).contiguous()


def store_kv_cache(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                   slot_mapping: torch.Tensor, k_scale: Optional[torch.Tensor] = None,
                   v_scale: Optional[torch.Tensor] = None, cache_dtype: str = "fp16") -> None:
    """Scatter new K/V rows into the cache.  ``key`` / ``value`` ``[tokens, kv_heads, head_dim]`` (or already
    flattened to ``[tokens, kv_heads*head_dim]``); caches ``[blocks, block_size, kv_heads, head_dim]``; slot ``-1``
    skips the token.  An fp8 cache (uint8 storage) needs its per-(block, head) scale tensors."""
    T = key.shape[0]
    k2, v2 = key.reshape(T, -1), value.reshape(T, -1)
    if k_cache.dtype == torch.uint8 and (k_scale is None or v_scale is None):
        raise ValueError("an fp8 KV cache needs k_scale / v_scale")
    ops.kv_store(k2, v2, k_cache, v_cache, _segments_from_slots(slot_mapping, k_cache.shape[1]).to(key.device),
                 k_scale, v_scale)


class PagedAttention(torch.nn.Module):
    """``forward(q, k, v)``: store the new K/V rows, then variable-length causal attention over the step's own
    rows (prefill) or one query token per sequence against its pages (decode)."""

    def __init__(self, num_heads: int, num_kv_heads: int, head_dim: int, cache_dtype: str = "fp16"):
        super().__init__()
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.scale = head_dim ** -0.5
        self.cache_dtype = cache_dtype
        self.k_cache: Optional[torch.Tensor] = None      # [blocks, block_size, kv_heads, head_dim]
        self.v_cache: Optional[torch.Tensor] = None
        self.k_scale: Optional[torch.Tensor] = None      # fp8: [blocks, kv_heads]
        self.v_scale: Optional[torch.Tensor] = None

    def bind_cache(self, k_cache, v_cache, k_scale=None, v_scale=None):
        """Views of this layer's part of the pool (``BlockPool.layer_kv(i)`` / ``layer_scales(i)``)."""
        self.k_cache, self.v_cache, self.k_scale, self.v_scale = k_cache, v_cache, k_scale, v_scale
        return self

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                ctx: Optional[InferenceContext] = None) -> torch.Tensor:
        ctx = ctx if ctx is not None else get_context()
        if ctx is None:
            raise RuntimeError("no InferenceContext: pass one or call set_context() first")
        T = q.shape[0]
        q2, k2, v2 = q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)
        if self.k_cache is not None:
            if ctx.store_segments is not None:
                ops.kv_store(k2, v2, self.k_cache, self.v_cache, ctx.store_segments, self.k_scale, self.v_scale)
            elif ctx.slot_mapping is not None:
                store_kv_cache(k2, v2, self.k_cache, self.v_cache, ctx.slot_mapping, self.k_scale, self.v_scale)
        out = self._prefill_attention(q2, k2, v2, ctx) if ctx.is_prefill else self._decode_attention(q2, ctx)
        return out.reshape(T, self.num_heads, self.head_dim)

    def _prefill_attention(self, q, k, v, ctx: InferenceContext) -> torch.Tensor:
        if ctx.block_tables is not None and self.k_cache is not None and ctx.cu_seqlens_k is not None:
            # keys / values read in place through the block table (src/inference/attention.py:248-257)
            return ops.paged_prefill_attention(q, self.k_cache, self.v_cache, ctx.block_tables, ctx.cu_seqlens_q,
                                               ctx.cu_seqlens_k, ctx.max_seqlen_q, self.num_heads, self.scale,
                                               self.k_scale, self.v_scale)
        if ctx.gather_slots is not None:          # part of the keys (a cached prefix, earlier chunks) lives in pages
            k, v = ops.kv_gather(self.k_cache, self.v_cache, ctx.gather_slots, q.dtype, self.k_scale, self.v_scale)
        cu_k = ctx.cu_seqlens_k if ctx.cu_seqlens_k is not None else ctx.cu_seqlens_q
        return ops.varlen_attention(q, k, v, ctx.cu_seqlens_q, cu_k, ctx.max_seqlen_q, self.num_heads,
                                    self.num_kv_heads)

    def _split(self, ctx: InferenceContext):
        return 0, 1

    def _decode_attention(self, q, ctx: InferenceContext) -> torch.Tensor:
        if self.k_cache is None:
            raise RuntimeError("decode needs a bound KV cache (bind_cache)")
        part, nsplit = self._split(ctx)
        return ops.paged_decode_attention(q, self.k_cache, self.v_cache, ctx.block_tables, ctx.context_lens,
                                          self.num_heads, scale=self.scale, k_scale=self.k_scale, v_scale=self.v_scale,
                                          partition=part, nsplit=nsplit)


class PartitionedPagedAttention(PagedAttention):
    """Decode splits every sequence into ``partition_size``-token ranges once the longest context exceeds it;
    the partial results are merged exactly with the log-sum-exp rule (one extra small kernel)."""

    def __init__(self, num_heads: int, num_kv_heads: int, head_dim: int, cache_dtype: str = "fp16",
                 partition_size: int = 512):
        super().__init__(num_heads, num_kv_heads, head_dim, cache_dtype)
        self.partition_size = max(64, partition_size // 64 * 64)

    def _split(self, ctx: InferenceContext):
        longest = ctx.max_context_len or (int(ctx.context_lens.max()) if ctx.context_lens is not None else 0)
        if longest <= self.partition_size:
            return 0, 1
        return self.partition_size, (longest + self.partition_size - 1) // self.partition_size
