"""Per-step attention metadata handed explicitly to the kernels (the reference keeps it in a module
global, src/inference/context.py:22-75)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class InferenceContext:
    is_prefill: bool
    num_seqs: int
    # decode / paged attention
    block_tables: Optional[torch.Tensor] = None      # int32 [num_seqs, max_blocks] (padding: -1)
    context_lens: Optional[torch.Tensor] = None      # int32 [num_seqs], including the tokens of this step
    max_context_len: int = 0
    # KV store: int32 [nseg, 4] = (block id, first token row, count, first slot in block)
    store_segments: Optional[torch.Tensor] = None
    # prefill (variable length)
    cu_seqlens_q: Optional[torch.Tensor] = None      # int32 [num_seqs + 1]
    cu_seqlens_k: Optional[torch.Tensor] = None      # int32 [num_seqs + 1]
    max_seqlen_q: int = 0
    total_q: int = 0
    total_k: int = 0
    gather_slots: Optional[torch.Tensor] = None      # int32 [total_k]: cache slot of every key row (None:
                                                     # every sequence starts at position 0 -> use the chunk's own K/V)
    positions: Optional[torch.Tensor] = None         # int32 [total_q]
    last_token_rows: Optional[torch.Tensor] = None   # int64 [num_seqs]: row of each sequence's last query
    # ---- fields of the reference's context that the kernels here do not need (src/inference/context.py:22-40):
    max_seqlen_k: int = 0                            # filled by prepare_prefill for callers that want it
    slot_mapping: Optional[torch.Tensor] = None      # per-token slot ids; the store kernel takes `store_segments`

    def slots_from_segments(self, block_size: int = 16) -> Optional[torch.Tensor]:
        """The reference's ``slot_mapping`` (int64 ``[tokens]``: ``block * block_size + offset``, ``-1`` = skip)
        expanded from the segment list."""
        if self.store_segments is None:
            return None
        seg = self.store_segments.cpu().tolist()
        n = max((row + cnt for blk, row, cnt, _ in seg if blk >= 0), default=0)
        out = torch.full((n,), -1, dtype=torch.int64)
        for blk, row, cnt, first in seg:
            if blk >= 0 and cnt > 0:
                out[row:row + cnt] = blk * block_size + first + torch.arange(cnt)
        return out


# The reference passes the context through a module-level global that attention layers read
# (src/inference/context.py:43-75); the engine here hands it to ``ModelRunner.forward`` explicitly, and these
# three helpers exist for code written against the global style.
_CONTEXT: Optional[InferenceContext] = None


_SET_CONTEXT_ORDER = ("cu_seqlens_q", "cu_seqlens_k", "max_seqlen_q", "max_seqlen_k", "slot_mapping", "context_lens",
                      "block_tables")


def set_context(is_prefill: bool, *args, **fields) -> InferenceContext:
    """Publish the step's metadata.  Fields by keyword; positionally they follow the reference's order
    (src/inference/context.py:43-62): cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, slot_mapping,
    context_lens, block_tables."""
    global _CONTEXT
    if len(args) > len(_SET_CONTEXT_ORDER):
        raise TypeError("set_context() takes at most %d positional fields" % len(_SET_CONTEXT_ORDER))
    for name, value in zip(_SET_CONTEXT_ORDER, args):
        if name in fields:
            raise TypeError(f"set_context() got multiple values for {name!r}")
        if value is not None:
            fields[name] = value
    _CONTEXT = InferenceContext(is_prefill, fields.pop("num_seqs", 0), **fields)
    return _CONTEXT


def get_context() -> Optional[InferenceContext]:
    return _CONTEXT


def reset_context():
    global _CONTEXT
    _CONTEXT = None

