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
