"""Paged KV cache: blocks, the block pool, per-sequence block tables and the manager.

Same structures and policies as the reference (src/inference/kv_cache.py:32-486): reference-counted
blocks, FIFO free list, rollback when an allocation cannot complete, one spare block kept by
``can_allocate``, double-free detection.  Storage differs: one tensor
``[2, layers, blocks, block_size, kv_heads, head_dim]`` in the model's 16-bit dtype, or fp8-e4m3 bytes
with one fp32 scale per (block, kv head) — the reference keeps per-token scales.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Deque, Dict, List, Optional

import torch

from ..obs.logging import get_logger

# fp8 K/V is stored as e4m3 bytes (uint8 tensors, one fp32 scale per block and kv head; the kernels convert); these two
# names say so in the reference's terms (src/inference/kv_cache.py:30-38)
HAS_FP8 = hasattr(torch, "float8_e4m3fn")
_FP8_DTYPE = getattr(torch, "float8_e4m3fn", None)

logger = get_logger("infer.kv_cache")


@dataclass
class Block:
    block_id: int
    ref_count: int = 0
    token_count: int = 0
    block_hash: Optional[int] = None
    block_size: int = 16

    def reset(self):
        self.ref_count, self.token_count, self.block_hash = 0, 0, None

    # the reference's field names (src/inference/kv_cache.py:48-60)
    @property
    def hash_value(self) -> Optional[int]:
        return self.block_hash

    @hash_value.setter
    def hash_value(self, v: Optional[int]):
        self.block_hash = v

    @property
    def is_full(self) -> bool:
        return self.token_count >= self.block_size


class BlockPool:
    def __init__(self, num_blocks: int, block_size: int, num_layers: int, num_kv_heads: int, head_dim: int,
                 dtype: torch.dtype = torch.bfloat16, device="cpu", kv_cache_dtype: str = "fp16",
                 allocate: bool = True, cache_dtype: Optional[str] = None):
        kv_cache_dtype = cache_dtype if cache_dtype is not None else kv_cache_dtype     # `cache_dtype`: the reference's name
        self.num_blocks, self.block_size = num_blocks, block_size
        self.num_layers, self.num_kv_heads, self.head_dim = num_layers, num_kv_heads, head_dim
        self.fp8 = kv_cache_dtype == "fp8"
        self.dtype, self.device = dtype, torch.device(device)
        self.blocks = [Block(i, block_size=block_size) for i in range(num_blocks)]
        self.free_list: Deque[int] = deque(range(num_blocks))
        self.kv: Optional[torch.Tensor] = None
        self.scales: Optional[torch.Tensor] = None
        self.double_free_count = 0
        if allocate:
            self._allocate()

    def _allocate(self):
        shape = (2, self.num_layers, self.num_blocks, self.block_size, self.num_kv_heads, self.head_dim)
        try:
            self.kv = torch.zeros(shape, dtype=torch.uint8 if self.fp8 else self.dtype, device=self.device)
        except RuntimeError as e:  # out of device memory: keep running with host storage
            logger.warning("KV pool does not fit on %s (%s); falling back to host memory", self.device, e)
            self.device = torch.device("cpu")
            self.kv = torch.zeros(shape, dtype=torch.uint8 if self.fp8 else self.dtype, device=self.device)
        if self.fp8:
            self.scales = torch.zeros((2, self.num_layers, self.num_blocks, self.num_kv_heads),
                                      dtype=torch.float32, device=self.device)

    # ---- allocation ---------------------------------------------------------------------------------
    def allocate(self) -> Optional[Block]:
        if not self.free_list:
            return None
        b = self.blocks[self.free_list.popleft()]
        b.reset()
        b.ref_count = 1
        return b

    def share(self, block_id: int) -> Block:
        """Take another reference on a block that is in use (prefix reuse)."""
        b = self.blocks[block_id]
        if b.ref_count == 0:        # cached but unreferenced: pull it off the free list
            try:
                self.free_list.remove(block_id)
            except ValueError:
                pass
        b.ref_count += 1
        return b

    def free(self, block: Block):
        if block.ref_count <= 0:
            self.double_free_count += 1
            logger.warning("double free of block %d ignored", block.block_id)
            return
        block.ref_count -= 1
        if block.ref_count == 0:
            self.free_list.append(block.block_id)

    def get_block(self, block_id: int) -> Block:
        return self.blocks[block_id]

    @property
    def num_free_blocks(self) -> int:
        return len(self.free_list)

    @property
    def num_used_blocks(self) -> int:
        return self.num_blocks - len(self.free_list)

    @property
    def utilization(self) -> float:
        return self.num_used_blocks / max(1, self.num_blocks)

    # ---- storage views --------------------------------------------------------------------------------
    def layer_kv(self, layer: int):
        return self.kv[0, layer], self.kv[1, layer]

    def layer_scales(self, layer: int):
        if self.scales is None:
            return None, None
        return self.scales[0, layer], self.scales[1, layer]

    @property
    def kv_cache_tensor(self) -> Optional[torch.Tensor]:
        return self.kv

    def get_flattened_kv_cache(self) -> Optional[torch.Tensor]:
        """``[2, layers, blocks * block_size, kv_heads, head_dim]`` view of the pool, indexable by slot
        (``block_id * block_size + offset``); shares memory with the pool (src/inference/kv_cache.py:241-256)."""
        if self.kv is None:
            return None
        two, L, nb, bs = self.kv.shape[:4]
        return self.kv.view(two, L, nb * bs, *self.kv.shape[4:])


class BlockTable:
    def __init__(self, block_size: int):
        self.block_size = block_size
        self._blocks: List[Block] = []
        self.num_tokens = 0

    def append_block(self, block: Block):
        self._blocks.append(block)

    def get_physical_block_ids(self) -> List[int]:
        return [b.block_id for b in self._blocks]

    @property
    def last_block(self) -> Optional[Block]:
        return self._blocks[-1] if self._blocks else None

    @property
    def num_blocks(self) -> int:
        return len(self._blocks)

    @property
    def blocks(self) -> List[Block]:
        return self._blocks

    @property
    def capacity(self) -> int:
        return len(self._blocks) * self.block_size


class KVCacheManager:
    def __init__(self, block_pool: BlockPool, block_size: int = 16):
        self.pool, self.block_size = block_pool, block_size
        self.tables: Dict[object, BlockTable] = {}
        self.alloc_failures = 0

    def blocks_needed(self, num_tokens: int) -> int:
        return (num_tokens + self.block_size - 1) // self.block_size

    def can_allocate(self, num_tokens: int) -> bool:
        return self.pool.num_free_blocks >= self.blocks_needed(num_tokens) + 1   # keep one spare

    def allocate_for_sequence(self, seq_id, num_initial_tokens: int = 0,
                              shared_block_ids: Optional[List[int]] = None) -> Optional[BlockTable]:
        """New table covering ``num_initial_tokens``; ``shared_block_ids`` (a cached prefix) are
        referenced instead of allocated.  Rolls everything back and returns None when the pool runs dry."""
        assert seq_id not in self.tables, f"sequence {seq_id} already has a block table"
        table = BlockTable(self.block_size)
        for bid in shared_block_ids or []:
            table.append_block(self.pool.share(bid))
        need = self.blocks_needed(num_initial_tokens) - table.num_blocks
        for _ in range(max(0, need)):
            b = self.pool.allocate()
            if b is None:
                for blk in table.blocks:
                    self.pool.free(blk)
                self.alloc_failures += 1
                return None
            table.append_block(b)
        table.num_tokens = num_initial_tokens
        self.tables[seq_id] = table
        return table

    def ensure_capacity(self, seq_id, num_tokens: int) -> bool:
        """Grow the table to hold ``num_tokens`` tokens (chunked prefill / speculative lookahead)."""
        table = self.tables[seq_id]
        added = []
        while table.capacity < num_tokens:
            b = self.pool.allocate()
            if b is None:
                for blk in added:
                    table.blocks.pop()
                    self.pool.free(blk)
                self.alloc_failures += 1
                return False
            table.append_block(b)
            added.append(b)
        return True

    def append_token(self, seq_id) -> bool:
        table = self.tables[seq_id]
        if not self.ensure_capacity(seq_id, table.num_tokens + 1):
            return False
        table.num_tokens += 1
        return True

    def set_num_tokens(self, seq_id, n: int):
        self.tables[seq_id].num_tokens = n

    def trim(self, seq_id, num_tokens: int):
        """Drop blocks beyond ``num_tokens`` (rejected speculative tokens)."""
        table = self.tables[seq_id]
        keep = max(1, self.blocks_needed(num_tokens))
        while table.num_blocks > keep:
            self.pool.free(table.blocks.pop())
        table.num_tokens = num_tokens

    def free_sequence(self, seq_id):
        table = self.tables.pop(seq_id, None)
        if table is None:
            return
        for b in table.blocks:
            self.pool.free(b)

    def get_block_table(self, seq_id) -> List[int]:
        t = self.tables.get(seq_id)
        return [] if t is None else t.get_physical_block_ids()

    def get_seq_token_count(self, seq_id) -> int:
        t = self.tables.get(seq_id)
        return 0 if t is None else t.num_tokens

    def reset(self):
        for sid in list(self.tables):
            self.free_sequence(sid)

    def get_stats(self) -> dict:
        return {"num_blocks": self.pool.num_blocks, "free_blocks": self.pool.num_free_blocks,
                "used_blocks": self.pool.num_used_blocks, "utilization": self.pool.utilization,
                "num_sequences": len(self.tables), "alloc_failures": self.alloc_failures,
                "double_frees": self.pool.double_free_count}
