"""Hash-chain prefix cache over full KV blocks (src/inference/prefix_cache.py:56-265).

Block ``i`` of a prompt is keyed by ``hash(prev_hash, tokens_of_block_i)``; a hit is verified against the
stored token tuple, bumps LRU order, and returns the physical block ids, which the engine *shares*
(reference count) instead of recomputing — the reference matches prefixes but never reuses the blocks
(src/inference/engine.py:1111-1114).
"""
from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict
from typing import List, Tuple

try:
    import xxhash

    def _h(data: bytes) -> int:
        return xxhash.xxh64(data).intdigest()
except ImportError:  # pragma: no cover - depends on the image
    def _h(data: bytes) -> int:
        return int.from_bytes(hashlib.sha256(data).digest()[:8], "little")


class CachedBlock:
    __slots__ = ("hash_value", "block_id", "token_ids", "ref_count")

    def __init__(self, hash_value: int, block_id: int, token_ids: Tuple[int, ...]):
        self.hash_value, self.block_id, self.token_ids, self.ref_count = hash_value, block_id, token_ids, 0


class PrefixCache:
    def __init__(self, block_size: int = 16, max_cached_blocks: int = 1024):
        self.block_size, self.max_cached_blocks = block_size, max_cached_blocks
        self.entries: "OrderedDict[int, CachedBlock]" = OrderedDict()
        self.hits = self.misses = self.evictions = 0
        self.on_evict = None     # callback(block_id) so the owner can drop its reference

    def compute_block_hash(self, token_ids: List[int], prev_hash: int = 0) -> int:
        return _h(struct.pack(f"<Q{len(token_ids)}q", prev_hash & (2 ** 64 - 1), *token_ids))

    def _chain(self, token_ids: List[int]):
        prev = 0
        for s in range(0, len(token_ids) - self.block_size + 1, self.block_size):
            blk = tuple(token_ids[s:s + self.block_size])
            prev = self.compute_block_hash(list(blk), prev)
            yield prev, blk

    def match_prefix(self, token_ids: List[int]) -> Tuple[int, List[int]]:
        """Longest cached prefix in whole blocks -> (matched token count, block ids)."""
        ids: List[int] = []
        for hv, blk in self._chain(token_ids):
            e = self.entries.get(hv)
            if e is None or e.token_ids != blk:
                break
            self.entries.move_to_end(hv)
            e.ref_count += 1
            ids.append(e.block_id)
        if ids:
            self.hits += 1
        else:
            self.misses += 1
        return len(ids) * self.block_size, ids

    def insert(self, token_ids: List[int], block_ids: List[int]) -> List[int]:
        """Register the full blocks of a sequence; returns the block ids newly taken into the cache."""
        new = []
        for (hv, blk), bid in zip(self._chain(token_ids), block_ids):
            if hv in self.entries:
                self.entries.move_to_end(hv)
                continue
            if len(self.entries) >= self.max_cached_blocks:
                self.evict_lru(1)
                if len(self.entries) >= self.max_cached_blocks:
                    break
            self.entries[hv] = CachedBlock(hv, bid, blk)
            new.append(bid)
        return new

    def release_block(self, block_hash: int):
        e = self.entries.get(block_hash)
        if e is not None and e.ref_count > 0:
            e.ref_count -= 1

    def release_blocks(self, block_ids: List[int]):
        wanted = set(block_ids)
        for e in self.entries.values():
            if e.block_id in wanted and e.ref_count > 0:
                e.ref_count -= 1

    def evict_lru(self, num_blocks: int = 1) -> List[int]:
        """Evict least-recently-used entries nobody references; returns their block ids."""
        out = []
        for hv in list(self.entries):
            if len(out) >= num_blocks:
                break
            e = self.entries[hv]
            if e.ref_count == 0:
                del self.entries[hv]
                out.append(e.block_id)
                self.evictions += 1
                if self.on_evict:
                    self.on_evict(e.block_id)
        return out

    def invalidate_all(self) -> List[int]:
        ids = [e.block_id for e in self.entries.values()]
        if self.on_evict:
            for b in ids:
                self.on_evict(b)
        self.entries.clear()
        return ids

    @property
    def hit_rate(self) -> float:
        n = self.hits + self.misses
        return self.hits / n if n else 0.0

    @property
    def size(self) -> int:
        return len(self.entries)

    def get_stats(self) -> dict:
        return {"size": self.size, "hits": self.hits, "misses": self.misses, "hit_rate": self.hit_rate,
                "evictions": self.evictions, "max_cached_blocks": self.max_cached_blocks}
