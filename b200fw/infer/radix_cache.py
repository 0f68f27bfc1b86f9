"""Block-granular radix tree prefix cache (src/inference/radix_cache.py:59-320).

Each edge is one full block of tokens; children are keyed by the block's first token and verified on
the whole block; a conflicting child is replaced only when nobody references it; eviction removes
least-recently-used leaves.  Same interface as :class:`PrefixCache`.
"""
from __future__ import annotations

import itertools
from typing import Dict, List, Optional, Tuple


class RadixNode:
    __slots__ = ("tokens", "block_id", "children", "parent", "ref_count", "last_access")

    def __init__(self, tokens: Tuple[int, ...] = (), block_id: int = -1, parent: Optional["RadixNode"] = None):
        self.tokens, self.block_id, self.parent = tokens, block_id, parent
        self.children: Dict[int, "RadixNode"] = {}
        self.ref_count = 0
        self.last_access = 0


class RadixAttentionCache:
    def __init__(self, block_size: int = 16, max_nodes: int = 10000):
        self.block_size, self.max_nodes = block_size, max_nodes
        self.root = RadixNode()
        self.num_nodes = 0
        self._clock = itertools.count(1)
        self.hits = self.misses = self.evictions = 0
        self.on_evict = None

    def _blocks(self, token_ids: List[int]):
        for s in range(0, len(token_ids) - self.block_size + 1, self.block_size):
            yield tuple(token_ids[s:s + self.block_size])

    def match_prefix(self, token_ids: List[int]) -> Tuple[int, List[int]]:
        node, ids = self.root, []
        for blk in self._blocks(token_ids):
            child = node.children.get(blk[0])
            if child is None or child.tokens != blk:
                break
            child.last_access = next(self._clock)
            child.ref_count += 1
            ids.append(child.block_id)
            node = child
        if ids:
            self.hits += 1
        else:
            self.misses += 1
        return len(ids) * self.block_size, ids

    def insert(self, token_ids: List[int], block_ids: List[int]) -> List[int]:
        node, new = self.root, []
        for blk, bid in zip(self._blocks(token_ids), block_ids):
            child = node.children.get(blk[0])
            if child is not None and child.tokens != blk:
                if child.ref_count > 0 or child.children:
                    break                      # occupied by a different live block: stop here
                self._drop(child)
                child = None
            if child is None:
                if self.num_nodes >= self.max_nodes:
                    # never the node the new block hangs under: as the deepest node of this path it is a leaf, and
                    # evicting it would attach the new block to a detached node (unreachable, never evicted: a leak)
                    self.evict_lru(1, protect=node)
                    if self.num_nodes >= self.max_nodes:
                        break
                child = RadixNode(blk, bid, node)
                node.children[blk[0]] = child
                self.num_nodes += 1
                new.append(bid)
            child.last_access = next(self._clock)
            node = child
        return new

    def _drop(self, node: RadixNode):
        if node.parent is not None:
            node.parent.children.pop(node.tokens[0], None)
        self.num_nodes -= 1
        self.evictions += 1
        if self.on_evict:
            self.on_evict(node.block_id)

    def _leaves(self) -> List[RadixNode]:
        out, stack = [], [self.root]
        while stack:
            n = stack.pop()
            if n is not self.root and not n.children:
                out.append(n)
            stack.extend(n.children.values())
        return out

    def evict_lru(self, num_blocks: int = 1, protect: Optional[RadixNode] = None) -> List[int]:
        out = []
        for _ in range(num_blocks):
            cands = [n for n in self._leaves() if n.ref_count == 0 and n is not protect]
            if not cands:
                break
            victim = min(cands, key=lambda n: n.last_access)
            out.append(victim.block_id)
            self._drop(victim)
        return out

    def release_blocks(self, block_ids: List[int]):
        wanted = set(block_ids)
        stack = [self.root]
        while stack:
            n = stack.pop()
            if n.block_id in wanted and n.ref_count > 0:
                n.ref_count -= 1
            stack.extend(n.children.values())

    def release_block(self, block_hash: int):   # interface parity with PrefixCache (hash == block id here)
        self.release_blocks([block_hash])

    def invalidate_all(self) -> List[int]:
        ids, stack = [], list(self.root.children.values())
        while stack:
            n = stack.pop()
            ids.append(n.block_id)
            stack.extend(n.children.values())
        if self.on_evict:
            for b in ids:
                self.on_evict(b)
        self.root = RadixNode()
        self.num_nodes = 0
        return ids

    @property
    def hit_rate(self) -> float:
        n = self.hits + self.misses
        return self.hits / n if n else 0.0

    @property
    def size(self) -> int:
        return self.num_nodes

    def get_stats(self) -> dict:
        return {"size": self.size, "hits": self.hits, "misses": self.misses, "hit_rate": self.hit_rate,
                "evictions": self.evictions, "max_nodes": self.max_nodes}
