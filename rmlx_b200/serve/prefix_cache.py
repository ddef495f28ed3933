"""Radix tree from token-id prefixes to KV block ids, so requests that share a prompt prefix reuse
its cached pages (copy-on-write through ``BlockManager.fork``-style refcounts).

API of the reference's ``PrefixCache`` (crates/rmlx-nn/src/prefix_cache.rs:27-330): ``insert(tokens,
blocks)``, ``lookup(tokens) -> (matched_tokens, blocks)``, ``evict(n)`` (least recently used leaves
first). Matching is at block granularity: only whole blocks of ``block_size`` tokens are shared.
The reference leaves it unwired from its scheduler (prefix_cache.rs:9-17); here ``ServingEngine``
consults it on admission.
"""
from __future__ import annotations

import itertools
from typing import Dict, List, Optional, Sequence, Tuple


class _Node:
    __slots__ = ("children", "block", "last_used", "parent", "key")

    def __init__(self, parent=None, key=None, block: Optional[int] = None):
        self.children: Dict[Tuple[int, ...], "_Node"] = {}
        self.block = block
        self.last_used = 0
        self.parent = parent
        self.key = key


class PrefixCache:
    def __init__(self, block_size: int = 16, max_blocks: int = 0):
        self.block_size = block_size
        self.max_blocks = max_blocks          # 0 = unbounded
        self.root = _Node()
        self._clock = itertools.count(1)
        self._num_blocks = 0
        self.hits = 0
        self.misses = 0
        self._pending_evicted: List[int] = []

    def __len__(self) -> int:
        return self._num_blocks

    def _chunks(self, tokens: Sequence[int]):
        bs = self.block_size
        for i in range(0, len(tokens) - len(tokens) % bs, bs):
            yield tuple(int(t) for t in tokens[i:i + bs])

    def insert(self, tokens: Sequence[int], blocks: Sequence[int]) -> int:
        """Record that ``blocks[i]`` holds the KV of the i-th full block of ``tokens``. Returns the
        number of blocks newly recorded. Evicts old leaves when over ``max_blocks``; the caller
        releases the returned victims through ``take_evicted``."""
        return len(self.insert_blocks(tokens, blocks))

    def insert_blocks(self, tokens: Sequence[int], blocks: Sequence[int]) -> List[int]:
        """``insert`` that returns the block ids it newly recorded (the ones the caller must keep
        alive for the cache; chunks already present keep the block they had)."""
        node, new = self.root, []
        now = next(self._clock)
        for chunk, blk in zip(self._chunks(tokens), blocks):
            nxt = node.children.get(chunk)
            if nxt is None:
                nxt = _Node(node, chunk, int(blk))
                node.children[chunk] = nxt
                self._num_blocks += 1
                new.append(int(blk))
            nxt.last_used = now
            node = nxt
        if self.max_blocks and self._num_blocks > self.max_blocks:
            self._pending_evicted += self.evict(self._num_blocks - self.max_blocks)
        return new

    def lookup(self, tokens: Sequence[int]) -> Tuple[int, List[int]]:
        """Longest cached prefix: (number of matched tokens, their block ids)."""
        node, blocks = self.root, []
        now = next(self._clock)
        for chunk in self._chunks(tokens):
            nxt = node.children.get(chunk)
            if nxt is None:
                break
            nxt.last_used = now
            blocks.append(nxt.block)
            node = nxt
        if blocks:
            self.hits += 1
        else:
            self.misses += 1
        return len(blocks) * self.block_size, blocks

    def evict(self, n: int) -> List[int]:
        """Drop up to ``n`` least-recently-used leaf blocks; returns their block ids."""
        victims: List[int] = []
        for _ in range(n):
            leaves = []
            stack = [self.root]
            while stack:
                nd = stack.pop()
                if nd is not self.root and not nd.children:
                    leaves.append(nd)
                stack.extend(nd.children.values())
            if not leaves:
                break
            leaf = min(leaves, key=lambda x: x.last_used)
            del leaf.parent.children[leaf.key]
            self._num_blocks -= 1
            victims.append(leaf.block)
        return victims

    def take_evicted(self) -> List[int]:
        v, self._pending_evicted = self._pending_evicted, []
        return v

    def clear(self) -> List[int]:
        return self.evict(self._num_blocks)
