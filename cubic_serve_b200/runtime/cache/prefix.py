"""Prefix cache: completed 16-token KV pages shared across requests.

Keyed like the reference controller's cache (``runtime/performance.py:11018-11152``):
a rolling BLAKE2s digest over 16-token blocks (each key commits to the whole
prefix), LRU order, pages held by reference count so that a cached page can be
in use by live requests and is reclaimed only when the cache is its last owner.
"""
from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict

from .pool import PagePool

BLOCK = 16


def block_digests(tokens, extra: bytes = b"", limit_blocks: int | None = None) -> list[bytes]:
    """Chained digests of the full 16-token blocks of ``tokens``."""
    n = len(tokens) // BLOCK
    if limit_blocks is not None:
        n = min(n, limit_blocks)
    out = []
    prev = hashlib.blake2s(extra, digest_size=16).digest()
    for i in range(n):
        blk = tokens[i * BLOCK:(i + 1) * BLOCK]
        h = hashlib.blake2s(prev, digest_size=16)
        h.update(struct.pack(f"<{BLOCK}q", *[int(t) for t in blk]))
        prev = h.digest()
        out.append(prev)
    return out


class PrefixCache:
    def __init__(self, pool: PagePool, enabled: bool = True) -> None:
        self.pool = pool
        self.enabled = enabled
        self._map: OrderedDict[bytes, int] = OrderedDict()
        self.hits = 0
        self.lookups = 0
        self.hit_tokens = 0
        self.lookup_tokens = 0

    def __len__(self) -> int:
        return len(self._map)

    def match(self, tokens, extra: bytes = b"", max_tokens: int | None = None) -> list[int]:
        """Longest cached prefix (whole blocks); returned pages are retained for the caller.

        ``max_tokens`` caps the match (a request must always compute at least its last prompt token).
        """
        if not self.enabled:
            return []
        limit = None if max_tokens is None else max_tokens // BLOCK
        pages: list[int] = []
        found = []
        for d in block_digests(tokens, extra, limit):
            page = self._map.get(d)
            if page is None:
                break
            found.append(d)
            pages.append(page)
        self._touch(found)
        self.lookups += 1
        self.lookup_tokens += len(tokens)
        if pages:
            self.hits += 1
            self.hit_tokens += len(pages) * BLOCK
            self.pool.retain(pages)
        return pages

    def publish(self, tokens, pages, extra: bytes = b"") -> int:
        """Offer the fully written leading pages of a request; returns how many new blocks were kept."""
        if not self.enabled:
            return 0
        added = 0
        chain = block_digests(tokens, extra, len(pages))
        for d, page in zip(chain, pages):
            if d in self._map:
                continue
            self.pool.retain([page])
            self._map[d] = page
            added += 1
        self._touch(chain[:len(pages)])
        return added

    def _touch(self, chain) -> None:
        """Mark a chain of blocks as used, leaf first and root last: a block is only reachable through the blocks
        before it, so within a chain the LEAF must be the first to go.  (Touching in chain order would make the
        root the least recently used one; evicting it strands the rest of the chain, unreachable yet holding
        pages.)"""
        for d in reversed(chain):
            self._map.move_to_end(d)

    def evictable(self) -> int:
        """Entries whose page only the cache holds (what ``evict`` could free right now)."""
        return sum(1 for page in self._map.values() if self.pool.refcount(page) == 1)

    def evict(self, need_pages: int) -> int:
        """Drop least-recently-used entries whose page nobody else holds until ``need_pages`` were freed."""
        freed = 0
        for d in list(self._map.keys()):
            if freed >= need_pages:
                break
            page = self._map[d]
            if self.pool.refcount(page) == 1:
                del self._map[d]
                self.pool.release([page])
                freed += 1
        return freed

    def clear(self) -> None:
        for page in self._map.values():
            self.pool.release([page])
        self._map.clear()

    @property
    def hit_rate(self) -> float:
        return self.hit_tokens / self.lookup_tokens if self.lookup_tokens else 0.0
