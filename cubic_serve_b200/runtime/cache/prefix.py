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
    def __init__(self, pool: PagePool, enabled: bool = True, checkpoint_slots: tuple[int, ...] | None = None) -> None:
        """``checkpoint_slots``: rows of the executor's recurrent-state arrays set aside for snapshots.  Given (models
        with recurrent layers), a prefix can only be resumed where such a snapshot exists: ``match`` returns the longest
        cached prefix that ENDS at a checkpointed block, and ``publish_checkpoint`` records one (reference: the state
        slot snapshots shared by refcount beside the pages, ``runtime/performance.py:11018-11152``)."""
        self.pool = pool
        self.enabled = enabled
        self._map: OrderedDict[bytes, int] = OrderedDict()
        self.needs_checkpoint = checkpoint_slots is not None
        self._free_ckpt: list[int] = list(checkpoint_slots or ())
        self._ckpt: dict[bytes, int] = {}          # digest of a chain's last block -> checkpoint slot
        self.last_checkpoint: int | None = None    # snapshot slot of the prefix returned by the latest ``match``
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
        self.last_checkpoint = None
        if self.needs_checkpoint:
            # only a boundary with a snapshot of the recurrent state can be resumed from
            while found and found[-1] not in self._ckpt:
                found.pop()
                pages.pop()
            if found:
                self.last_checkpoint = self._ckpt[found[-1]]
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

    def publish_checkpoint(self, tokens, extra: bytes = b"") -> int | None:
        """Reserve a snapshot slot for the boundary at the end of ``tokens`` (whole blocks, already published as pages);
        returns the slot to copy the request's recurrent state into, or None (nothing free and nothing evictable, or the
        boundary is checkpointed already)."""
        if not self.enabled or not self.needs_checkpoint:
            return None
        chain = block_digests(tokens, extra)
        if not chain or chain[-1] not in self._map or chain[-1] in self._ckpt:
            return None
        if not self._free_ckpt:
            self._evict_checkpoint(exclude=set(chain))
        if not self._free_ckpt:
            return None
        slot = self._free_ckpt.pop()
        self._ckpt[chain[-1]] = slot
        return slot

    def _evict_checkpoint(self, exclude: set) -> None:
        """Free the least recently used snapshot whose block nobody else holds.  The block's page stays cached: it is
        still part of longer chains that end at another snapshot."""
        for d in list(self._map.keys()):
            if d in self._ckpt and d not in exclude and self.pool.refcount(self._map[d]) == 1:
                self._free_ckpt.append(self._ckpt.pop(d))
                return

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
                if d in self._ckpt:
                    self._free_ckpt.append(self._ckpt.pop(d))
                self.pool.release([page])
                freed += 1
        return freed

    def clear(self) -> None:
        for page in self._map.values():
            self.pool.release([page])
        self._map.clear()
        self._free_ckpt += list(self._ckpt.values())
        self._ckpt.clear()

    @property
    def hit_rate(self) -> float:
        return self.hit_tokens / self.lookup_tokens if self.lookup_tokens else 0.0
