"""Reference-counted page pool and copy-on-write bookkeeping for the paged KV cache.

Host-side twin of the device cache tensors: pages are integers, shared between
requests by reference count (prefix reuse), and written only by a sole owner
(copy-on-write otherwise).  Same responsibilities as the reference's free-list
heaps with COW + refcounts in the controller
(``runtime/performance.py:9184-9234,11632``) and ``runtime/cache/allocator.py:46``.
"""
from __future__ import annotations

import heapq


class OutOfPages(RuntimeError):
    """No free page is left (after prefix-cache eviction)."""


class PoolPoisoned(RuntimeError):
    """An invariant broke; the pool refuses further use (fail-closed like ``cache/pages.py:665``)."""


class PagePool:
    def __init__(self, num_pages: int, reserved: int = 1) -> None:
        """``reserved`` leading pages are never handed out (page 0 backs padding rows)."""
        if num_pages <= reserved:
            raise ValueError("pool needs more pages than it reserves")
        self.num_pages = num_pages
        self.reserved = reserved
        self._free = list(range(reserved, num_pages))
        heapq.heapify(self._free)
        self._ref = [0] * num_pages
        self._poisoned = False

    # ------------------------------------------------------------------
    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - self.reserved - len(self._free)

    def refcount(self, page: int) -> int:
        return self._ref[page]

    def _check(self) -> None:
        if self._poisoned:
            raise PoolPoisoned("page pool is poisoned")

    def poison(self) -> None:
        self._poisoned = True

    def alloc(self, n: int) -> list[int]:
        self._check()
        if n > len(self._free):
            raise OutOfPages(f"need {n} pages, {len(self._free)} free")
        pages = [heapq.heappop(self._free) for _ in range(n)]
        for p in pages:
            if self._ref[p] != 0:
                self.poison()
                raise PoolPoisoned(f"free page {p} has references")
            self._ref[p] = 1
        return pages

    def retain(self, pages) -> None:
        self._check()
        for p in pages:
            if self._ref[p] <= 0:
                self.poison()
                raise PoolPoisoned(f"retain of unowned page {p}")
            self._ref[p] += 1

    def release(self, pages) -> None:
        self._check()
        for p in pages:
            if self._ref[p] <= 0:
                self.poison()
                raise PoolPoisoned(f"release of unowned page {p}")
            self._ref[p] -= 1
            if self._ref[p] == 0:
                heapq.heappush(self._free, p)

    def writable(self, page: int) -> bool:
        """A page may be written in place only by its sole owner."""
        return self._ref[page] == 1

    def cow(self, page: int) -> tuple[int, bool]:
        """Return a page the caller may write: the same page if solely owned, else a fresh copy target.

        The boolean tells the caller to copy the old contents (device ``copy_pages``) before writing.
        """
        self._check()
        if self._ref[page] == 1:
            return page, False
        new = self.alloc(1)[0]
        self.release([page])
        return new, True
