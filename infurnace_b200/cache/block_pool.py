"""The pool of physical pages of one cache group.

The reference's ``cache/block_pool.py`` is an empty file; its documents ask for a pool
with atomic multi-page allocation and rollback and for randomised allocate/free traces
(docs/architecture.md:219-257, docs/roadmap.md:323-337, docs/numerical_validation.md:65-82).

Pages are handed out last-freed-first, so a page that a finished request gave back is
the next to be used: stale content in a reused page is met early if any kernel reads
past a request's own keys.
"""
from __future__ import annotations

from typing import List

from ..errors import CacheError, OutOfPages


class BlockPool:
    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise CacheError("a pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # pop() gives page 0 first
        self._held = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self, n: int) -> List[int]:
        """``n`` pages, or :class:`OutOfPages` with the pool unchanged."""
        if n < 0:
            raise CacheError("cannot allocate a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"asked for {n} pages, {len(self._free)} free of {self.num_pages}")
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._held[p] = True
        return pages

    def free(self, pages) -> None:
        pages = list(pages)
        seen = set()
        for p in pages:                      # check everything before changing anything
            if not isinstance(p, int) or not 0 <= p < self.num_pages:
                raise CacheError(f"page id {p!r} is not in this pool")
            if not self._held[p] or p in seen:
                raise CacheError(f"page {p} is freed twice")
            seen.add(p)
        for p in pages:
            self._held[p] = False
            self._free.append(p)

    def is_held(self, page: int) -> bool:
        return self._held[page]

    def check(self) -> None:
        """Every page is either free once or held, never both."""
        if len(set(self._free)) != len(self._free):
            raise CacheError("a page is on the free list twice")
        for p in self._free:
            if self._held[p]:
                raise CacheError(f"page {p} is both free and held")
        if sum(self._held) + len(self._free) != self.num_pages:
            raise CacheError("a page is lost: held + free != total")
