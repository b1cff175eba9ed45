"""Allocator of fixed-size cache pages: a free list and reference counts.

Semantics follow the reference's ``BlockManager`` (src/qwen25vl_lite/cache.py:36-91):
``allocate(n)`` is all-or-nothing and raises a ``MemoryError`` when fewer than ``n`` pages
are free (:44-57); pages are handed out from the top of the free list (LIFO), so a page
that was just given back is the next one used; frees are strict -- an id out of range, a
page that is not held, or a second free raises (:64-88).
"""

from __future__ import annotations

from typing import List, Sequence


class OutOfPages(MemoryError):
    """Fewer free pages than a request for pages asked for."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("num_pages must be positive")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(num_pages))
        self._refs: List[int] = [0] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def in_use(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self, n: int = 1) -> List[int]:
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"cannot allocate {n} pages; only {len(self._free)} of {self.num_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._refs[p] = 1
        return out

    def fork(self, pages: Sequence[int]) -> None:
        """One more holder for each page (pages shared between requests)."""
        for p in pages:
            self._held(p)
            self._refs[p] += 1

    def free(self, pages: Sequence[int]) -> None:
        """Drops one holder of each page; a page without holders returns to the free list."""
        for p in pages:
            p = self._held(p)
            self._refs[p] -= 1
            if self._refs[p] == 0:
                self._free.append(p)

    def refcount(self, page: int) -> int:
        return self._refs[page]

    def _held(self, p) -> int:
        p = int(p)
        if not 0 <= p < self.num_pages:
            raise ValueError(f"page id {p} is outside [0, {self.num_pages})")
        if self._refs[p] <= 0:
            raise ValueError(f"page {p} is not held (double free, or never allocated)")
        return p

    def check(self) -> None:
        """Every page is either free (once) or held; raises AssertionError otherwise."""
        free = set(self._free)
        assert len(free) == len(self._free), "a page is on the free list twice"
        for p in range(self.num_pages):
            assert (self._refs[p] == 0) == (p in free), f"page {p}: refcount {self._refs[p]}, free={p in free}"
