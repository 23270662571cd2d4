"""Page ownership on the host: a free list and reference counts for one pool of pages.

Parity: runtime/cache.py:10-32,79-84,100-107 (free list used LIFO, reference counts,
`MemoryError` on exhaustion with nothing changed, an invariant check).
"""
from __future__ import annotations

from typing import Iterable, List

import numpy as np


class OutOfPages(MemoryError):
    """The pool cannot give the pages a step needs; nothing was changed."""


class PagePool:
    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.n_pages = n_pages
        self.refs = np.zeros(n_pages, dtype=np.int32)
        self.free: List[int] = list(reversed(range(n_pages)))
        self.peak = 0
        self.taken = 0      # pages handed out so far, counting a page again each time it is reused

    @property
    def n_free(self) -> int:
        return len(self.free)

    @property
    def n_used(self) -> int:
        return self.n_pages - len(self.free)

    def allocate(self, count: int) -> List[int]:
        """Take `count` pages, all or none."""
        if count > len(self.free):
            raise OutOfPages(f"KV page pool exhausted: {count} pages wanted, {len(self.free)} free of {self.n_pages}")
        pages = [self.free.pop() for _ in range(count)]
        for page in pages:
            self.refs[page] = 1
        self.peak = max(self.peak, self.n_used)
        self.taken += count
        return pages

    def retain(self, page: int) -> None:
        if self.refs[page] <= 0:
            raise AssertionError(f"page {page} is not held by anyone")
        self.refs[page] += 1

    def release(self, page: int) -> None:
        if self.refs[page] <= 0:
            raise AssertionError(f"page {page} freed twice")
        self.refs[page] -= 1
        if self.refs[page] == 0:
            self.free.append(page)

    def check(self, tables: Iterable[Iterable[int]]) -> None:
        """Every page is held exactly as often as tables name it; free pages are exactly the unheld ones."""
        expected = np.zeros_like(self.refs)
        for table in tables:
            for page in table:
                if page >= 0:
                    expected[page] += 1
        if not np.array_equal(expected, self.refs):
            bad = np.flatnonzero(expected != self.refs)[:8].tolist()
            raise AssertionError(f"reference counts disagree with the block tables at pages {bad}")
        if len(self.free) != len(set(self.free)):
            raise AssertionError("a page is on the free list twice")
        if set(self.free) != set(np.flatnonzero(self.refs == 0).tolist()):
            raise AssertionError("the free list and the reference counts disagree")
