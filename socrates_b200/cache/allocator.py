"""Host-side free list of cache pages.

Same contract as the reference's BlockAllocator (model/paging.py:22-65): pages are
numbered 1..num_pages, page 0 is the null page and is never handed out, freed pages
are reused last-in first-out, `alloc` fails without side effects, and `free`
validates every page before it changes anything.
"""

from __future__ import annotations

from typing import Iterable, List


class OutOfPages(Exception):
    """More pages were asked for than are free."""


def pages_for(tokens: int, page_size: int) -> int:
    """Pages that `tokens` slots occupy, rounded up (model/paging.py:17-19)."""
    return -(-tokens // page_size)


class PageAllocator:
    NULL = 0

    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise ValueError("a pool needs at least one usable page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages, 0, -1))   # popped from the end: 1, 2, 3, ...
        self._used: set[int] = set()

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_used(self) -> int:
        return len(self._used)

    def alloc(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError(f"cannot allocate {n} pages")
        if n > len(self._free):
            raise OutOfPages(f"asked for {n} pages, {len(self._free)} free")
        out = [self._free.pop() for _ in range(n)]
        self._used.update(out)
        return out

    def free(self, pages: Iterable[int]) -> None:
        pages = list(pages)
        seen = set()
        for p in pages:
            if p == self.NULL:
                raise ValueError("page 0 is the null page and is never allocated")
            if p not in self._used or p in seen:
                raise ValueError(f"page {p} freed twice, or never allocated")
            seen.add(p)
        for p in reversed(pages):
            self._used.remove(p)
            self._free.append(p)

    def check(self) -> None:
        """Every page is either free or used, exactly once."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a page is on the free list twice")
        if free & self._used:
            raise AssertionError(f"pages both free and used: {sorted(free & self._used)}")
        if free | self._used != set(range(1, self.num_pages + 1)):
            raise AssertionError("a page was lost")
