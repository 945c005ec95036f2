"""Host-side bookkeeping of which cache pages are out and which can be handed out.

The contract is the one the reference's block allocator keeps (model/paging.py:22-65):
usable pages are numbered 1..num_pages, page 0 stands for "no page" and never leaves,
the page given back last is handed out first, a request for more pages than are free
changes nothing, and a `free` that names a bad page changes nothing either.

The form is this engine's own: a fixed stack of page numbers with a fill mark, and
one state byte per page.  The byte answers "is this page out?" in O(1), which is
what `free`, `holds` and `check` are built on; a cache group with hundreds of
thousands of pages allocates nothing after construction.
"""

from __future__ import annotations

from array import array
from typing import Iterable, List

_IN, _OUT, _LEAVING = 0, 1, 2        # page state: in the stack, held by a row, named by the free() in progress


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
        # _stack[:_fill] are the pages that are in; the top of the stack leaves first, and
        # the stack starts with page 1 on top
        self._stack = array("i", range(num_pages, 0, -1))
        self._fill = num_pages
        self._state = bytearray(num_pages + 1)
        self._state[self.NULL] = _LEAVING                 # never in, never out: no transition accepts it

    @property
    def n_free(self) -> int:
        return self._fill

    @property
    def n_used(self) -> int:
        return self.num_pages - self._fill

    def holds(self, page: int) -> bool:
        """Whether `page` is out (held by somebody) right now."""
        return 0 < page <= self.num_pages and self._state[page] == _OUT

    def alloc(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError(f"a request for {n} pages makes no sense")
        if n > self._fill:
            raise OutOfPages(f"{n} pages wanted but only {self._fill} of {self.num_pages} are in")
        top = self._fill
        taken = [self._stack[top - 1 - i] for i in range(n)]
        self._fill = top - n
        for p in taken:
            self._state[p] = _OUT
        return taken

    def free(self, pages: Iterable[int]) -> None:
        pages = [int(p) for p in pages]
        # first pass marks, so a page named twice in one call is seen; any fault undoes the marks
        for i, p in enumerate(pages):
            if not 0 <= p <= self.num_pages or self._state[p] != _OUT:
                for q in pages[:i]:
                    self._state[q] = _OUT
                if p == self.NULL:
                    raise ValueError("the null page (0) is nobody's to give back")
                raise ValueError(f"page {p} is not out: given back already, named twice, or not of this pool")
            self._state[p] = _LEAVING
        # pushed back to front, so the pages come out again in the order they were named
        for p in reversed(pages):
            self._stack[self._fill] = p
            self._fill += 1
            self._state[p] = _IN

    def check(self) -> None:
        """Every usable page is in the stack exactly once or out, never both, none missing."""
        seen = bytearray(self.num_pages + 1)
        for i in range(self._fill):
            p = self._stack[i]
            if not 0 < p <= self.num_pages:
                raise AssertionError(f"the stack holds {p}, which is no page of this pool")
            if seen[p]:
                raise AssertionError(f"page {p} is in the stack twice")
            if self._state[p] != _IN:
                raise AssertionError(f"page {p} is in the stack and marked as out")
            seen[p] = 1
        out = sum(1 for p in range(1, self.num_pages + 1) if self._state[p] == _OUT)
        stale = [p for p in range(1, self.num_pages + 1) if self._state[p] == _LEAVING]
        if stale:
            raise AssertionError(f"pages left half-freed: {stale}")
        if out + self._fill != self.num_pages:
            raise AssertionError("a page was lost: neither in the stack nor out")
