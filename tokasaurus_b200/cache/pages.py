"""Page ownership on the host: which pages of a pool are free and who holds the others.

The reference's allocator (tokasaurus/manager/allocator.py:129-418) also keeps a prefix tree for
sharing pages between requests; this one hands out whole pages to one owner each, from a LIFO
free list so that a page given back is the next one handed out (stale contents must never
show).  ``NoSpaceError`` is the reference's ``NoSpaceException`` (allocator.py:60-61).
"""

from __future__ import annotations


class NoSpaceError(ValueError):
    """The pool has fewer free pages than were asked for."""


class PageAllocator:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: list[int] = list(range(num_pages - 1, -1, -1))  # pop() gives page 0 first
        self._owner: list[object | None] = [None] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, n: int, owner: object) -> list[int]:
        if owner is None:
            raise ValueError("pages need an owner")
        if n > len(self._free):
            raise NoSpaceError(f"asked for {n} pages, {len(self._free)} of {self.num_pages} are free")
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._owner[p] = owner
        return pages

    def release(self, pages: list[int], owner: object) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page {p} is not in this pool")
            if self._owner[p] is None:
                raise ValueError(f"page {p} is freed twice")
            if self._owner[p] != owner:
                raise ValueError(f"page {p} belongs to {self._owner[p]!r}, not to {owner!r}")
        if len(set(pages)) != len(pages):
            raise ValueError("a page is named twice in one release")
        for p in pages:
            self._owner[p] = None
            self._free.append(p)

    def owner_of(self, page: int):
        return self._owner[page]

    def check(self) -> None:
        """Every page is free or owned, never both, never twice in the free list."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a page is in the free list twice")
        for p in range(self.num_pages):
            if (p in free) == (self._owner[p] is not None):
                raise AssertionError(f"page {p}: free={p in free}, owner={self._owner[p]!r}")
