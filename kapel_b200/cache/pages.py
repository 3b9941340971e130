"""Pages of a cache and the pool that hands them out.

Kapel keeps a free list with reference counts and a typed `CacheFull{needed, free}`
(crates/kapel-models/src/cache.rs:148-150,419-433; crates/kapel-models/src/lib.rs:70-77).
Here pages are never shared, so a page is either free or held by exactly one owner; the pool
checks that on every call.
"""
from __future__ import annotations

from typing import List


class CacheFull(RuntimeError):
    """A pool has fewer free pages than a step needs."""

    def __init__(self, needed: int, free: int, group: str = ""):
        self.needed, self.free, self.group = needed, free, group
        where = f" in group {group}" if group else ""
        super().__init__(f"cache full{where}: {needed} pages needed, {free} free")


class PagePool:
    """`n_pages` pages numbered from 0; the page freed last is taken first."""

    def __init__(self, n_pages: int):
        if n_pages < 0:
            raise ValueError(f"a pool cannot have {n_pages} pages")
        self.n_pages = n_pages
        # Pop takes from the end: page 0 first in a fresh pool.
        self._free: List[int] = list(range(n_pages - 1, -1, -1))
        self._held = [False] * n_pages

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return self.n_pages - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheFull(1, 0)
        page = self._free.pop()
        if self._held[page]:
            raise AssertionError(f"page {page} was on the free list while held")
        self._held[page] = True
        return page

    def give(self, page: int) -> None:
        if not 0 <= page < self.n_pages:
            raise ValueError(f"page {page} is not of this pool (0..{self.n_pages - 1})")
        if not self._held[page]:
            raise ValueError(f"page {page} is given back twice")
        self._held[page] = False
        self._free.append(page)

    def is_held(self, page: int) -> bool:
        return self._held[page]

    def check(self) -> None:
        """Every page is free or held, never both, none lost."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a page is on the free list twice")
        for p in range(self.n_pages):
            if self._held[p] == (p in free):
                raise AssertionError(f"page {p}: held={self._held[p]} but on the free list={p in free}")
