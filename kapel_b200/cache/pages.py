"""Pages of a cache and the pool that hands them out.

Kapel keeps a free list with reference counts and a typed `CacheFull{needed, free}`
(crates/kapel-models/src/cache.rs:148-150,419-433; crates/kapel-models/src/lib.rs:70-77).
Here pages are never shared, so a page is either free or held by exactly one owner; the pool
checks that on every call. The bookkeeping itself is in the host library
(`csrc/host/cache_core.cpp`), built with the C++ compiler alone at first use.
"""
from __future__ import annotations

import ctypes

from ..hostlib import host_library  # noqa: F401  (the manager takes it from here)


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
        self._lib = host_library()
        self._h = self._lib.kp_create(n_pages)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.kp_destroy(self._h)
            self._h = None

    @property
    def free(self) -> int:
        return self._lib.kp_free(self._h)

    @property
    def held(self) -> int:
        return self.n_pages - self.free

    def take(self) -> int:
        page = self._lib.kp_take(self._h)
        if page == -1:
            raise CacheFull(1, 0)
        if page < 0:
            raise AssertionError("a page was on the free list while held")
        return page

    def give(self, page: int) -> None:
        r = self._lib.kp_give(self._h, int(page))
        if r == -1:
            raise ValueError(f"page {page} is not of this pool (0..{self.n_pages - 1})")
        if r == -2:
            raise ValueError(f"page {page} is given back twice")

    def is_held(self, page: int) -> bool:
        return bool(self._lib.kp_is_held(self._h, int(page)))

    def check(self) -> None:
        """Every page is free or held, never both, none lost."""
        msg = ctypes.create_string_buffer(256)
        if self._lib.kp_check(self._h, msg, 256):
            raise AssertionError(msg.value.decode())
