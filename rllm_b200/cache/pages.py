"""Page and slot bookkeeping on the host: who holds which page.

A pool hands out page numbers from a LIFO free list (so a page given back is the next
one handed out: reuse is immediate, as in the reference's `KvPool`,
src/model/kv_cache.rs:779, 852-857). Holding is tracked per page so that a page can
never be lost, held twice or freed twice; violations raise instead of corrupting the
cache (the reference panics on a stale handle, src/model/kv_cache.rs:864-875)."""
from __future__ import annotations


class OutOfPages(RuntimeError):
    """No free page (or state slot) is left; the caller decides who has to wait."""


class CacheError(RuntimeError):
    """A bookkeeping rule was broken (double free, unknown page, ...)."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise ValueError("num_pages must be >= 0")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))    # pop() yields 0, 1, 2, ...
        self._owner: list[object | None] = [None] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self, owner) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        page = self._free.pop()
        if self._owner[page] is not None:
            raise CacheError(f"page {page} was on the free list while held by {self._owner[page]!r}")
        self._owner[page] = owner
        return page

    def free(self, page: int, owner) -> None:
        if not 0 <= page < self.num_pages:
            raise CacheError(f"page {page} does not exist")
        if self._owner[page] is None:
            raise CacheError(f"page {page} freed twice")
        if self._owner[page] != owner:
            raise CacheError(f"page {page} is held by {self._owner[page]!r}, not {owner!r}")
        self._owner[page] = None
        self._free.append(page)

    def owner(self, page: int):
        return self._owner[page]

    def check(self) -> None:
        """Every page is either free or held, never both, never neither."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError("a page is on the free list twice")
        for p in range(self.num_pages):
            if (p in free) == (self._owner[p] is not None):
                raise CacheError(f"page {p}: free-list and holder disagree")
