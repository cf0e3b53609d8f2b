"""Page and slot bookkeeping on the host: who holds which page.

A pool hands out page numbers from a LIFO free list (so a page given back is the next
one handed out: reuse is immediate, as in the reference's `KvPool`,
src/model/kv_cache.rs:779, 852-857). Holding is tracked per page so that a page can
never be lost, held twice or freed twice; violations raise instead of corrupting the
cache (the reference panics on a stale handle, src/model/kv_cache.rs:864-875).

The bookkeeping itself is native (csrc/host_runtime.cpp); this class gives it the holders'
own names: a holder may be any hashable object."""
from __future__ import annotations

from .native import lib


class OutOfPages(RuntimeError):
    """No free page (or state slot) is left; the caller decides who has to wait."""


class CacheError(RuntimeError):
    """A bookkeeping rule was broken (double free, unknown page, ...)."""


class Holders:
    """Holder object <-> the 64-bit key the native side stores."""

    def __init__(self):
        self._key: dict[object, int] = {}
        self._obj: dict[int, object] = {}
        self._next = 0

    def key(self, obj) -> int:
        k = self._key.get(obj)
        if k is None:
            k = self._key[obj] = self._next
            self._obj[k] = obj
            self._next += 1
        return k

    def obj(self, key: int):
        return self._obj.get(key)

    def forget(self, obj) -> None:
        k = self._key.pop(obj, None)
        if k is not None:
            self._obj.pop(k, None)


class PagePool:
    def __init__(self, num_pages: int, _ptr=None, _holders: Holders | None = None, _owner=None):
        if num_pages < 0:
            raise ValueError("num_pages must be >= 0")
        self._L = lib()
        self._owned = _ptr is None              # a pool inside a native cache is freed with the cache
        self._ptr = self._L.pool_new(num_pages) if _ptr is None else _ptr
        self._keep = _owner                     # keeps the native cache alive while this view exists
        self.holders = _holders or Holders()
        self.num_pages = num_pages

    def __del__(self):
        if getattr(self, "_owned", False) and self._ptr:
            self._L.pool_delete(self._ptr)
            self._ptr = None

    @property
    def num_free(self) -> int:
        return self._L.pool_num_free(self._ptr)

    def alloc(self, owner) -> int:
        page = self._L.pool_alloc(self._ptr, self.holders.key(owner))
        if page == -1:
            raise OutOfPages("no free page")
        if page < 0:
            raise CacheError("a page was on the free list while held")
        return page

    def free(self, page: int, owner) -> None:
        rc = self._L.pool_release(self._ptr, page, self.holders.key(owner))
        if rc == -1:
            raise CacheError(f"page {page} does not exist")
        if rc == -2:
            raise CacheError(f"page {page} freed twice")
        if rc == -3:
            raise CacheError(f"page {page} is held by {self.owner(page)!r}, not {owner!r}")

    def owner(self, page: int):
        k = self._L.pool_holder(self._ptr, page)
        return None if k == self._L.NOBODY else self.holders.obj(k)

    def check(self) -> None:
        """Every page is either free or held, never both, never neither."""
        rc = self._L.pool_check(self._ptr)
        if rc == -2:
            raise CacheError("a page is on the free list twice")
        if rc:
            raise CacheError("a page's free-list entry and its holder disagree")
