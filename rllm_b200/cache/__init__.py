from .manager import CacheGroup, CacheManager, RequestCache, pages_for
from .pages import CacheError, OutOfPages, PagePool

__all__ = ["CacheGroup", "CacheManager", "RequestCache", "pages_for", "CacheError",
           "OutOfPages", "PagePool"]
