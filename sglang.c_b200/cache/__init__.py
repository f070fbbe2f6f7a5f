from .manager import CacheError, CacheManager
from .needs import CacheBinding, CacheNeed
from .pages import PagePool, PagePoolError

__all__ = ["CacheError", "CacheManager", "CacheBinding", "CacheNeed", "PagePool", "PagePoolError"]
