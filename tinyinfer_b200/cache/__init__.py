from .manager import (CacheExhausted, CacheGroup, CacheManager, PagePool, RequestCache,
                      group_cache_needs)
from .storage import CacheStorage, bytes_per_page

__all__ = ["CacheExhausted", "CacheGroup", "CacheManager", "PagePool", "RequestCache",
           "group_cache_needs", "CacheStorage", "bytes_per_page"]
