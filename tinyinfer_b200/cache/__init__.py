from .manager import (CacheExhausted, CacheGroup, CacheManager, PagePool, RequestCache,
                      group_cache_needs, hash_page, prefix_caching_possible)
from .storage import CacheStorage, bytes_per_page

__all__ = ["CacheExhausted", "CacheGroup", "CacheManager", "PagePool", "RequestCache",
           "group_cache_needs", "hash_page", "prefix_caching_possible", "CacheStorage", "bytes_per_page"]
