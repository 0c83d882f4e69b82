from .manager import CacheError, CacheGroup, CacheManager, PagePool, PagedKVView, RequestCache  # noqa: F401
