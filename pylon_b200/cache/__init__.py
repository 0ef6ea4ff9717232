from pylon_b200.cache.manager import CacheError, CacheGroup, CacheManager, OutOfPages, PagePool, RequestCache  # noqa: F401
