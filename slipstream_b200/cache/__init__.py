from .manager import AllocStatus, CacheError, CacheManager, GroupLayout, OutOfPages, PagePool, RequestPages
from .store import PagedStore

__all__ = ["AllocStatus", "CacheError", "CacheManager", "GroupLayout", "OutOfPages", "PagePool",
           "RequestPages", "PagedStore"]
