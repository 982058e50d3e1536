from .manager import AllocStatus, CacheError, CacheManager, GroupLayout, OutOfPages, PagePool, RequestPages, pool_sizes, tokens_that_fit
from .store import PagedStore

__all__ = ["AllocStatus", "CacheError", "CacheManager", "GroupLayout", "OutOfPages", "PagePool",
           "RequestPages", "PagedStore", "pool_sizes", "tokens_that_fit"]
