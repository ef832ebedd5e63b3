"""Cache: page pools, block tables, state slots and their device arrays."""
from .manager import (CacheError, CacheManager, GroupLayout, PagePool, RequestCache,
                      first_needed_block, pages_for)
from .storage import CachePlan, CacheStorage, FixedStateView, PagedKVView, plan_cache

__all__ = ["CacheError", "CacheManager", "GroupLayout", "PagePool", "RequestCache",
           "first_needed_block", "pages_for", "CachePlan", "CacheStorage", "FixedStateView",
           "PagedKVView", "plan_cache"]
