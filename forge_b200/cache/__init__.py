from .manager import CacheManager, GroupSpec
from .pages import CacheError, OutOfPages, PagePool
from .storage import CacheStorage, LayerCache, bytes_per_page, group_name, plan_groups

__all__ = ["CacheManager", "GroupSpec", "CacheError", "OutOfPages", "PagePool", "CacheStorage", "LayerCache",
           "bytes_per_page", "group_name", "plan_groups"]
