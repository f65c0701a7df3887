from .manager import NO_PAGE, CacheGroup, CacheManager, group_entries
from .pages import PageError, PagePool

__all__ = ["NO_PAGE", "CacheGroup", "CacheManager", "group_entries", "PageError", "PagePool"]
