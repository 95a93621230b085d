"""The cache manager: paged keys and values in groups, block tables, request slots, fixed-size per-request state."""
from .manager import CacheGroup, CacheManager
from .pages import OutOfPages, PageError, PagePool

__all__ = ["CacheGroup", "CacheManager", "OutOfPages", "PageError", "PagePool"]
