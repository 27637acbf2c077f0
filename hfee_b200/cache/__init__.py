from .needs import FixedState, PagedKV
from .pages import OutOfPages, PagePool
from .manager import CacheManager, CacheView

__all__ = ["FixedState", "PagedKV", "OutOfPages", "PagePool", "CacheManager", "CacheView"]
