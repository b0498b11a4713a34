"""The cache manager: pages, block tables, groups of layers, state slots."""
from .manager import CacheManager, CacheView, NoFreeSlot
from .pages import OutOfPages, PagePool

__all__ = ["CacheManager", "CacheView", "NoFreeSlot", "OutOfPages", "PagePool"]
