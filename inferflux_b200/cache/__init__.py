"""Paged key/value cache, block tables and per-request state slots."""
from .manager import CacheManager, CacheView, OutOfSlots
from .pages import OutOfPages, PageAccountingError, PageAllocator

__all__ = ["CacheManager", "CacheView", "OutOfSlots", "OutOfPages", "PageAccountingError", "PageAllocator"]
