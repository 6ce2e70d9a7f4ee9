from .page_table import CacheError, GroupGeometry, OutOfPages, OutOfSlots, PageTable
from .pools import CachePools, PagedView, StateView

__all__ = ["CacheError", "GroupGeometry", "OutOfPages", "OutOfSlots", "PageTable", "CachePools", "PagedView",
           "StateView"]
