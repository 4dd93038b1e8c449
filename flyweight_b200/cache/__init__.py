from .manager import (PAGE_SIZE, CacheManager, LayerCache, OutOfPages, OutOfSlots, PageGroup,
                      PagePool)

__all__ = ["PAGE_SIZE", "CacheManager", "LayerCache", "OutOfPages", "OutOfSlots", "PageGroup",
           "PagePool"]
