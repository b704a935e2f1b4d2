from .manager import (CacheError, CacheManager, GroupInfo, LayerCache, OutOfPages, PageTable,
                      host_library)

__all__ = ["CacheError", "CacheManager", "GroupInfo", "LayerCache", "OutOfPages", "PageTable",
           "host_library"]
