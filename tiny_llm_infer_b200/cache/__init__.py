from .manager import CacheError, CacheManager, LayerCacheView, OutOfPages, OutOfSlots, PagePool
