from dispec_b200.cache.manager import CacheGroupSpec, CacheManager, OutOfSlotsError
from dispec_b200.cache.pages import OutOfBlocksError, OutOfPagesError, PagePool

__all__ = ["CacheGroupSpec", "CacheManager", "OutOfSlotsError", "OutOfBlocksError",
           "OutOfPagesError", "PagePool"]
