from dispec_b200.cache.manager import (CacheGroupSpec, CacheManager, CacheTensor, OutOfSlotsError,
                                        key_value_tensors)
from dispec_b200.cache.pages import OutOfBlocksError, OutOfPagesError, PagePool

__all__ = ["CacheGroupSpec", "CacheManager", "CacheTensor", "key_value_tensors", "OutOfSlotsError", "OutOfBlocksError",
           "OutOfPagesError", "PagePool"]
