from .manager import CacheManager, LayerCacheView, OutOfPages, OutOfSlots, PageError
from .spec import FixedStateSpec, PagedKVSpec
