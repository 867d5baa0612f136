from .manager import CacheManager, LayerCacheView, OutOfPages, OutOfSlots
from .page_pool import PageError, PagePool
from .spec import FixedStateSpec, PagedKVSpec
