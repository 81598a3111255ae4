from .allocator import NumberPool, OutOfPagesError, OutOfSlotsError
from .kv_cache import DEFAULT_PAGE_SIZE, Cache, LayerCache, PagedGroup, StateGroup, register_cache_kind
