from tokasaurus_b200.cache.pages import NoSpaceError, PageAllocator  # noqa: F401
from tokasaurus_b200.cache.slots import NoSlotError, StateSlotAllocator  # noqa: F401
from tokasaurus_b200.cache.manager import (  # noqa: F401
    CacheGroup,
    CacheManager,
    PagedLayerCache,
    RequestCache,
    StateLayerCache,
)
