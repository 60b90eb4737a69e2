from .allocator import FreeList
from .paged import PAGE, Group, KvRequest, PagedCache, StateRequest, round_up

__all__ = ["FreeList", "PAGE", "Group", "KvRequest", "PagedCache", "StateRequest", "round_up"]
