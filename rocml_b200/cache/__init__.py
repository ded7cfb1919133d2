"""The cache: slots, pages, groups of layers with storage of their own, per-sequence state."""
from .pages import FreeList
from .requirements import KVRequirement, StateRequirement
from .sequence_cache import PAGE, CacheView, KVGroup, SequenceCache, StateGroup, pages_for

__all__ = ["FreeList", "KVRequirement", "StateRequirement", "PAGE", "CacheView", "KVGroup",
           "SequenceCache", "StateGroup", "pages_for"]
