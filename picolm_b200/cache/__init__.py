from .allocator import CacheFull, IndexPool
from .sequence_cache import (PAGE_TOKENS, KVGroup, KVLayerCache, SequenceCache, StateLayerCache, pages_for)
from .spec import CacheSpec

__all__ = ["CacheFull", "IndexPool", "PAGE_TOKENS", "KVGroup", "KVLayerCache", "SequenceCache",
           "StateLayerCache", "pages_for", "CacheSpec"]
