"""Slots, paged keys/values per layer group, and fixed-size per-sequence state."""
from .allocators import CacheError, CacheFull, IndexPool
from .cache import (PAGE_TOKENS, Cache, CacheRequest, KVGroup, KVLayerView, KVRequest, StateGroup,
                    StateLayerView, StateRequest)

__all__ = ["CacheError", "CacheFull", "IndexPool", "PAGE_TOKENS", "Cache", "CacheRequest", "KVGroup",
           "KVLayerView", "KVRequest", "StateGroup", "StateLayerView", "StateRequest"]
