"""The paged sequence cache."""
from .pool import CacheFull, IndexPool, PoolError
from .sequence_cache import (ContextOverflow, KVGroup, KVView, LayerCacheView, SequenceCache,
                             pages_for)

__all__ = ["CacheFull", "IndexPool", "PoolError", "ContextOverflow", "KVGroup", "KVView",
           "LayerCacheView", "SequenceCache", "pages_for"]
