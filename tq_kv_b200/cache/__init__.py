"""The cache: slots per sequence, paged key/value storage per group of layers,
fixed-size state per sequence."""
from .pool import CacheError, GroupPages, IndexPool, SlotBook
from .storage import PAGE_TOKENS, KVGroup, KVLayerView, KVRequest, SequenceCache, StateRequest

__all__ = ["CacheError", "GroupPages", "IndexPool", "KVGroup", "KVLayerView", "KVRequest", "PAGE_TOKENS",
           "SequenceCache", "SlotBook", "StateRequest"]
