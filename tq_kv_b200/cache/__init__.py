"""The cache: slots per sequence, paged key/value storage per group of layers,
fixed-size state per sequence."""
from .pool import CacheError, GroupPages, IndexPool, SlotBook
from .storage import PAGE_TOKENS, KVGroup, KVLayerView, KVRequest, SequenceCache, StateRequest, ring_pages_for

__all__ = ["CacheError", "GroupPages", "IndexPool", "KVGroup", "KVLayerView", "KVRequest", "PAGE_TOKENS",
           "SequenceCache", "SlotBook", "StateRequest", "ring_pages_for"]
