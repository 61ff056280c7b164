"""The cache: slots per sequence, paged key/value storage per group of layers,
fixed-size state per sequence."""
from .pool import CacheError, PageGroup, SlotBook, StepError, StepLayout
from .storage import PAGE_TOKENS, KVGroup, KVLayerView, KVRequest, SequenceCache, StateRequest, ring_pages_for

__all__ = ["CacheError", "KVGroup", "KVLayerView", "KVRequest", "PAGE_TOKENS", "PageGroup", "SequenceCache",
           "SlotBook", "StateRequest", "StepError", "StepLayout", "ring_pages_for"]
