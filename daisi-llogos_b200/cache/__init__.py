"""Slots, pages and fixed-size state of live sequences."""
from .slots import CacheError, FreeList, SlotTable
from .store import PAGE, KvGroup, KvView, SequenceCache, StateView, pages_for

__all__ = ["CacheError", "FreeList", "SlotTable", "PAGE", "KvGroup", "KvView", "SequenceCache", "StateView",
           "pages_for"]
