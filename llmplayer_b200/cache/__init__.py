"""Slots, pages and per-sequence state."""
from .pages import PAGE_SIZE, FreeList, PageMap
from .sequence_cache import KVRequest, KVView, SequenceCache, StateRequest, StateView

__all__ = ["PAGE_SIZE", "FreeList", "PageMap", "KVRequest", "KVView", "SequenceCache", "StateRequest", "StateView"]
