from .pages import PAGE_TOKENS, CacheFull, PagePool, SequenceSlots, SlotError, pages_for
from .store import BundleRequest, Cache, CacheRequest, KVRequest, KVView, StateRequest

__all__ = ["PAGE_TOKENS", "CacheFull", "PagePool", "SequenceSlots", "SlotError", "pages_for",
           "BundleRequest", "Cache", "CacheRequest", "KVRequest", "KVView", "StateRequest"]
