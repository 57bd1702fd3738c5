"""The paged cache, the slots and the per-sequence state."""
from .pages import PAGE, CacheFull, PagePool, SlotPool, pages_for
from .cache import Cache, KVGroup, KVSpec, StateSpec

__all__ = ["PAGE", "CacheFull", "PagePool", "SlotPool", "pages_for", "Cache", "KVGroup",
           "KVSpec", "StateSpec"]
