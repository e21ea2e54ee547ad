"""The cache: slots per sequence, paged keys and values per group, fixed-size state."""
from .layout import CacheLayout, Group, KVNeed, StateNeed
from .pages import PAGE_SIZE, CacheError, CacheFull, IdPool, SlotBook
from .device import DeviceCache, KVView

__all__ = ["CacheLayout", "Group", "KVNeed", "StateNeed", "PAGE_SIZE", "CacheError", "CacheFull",
           "IdPool", "SlotBook", "DeviceCache", "KVView"]
