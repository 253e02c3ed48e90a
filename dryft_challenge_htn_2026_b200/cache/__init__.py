"""Sequence slots, paged key/value storage per group of layers, fixed-size per-sequence state."""
from .cache import Cache, KVGroup, KVView, StateGroup, StateView
from .pool import CacheFull, PagePool, SlotTable
from .requests import KVRequest, StateRequest

__all__ = ["Cache", "KVGroup", "KVView", "StateGroup", "StateView", "CacheFull", "PagePool", "SlotTable", "KVRequest",
           "StateRequest"]
