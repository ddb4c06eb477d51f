from .pages import PagePool, SlotTable
from .kv import CacheGroup, KVCache, SequenceRecord

__all__ = ["PagePool", "SlotTable", "CacheGroup", "KVCache", "SequenceRecord"]
