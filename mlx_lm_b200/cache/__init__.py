from .manager import CacheManager, KVGroup, NoFreeSlot, OutOfPages, PagePool, RequestCache, StateGroup

__all__ = ["CacheManager", "KVGroup", "NoFreeSlot", "OutOfPages", "PagePool", "RequestCache", "StateGroup"]
