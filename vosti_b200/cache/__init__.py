from .manager import RELEASED, CacheGroup, CacheManager, LayerCache, OutOfSlots, Residency
from .pages import OutOfPages, PageAccountingError, PagePool, chain_hash

__all__ = ["RELEASED", "CacheGroup", "CacheManager", "LayerCache", "OutOfSlots", "Residency",
           "OutOfPages", "PageAccountingError", "PagePool", "chain_hash"]
