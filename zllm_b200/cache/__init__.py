from .manager import CacheManager, KVGroup, KVLayerView, NO_PAGE, PagePool, StateView

__all__ = ["CacheManager", "KVGroup", "KVLayerView", "NO_PAGE", "PagePool", "StateView"]
