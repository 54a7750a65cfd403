"""The cache: a slot per sequence, paged keys and values per group of layers, fixed-size state beside it."""
from .book import CacheBook, CacheError, PagePool

__all__ = ["CacheBook", "CacheError", "PagePool", "KVCache", "CacheView", "StateArea", "PAGE_SIZE"]


def __getattr__(name):  # device classes import torch lazily
    if name in ("KVCache", "CacheView", "StateArea", "PAGE_SIZE"):
        from . import kv_cache
        return getattr(kv_cache, name)
    raise AttributeError(name)
