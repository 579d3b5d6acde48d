from .manager import CacheError, CacheManager, GroupSpec, PagePool, SequenceCache

__all__ = ["CacheError", "CacheManager", "GroupSpec", "PagePool", "SequenceCache"]
