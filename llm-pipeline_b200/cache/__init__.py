"""Paged key/value cache, block tables, and per-request state slots."""

from .manager import CacheError, CacheGroup, CacheManager, PagePool
from .spec import KVPagesSpec, PagesSpec, StateSpec, TokenPagesSpec

__all__ = ["CacheError", "CacheGroup", "CacheManager", "PagePool", "KVPagesSpec", "PagesSpec", "StateSpec", "TokenPagesSpec"]
