"""Paged keys and values, block tables and per-request state slots."""
from .pages import UNMAPPED, CacheManager, KvGroup, KvNeed, OutOfPages, PagePool, StateNeed, StateSlots

__all__ = ["UNMAPPED", "CacheManager", "KvGroup", "KvNeed", "OutOfPages", "PagePool", "StateNeed", "StateSlots"]
