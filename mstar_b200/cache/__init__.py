"""Paged key/value cache and per-request state slots."""
from .manager import BatchIndex, CacheExhausted, CacheManager, GroupConfig, NoFreeSlot, SequenceTooLong

__all__ = ["BatchIndex", "CacheExhausted", "CacheManager", "GroupConfig", "NoFreeSlot",
           "SequenceTooLong"]
