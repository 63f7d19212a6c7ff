"""Paged key/value cache and per-request state slots."""
from .manager import (CacheBinding, CacheError, CacheManager, CacheStorage, OutOfPages, OutOfSlots, PageAllocator,
                      PagedGroup, RequestCache, StateGroup)
