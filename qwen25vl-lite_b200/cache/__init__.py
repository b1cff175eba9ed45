"""Paged cache: page pools, groups of layers, block tables, per-request state slots."""

from .manager import CacheGroup, CacheManager, NoFreeSlot, RequestCache, StopNeeds  # noqa: F401
from .page_pool import OutOfPages, PagePool  # noqa: F401
