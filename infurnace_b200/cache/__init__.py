"""Paged key/value cache with per-request block tables, in groups, and state slots."""
from .block_pool import BlockPool  # noqa: F401
from .manager import CacheManager, CacheLayout, KVGroup, StateGroup, RELEASED  # noqa: F401
