"""Paged key/value cache with groups, block tables and per-request state slots."""
from .block_pool import BlockPool
from .manager import FREED, BlockTable, CacheManager, GroupSpec, RequestCache, blocks_for
from .state_slots import StateSlots

__all__ = ["BlockPool", "FREED", "BlockTable", "CacheManager", "GroupSpec", "RequestCache", "blocks_for", "StateSlots"]
