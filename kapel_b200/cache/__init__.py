"""Paged keys and values by layer group, block tables, and slots of per-request state."""
from .manager import CacheGroup, CacheManager, CacheNeeds, GroupPlan, PagedKV, Plan, StateSpec
from .pages import CacheFull, PagePool
