from tinyserve_llm_b200.cache.manager import (
    AdmissionCost,
    CacheLayout,
    CacheManager,
    CacheStats,
    GroupLayout,
    NullStorage,
    plan_layout,
)
from tinyserve_llm_b200.cache.pool import CacheFull, PagePool
from tinyserve_llm_b200.cache.prefix_index import CachedPage, PrefixIndex, Reuse, shared_run
from tinyserve_llm_b200.cache.storage import DeviceCacheStorage, EntryBinding

__all__ = ["AdmissionCost", "CacheFull", "CacheLayout", "CacheManager", "CacheStats", "CachedPage", "DeviceCacheStorage",
           "EntryBinding", "GroupLayout", "NullStorage", "PagePool", "PrefixIndex", "Reuse", "plan_layout", "shared_run"]
