from tinyserve_llm_b200.cache.manager import (
    AdmissionCost,
    CacheFull,
    CacheLayout,
    CacheManager,
    CacheStats,
    GroupLayout,
    NullStorage,
    plan_layout,
)
from tinyserve_llm_b200.cache.prefix_tree import PageNode, PrefixMatch, PrefixTree, TokenTrie
from tinyserve_llm_b200.cache.storage import DeviceCacheStorage, EntryBinding

__all__ = ["AdmissionCost", "CacheFull", "CacheLayout", "CacheManager", "CacheStats", "DeviceCacheStorage",
           "EntryBinding", "GroupLayout", "NullStorage", "PageNode", "PrefixMatch", "PrefixTree", "TokenTrie",
           "plan_layout"]
