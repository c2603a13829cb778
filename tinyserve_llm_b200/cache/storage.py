"""
Device side of the cache: one key pool and one value pool per layer group, laid out
[page][entry][kv head][token in page][head_dim] so that the keys of one (page, entry, head) are one
contiguous tile, and a pool of fixed-size per-request state slots.

tinyserve-llm keeps one pool pair [blocks, layers, block_size, kv_heads, head_dim]
(kvcache/storage.py:25-27); page-first order is kept (a page's keys for all layers are contiguous,
so copy-on-write is one kernel), heads come before tokens so that the attention kernels read whole
tiles.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from tinyserve_llm_b200.cache.manager import CacheLayout


@dataclass
class EntryBinding:
    """What a mixer's kernels need to address one cache entry in one step."""

    k_pool: torch.Tensor
    v_pool: torch.Tensor
    page_stride: int          # elements between consecutive pages
    entry_offset: int         # elements from a page's start to this entry
    page_tokens: int
    num_pages: int
    block_table: torch.Tensor | None = None     # int32 [sequences, table_width] on the device, set per step
    table_width: int = 0
    writes: bool = True
    group: int = 0
    state: torch.Tensor | None = None            # uint8 [slots, bytes of this entry's state]
    state_slots: torch.Tensor | None = None      # int32 [sequences] on the device, set per step


class DeviceCacheStorage:
    def __init__(self, layout: CacheLayout, num_pages: int | list[int], dtype: torch.dtype, device: torch.device,
                 ops, num_state_slots: int = 0) -> None:
        self.layout = layout
        self.ops = ops
        self.dtype = dtype
        self.device = torch.device(device)
        counts = [num_pages] * len(layout.groups) if isinstance(num_pages, int) else list(num_pages)
        self.num_pages = counts
        self.k_pools, self.v_pools = [], []
        for group, pages in zip(layout.groups, counts):
            shape = (pages, len(group.entries), group.num_kv_heads, layout.page_tokens, group.head_dim)
            self.k_pools.append(torch.zeros(shape, dtype=dtype, device=self.device))
            self.v_pools.append(torch.zeros(shape, dtype=dtype, device=self.device))
        self.state = None
        if layout.state_bytes:
            self.state = torch.zeros((max(num_state_slots, 1), layout.state_bytes), dtype=torch.uint8, device=self.device)

    @staticmethod
    def bytes_per_page(layout: CacheLayout, dtype: torch.dtype) -> list[int]:
        """Keys and values of one page across the entries of each group."""
        return [2 * len(g.entries) * g.num_kv_heads * layout.page_tokens * g.head_dim * dtype.itemsize
                for g in layout.groups]

    def entry_binding(self, entry: int) -> EntryBinding | None:
        """Geometry of a cache entry (block table and state rows are filled in per step)."""
        try:
            g, index = self.layout.group_of(entry)
        except KeyError:
            binding = None
        else:
            group = self.layout.groups[g]
            per_entry = group.num_kv_heads * self.layout.page_tokens * group.head_dim
            binding = EntryBinding(self.k_pools[g], self.v_pools[g], per_entry * len(group.entries), per_entry * index,
                                   self.layout.page_tokens, self.num_pages[g], group=g)
        offset = self.layout.state_offsets[entry] if entry < len(self.layout.state_offsets) else -1
        if offset >= 0:
            sizes = self.layout.state_sizes
            size = sizes[entry] if entry < len(sizes) and sizes[entry] else self.layout.state_bytes - offset
            view = self.state[:, offset:offset + size]
            if binding is None:
                binding = EntryBinding(None, None, 0, 0, self.layout.page_tokens, 0, group=-1)
            binding.state = view
        return binding

    # ------------------------------------------------------------------ what the manager asks for
    def copy_slots(self, group: int, src_page: int, dst_page: int, num_slots: int) -> None:
        self.ops.copy_page_slots(self.k_pools[group], self.v_pools[group], src_page, dst_page, num_slots)

    def copy_state(self, src_slot: int, dst_slot: int) -> None:
        self.state[dst_slot].copy_(self.state[src_slot])

    def clear_state(self, slot: int) -> None:
        self.state[slot].zero_()
