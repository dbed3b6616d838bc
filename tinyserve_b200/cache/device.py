"""Device memory of the cache: one tensor per group, and the state-slot tensors.

Layout of a group: [entry, 2 (keys, values), page, kv_head, slot, head_dim], so the
share of one KV head in one page is one contiguous run of page_size * head_dim
elements.  tinyserve keeps [2, page, slot, kv_head, head_dim] per layer
(serve.py:1791-1796)."""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class CacheEntry:
    group: int
    k: torch.Tensor      # [page, kv_head, slot, head_dim]
    v: torch.Tensor


class DeviceCache:
    def __init__(self, model, num_pages, page_size: int, num_slots: int, dtype, device):
        counts = [num_pages] * len(model.cache_groups) if isinstance(num_pages, int) else list(num_pages)
        self.page_size = page_size
        self.pools = []
        for spec, entries, pages in zip(model.cache_groups, model.group_sizes, counts):
            self.pools.append(torch.zeros(entries, 2, pages, spec.num_kv_heads, page_size,
                                          spec.head_dim, dtype=dtype, device=device))
        self.entries = [CacheEntry(info.group, self.pools[info.group][info.index_in_group, 0],
                                   self.pools[info.group][info.index_in_group, 1])
                        for info in model.cache_entries]
        self.states = [torch.zeros((num_slots,) + tuple(s.shape), dtype=getattr(torch, s.dtype),
                                   device=device) for s in model.state_entries]

    @staticmethod
    def bytes_per_page(model, page_size: int, element_size: int) -> list:
        return [2 * n * spec.num_kv_heads * page_size * spec.head_dim * element_size
                for spec, n in zip(model.cache_groups, model.group_sizes)]

    def zero_state(self, slot: int) -> None:
        for s in self.states:
            s[slot].zero_()
