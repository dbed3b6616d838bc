"""Device memory of the cache: per group one tensor for each thing its mixers keep per token,
and the state-slot tensors.

Layout of a cache tensor: [entry, page, head, slot, width], so the share of one head in one page
is one contiguous run of page_size * width elements (attention: "k" and "v" of kv_heads heads of
head_dim; a mixer may keep other tensors, see ``parts.CacheSpec``).  tinyserve keeps
[2, page, slot, kv_head, head_dim] per layer (serve.py:1791-1796)."""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class CacheEntry:
    group: int
    tensors: dict        # name -> [page, head, slot, width]

    @property
    def k(self) -> torch.Tensor:
        return self.tensors["k"]

    @property
    def v(self) -> torch.Tensor:
        return self.tensors["v"]


class DeviceCache:
    def __init__(self, model, num_pages, page_size: int, num_slots: int, dtype, device):
        counts = [num_pages] * len(model.cache_groups) if isinstance(num_pages, int) else list(num_pages)
        self.page_size = page_size
        self.pools = []          # per group: {tensor name: [entry, page, head, slot, width]}
        for spec, entries, pages in zip(model.cache_groups, model.group_sizes, counts):
            self.pools.append({t.name: torch.zeros(entries, pages, t.heads, page_size, t.width,
                                                   dtype=dtype, device=device) for t in spec.tensors})
        self.entries = [CacheEntry(info.group, {name: pool[info.index_in_group]
                                                for name, pool in self.pools[info.group].items()})
                        for info in model.cache_entries]
        self.states = [torch.zeros((num_slots,) + tuple(s.shape), dtype=getattr(torch, s.dtype),
                                   device=device) for s in model.state_entries]

    @staticmethod
    def bytes_per_page(model, page_size: int, element_size: int) -> list:
        return [n * spec.elements_per_token() * page_size * element_size
                for spec, n in zip(model.cache_groups, model.group_sizes)]

    def zero_state(self, slots) -> None:
        """Zero the state of the given slots (a request that starts there finds no trace of the
        one before)."""
        if not self.states or not len(slots):
            return
        index = torch.as_tensor(slots, dtype=torch.long, device=self.states[0].device)
        for s in self.states:
            s.index_fill_(0, index, 0)
