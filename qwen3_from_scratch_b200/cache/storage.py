"""Device memory behind the cache manager: the pages of every group and the state slots.

One group = one tensor ``[caches, 2, num_pages, kv_heads, page_size, head_dim]`` in the compute
dtype (index 0 of the second axis holds keys, 1 values).  A page's keys of one head are
contiguous (page_size x head_dim), which is the unit the attention kernels fetch.
State caches are ``[max_seqs, *shape]`` tensors, zero when a slot is handed to a new request.
"""

from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch

from .manager import CacheLayout


class CacheStorage:
    def __init__(self, layout: CacheLayout, page_size: int, max_seqs: int, device, dtype: torch.dtype):
        self.layout, self.page_size, self.dtype = layout, page_size, dtype
        self.group_pages: List[torch.Tensor] = []
        self._where: Dict[int, Tuple[int, int]] = {}
        for g, group in enumerate(layout.groups):
            spec = group.spec
            self.group_pages.append(torch.zeros(
                len(group.cache_ids), 2, group.num_pages, spec.num_kv_heads, page_size, spec.head_dim,
                dtype=dtype, device=device))
            for i, cache_id in enumerate(group.cache_ids):
                self._where[cache_id] = (g, i)
        self.states: Dict[int, torch.Tensor] = {}
        for cache_id, spec in layout.states.items():
            sdtype = torch.float32 if spec.dtype == "float32" else dtype
            self.states[cache_id] = torch.zeros(max_seqs, *spec.shape, dtype=sdtype, device=device)

    def group_of(self, cache_id: int) -> int:
        return self._where[cache_id][0]

    def kv_pages(self, cache_id: int) -> Tuple[torch.Tensor, torch.Tensor]:
        g, i = self._where[cache_id]
        return self.group_pages[g][i, 0], self.group_pages[g][i, 1]

    def clear_slot(self, slot: int) -> None:
        for state in self.states.values():
            state[slot].zero_()

    def poison(self, freed: Sequence[Tuple[int, int]]) -> None:
        """Fills pages that were given back with NaN, so that a read past a request's keys shows."""
        by_group: Dict[int, List[int]] = {}
        for g, page in freed:
            by_group.setdefault(g, []).append(page)
        for g, pages in by_group.items():
            idx = torch.tensor(sorted(set(pages)), device=self.group_pages[g].device)
            self.group_pages[g][:, :, idx] = float("nan")

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.group_pages) + sum(
            t.numel() * t.element_size() for t in self.states.values())
