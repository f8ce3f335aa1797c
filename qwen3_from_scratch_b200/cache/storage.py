"""Device memory behind the cache manager: the pages of every group and the state slots.

A group's caches declare named planes (``PagedCacheSpec.planes``; ``k`` and ``v`` for attention).  Every
plane of a group is one tensor ``[caches, num_pages, heads, page_size, width]`` in the plane's dtype, so
that one cache's pages of one plane are a contiguous ``[num_pages, heads, page_size, width]`` array and a
page's vectors of one head are contiguous (page_size x width), which is the unit the attention kernels
fetch.  State caches are ``[max_seqs, *shape]`` tensors, zero when a slot is handed to a new request.
"""

from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch

from .manager import CacheLayout


class CacheStorage:
    def __init__(self, layout: CacheLayout, page_size: int, max_seqs: int, device, dtype: torch.dtype):
        self.layout, self.page_size, self.dtype = layout, page_size, dtype
        self.group_planes: List[Dict[str, torch.Tensor]] = []  # per group: plane name -> its tensor
        self._where: Dict[int, Tuple[int, int]] = {}
        for g, group in enumerate(layout.groups):
            planes = {}
            for plane in group.spec.planes:
                pdtype = torch.float32 if plane.dtype == "float32" else dtype
                planes[plane.name] = torch.zeros(len(group.cache_ids), group.num_pages, plane.heads, page_size,
                                                 plane.width, dtype=pdtype, device=device)
            self.group_planes.append(planes)
            for i, cache_id in enumerate(group.cache_ids):
                self._where[cache_id] = (g, i)
        self.states: Dict[int, torch.Tensor] = {}
        for cache_id, spec in layout.states.items():
            sdtype = torch.float32 if spec.dtype == "float32" else dtype
            self.states[cache_id] = torch.zeros(max_seqs, *spec.shape, dtype=sdtype, device=device)

    def group_of(self, cache_id: int) -> int:
        return self._where[cache_id][0]

    def planes(self, cache_id: int) -> Dict[str, torch.Tensor]:
        """Plane name -> ``[num_pages, heads, page_size, width]`` of one cache."""
        g, i = self._where[cache_id]
        return {name: t[i] for name, t in self.group_planes[g].items()}

    def kv_pages(self, cache_id: int) -> Tuple[torch.Tensor, torch.Tensor]:
        planes = self.planes(cache_id)
        return planes["k"], planes["v"]

    def clear_slot(self, slot: int) -> None:
        for state in self.states.values():
            state[slot].zero_()

    def poison(self, freed: Sequence[Tuple[int, int]]) -> None:
        """Fills pages that were given back with NaN, so that a read past a request's keys shows."""
        by_group: Dict[int, List[int]] = {}
        for g, page in freed:
            by_group.setdefault(g, []).append(page)
        for g, pages in by_group.items():
            for t in self.group_planes[g].values():
                idx = torch.tensor(sorted(set(pages)), device=t.device)
                t[:, idx] = float("nan")

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for planes in self.group_planes for t in planes.values()) + sum(
            t.numel() * t.element_size() for t in self.states.values())
