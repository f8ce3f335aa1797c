"""Cache manager: who holds which page and which state slot.  Host side only, no device code.

Keys and values live in pages of ``page_size`` tokens.  Caches (one per entry of the model's
run order that keeps keys/values) with the same needs form a *group*: the same planes (for attention:
keys and values of so many heads of such a size) and the same window.  A group has a page pool of its own, and every request has one block table
per group: logical page i of the request -> page id, shared by all caches of the group (page
p addresses the same slot in each of them, as in the reference's one tensor for all layers,
inference/kv_cache/paged_cache.py:21-33).

Pages are taken incrementally as a request grows (the reference's ``allocate``/``can_allocate``,
inference/block_manager.py:85-106) and given back
  * when the request ends or is preempted (``close``), and
  * in a group with a window, as soon as every position of a page is older than any
    later query can see (``advance``); its table entry becomes -1.
A page given back is handed out again at once (LIFO), so tests see reuse quickly.

Beside the pages there are ``max_seqs`` slots for state of fixed size; a request holds one
slot from ``open`` to ``close`` whether or not the model has such state.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from ..parts.base import PagedCacheSpec, StateSpec


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    pass


class OutOfSlots(CacheError):
    pass


@dataclass
class PageGroup:
    """Caches that share page ids: same planes and window."""

    spec: PagedCacheSpec
    cache_ids: List[int]
    num_pages: int = 0


@dataclass
class CacheLayout:
    """Which cache ids exist, grouped by need.  Built from the model (see ``layout_of``)."""

    groups: List[PageGroup] = field(default_factory=list)
    states: Dict[int, StateSpec] = field(default_factory=dict)

    def group_of(self, cache_id: int) -> int:
        for g, group in enumerate(self.groups):
            if cache_id in group.cache_ids:
                return g
        raise KeyError(f"cache {cache_id} holds no pages")


def layout_of(cache_specs: Dict[int, object]) -> CacheLayout:
    """``cache_specs``: cache id -> PagedCacheSpec | StateSpec | None (what each mixer asked for)."""
    layout = CacheLayout()
    by_spec: Dict[PagedCacheSpec, PageGroup] = {}
    for cache_id in sorted(cache_specs):
        spec = cache_specs[cache_id]
        if spec is None:
            continue
        if isinstance(spec, StateSpec):
            layout.states[cache_id] = spec
        elif isinstance(spec, PagedCacheSpec):
            names = [p.name for p in spec.planes]
            if not names or len(set(names)) != len(names):
                raise ValueError(f"cache {cache_id}: a paged cache needs planes with distinct names, got {names}")
            if spec not in by_spec:
                by_spec[spec] = PageGroup(spec, [])
                layout.groups.append(by_spec[spec])
            by_spec[spec].cache_ids.append(cache_id)
        else:
            raise TypeError(f"cache {cache_id}: unknown cache need {spec!r}")
    return layout


class _Pool:
    """Free list of one group, with ownership kept for the accounting checks."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self.free: List[int] = list(range(num_pages - 1, -1, -1))  # pop() hands out 0, 1, 2, ...
        self.owner: List[Optional[Hashable]] = [None] * num_pages

    def take(self, owner: Hashable) -> int:
        page = self.free.pop()
        if self.owner[page] is not None:
            raise CacheError(f"page {page} handed out while held by {self.owner[page]!r}")
        self.owner[page] = owner
        return page

    def give_back(self, page: int, owner: Hashable) -> None:
        if not 0 <= page < self.num_pages:
            raise CacheError(f"page {page} is outside the pool of {self.num_pages}")
        if self.owner[page] is None:
            raise CacheError(f"page {page} freed twice")
        if self.owner[page] != owner:
            raise CacheError(f"page {page} freed by {owner!r} but held by {self.owner[page]!r}")
        self.owner[page] = None
        self.free.append(page)


@dataclass
class _Request:
    slot: int
    length: int = 0  # tokens whose keys/values are in the cache
    tables: List[List[int]] = field(default_factory=list)  # per group: logical page -> page id or -1
    first_live: List[int] = field(default_factory=list)  # per group: first logical page not given back
    version: int = 0  # unique over the manager's life; renewed whenever a block table of the request changes


class CacheManager:
    def __init__(self, layout: CacheLayout, page_size: int, num_pages: int, max_seqs: int,
                 pages_per_group: Optional[Sequence[int]] = None):
        """``num_pages`` pages in every group's pool (or ``pages_per_group`` to size them apart)."""
        if page_size <= 0 or max_seqs <= 0:
            raise ValueError("page_size and max_seqs must be positive")
        self.layout = layout
        self.page_size = int(page_size)
        counts = list(pages_per_group) if pages_per_group is not None else [num_pages] * len(layout.groups)
        if len(counts) != len(layout.groups) or any(c <= 0 for c in counts):
            raise ValueError(f"need a positive page count for each of the {len(layout.groups)} groups")
        for group, count in zip(layout.groups, counts):
            group.num_pages = int(count)
        self._pools = [_Pool(int(c)) for c in counts]
        self.max_seqs = int(max_seqs)
        self._free_slots: List[int] = list(range(self.max_seqs - 1, -1, -1))
        self._requests: Dict[Hashable, _Request] = {}
        self.freed_log: Optional[List[Tuple[int, int]]] = None  # (group, page) of pages given back, if tracked
        self.on_open = None  # called with the slot when a request is opened (the storage clears its state)

    # ------------------------------------------------------------------ queries
    def __contains__(self, req: Hashable) -> bool:
        return req in self._requests

    def live_requests(self) -> List[Hashable]:
        return list(self._requests)

    def length(self, req: Hashable) -> int:
        return self._requests[req].length

    def slot(self, req: Hashable) -> int:
        return self._requests[req].slot

    def table(self, group: int, req: Hashable) -> List[int]:
        return self._requests[req].tables[group]

    def row_state(self, req: Hashable):
        """(tokens computed, state slot, table version) of a request in one lookup."""
        r = self._requests[req]
        return r.length, r.slot, r.version

    def table_version(self, req: Hashable) -> int:
        """A number that is renewed whenever one of the request's block tables changes, and that no
        other request, nor a later request of the same name, ever has."""
        return self._requests[req].version

    def _new_version(self) -> int:
        self._versions = getattr(self, "_versions", 0) + 1
        return self._versions

    def free_pages(self, group: int = 0) -> int:
        return len(self._pools[group].free)

    def free_slots(self) -> int:
        return len(self._free_slots)

    def capacity_tokens(self) -> int:
        """Tokens one request could hold if it had the cache to itself."""
        if not self._pools:
            return 1 << 62
        return min(p.num_pages for p in self._pools) * self.page_size

    def _first_needed_page(self, group: int, length: int) -> int:
        """First logical page a query at position >= ``length`` can still read."""
        window = self.layout.groups[group].spec.window
        if window is None:
            return 0
        return max(0, length - window + 1) // self.page_size

    def pages_needed(self, req: Hashable, new_length: int) -> List[int]:
        """Per group, how many more pages ``req`` needs to hold ``new_length`` tokens."""
        r = self._requests[req]
        last = (new_length - 1) // self.page_size if new_length > 0 else -1
        need = []
        for g in range(len(self._pools)):
            have = len(r.tables[g])
            need.append(max(0, last + 1 - have))
        return need

    def can_reserve(self, req: Hashable, new_length: int) -> bool:
        return all(n <= len(p.free) for n, p in zip(self.pages_needed(req, new_length), self._pools))

    # ------------------------------------------------------------------ life of a request
    def open(self, req: Hashable) -> int:
        """Gives ``req`` a state slot and empty block tables; returns the slot."""
        if req in self._requests:
            raise CacheError(f"request {req!r} is already open")
        if not self._free_slots:
            raise OutOfSlots(f"all {self.max_seqs} request slots are in use")
        slot = self._free_slots.pop()
        n = len(self._pools)
        self._requests[req] = _Request(slot=slot, tables=[[] for _ in range(n)], first_live=[0] * n,
                                       version=self._new_version())
        if self.on_open is not None:
            self.on_open(slot)
        return slot

    def reserve(self, req: Hashable, new_length: int) -> None:
        """Pages for positions < ``new_length`` in every group, or OutOfPages and nothing taken."""
        r = self._requests[req]
        if new_length < r.length:
            raise CacheError(f"request {req!r} holds {r.length} tokens, cannot reserve for {new_length}")
        need = self.pages_needed(req, new_length)
        for g, (n, pool) in enumerate(zip(need, self._pools)):
            if n > len(pool.free):
                raise OutOfPages(
                    f"request {req!r} needs {n} more pages in group {g} for {new_length} tokens, "
                    f"{len(pool.free)} of {pool.num_pages} are free")
        for g, (n, pool) in enumerate(zip(need, self._pools)):
            for _ in range(n):
                r.tables[g].append(pool.take(req))
            if n:
                r.version = self._new_version()

    def advance(self, req: Hashable, new_length: int) -> None:
        """Records that ``req`` now holds ``new_length`` tokens and gives back what windows have passed."""
        r = self._requests[req]
        if new_length < r.length:
            raise CacheError(f"request {req!r} cannot shrink from {r.length} to {new_length}")
        if new_length > 0 and any((new_length - 1) // self.page_size >= len(t) for t in r.tables):
            raise CacheError(f"request {req!r} advanced to {new_length} tokens beyond its reserved pages")
        r.length = new_length
        for g, pool in enumerate(self._pools):
            keep_from = min(self._first_needed_page(g, new_length), len(r.tables[g]))
            for i in range(r.first_live[g], keep_from):
                page = r.tables[g][i]
                if page >= 0:
                    pool.give_back(page, req)
                    r.tables[g][i] = -1
                    r.version = self._new_version()
                    if self.freed_log is not None:
                        self.freed_log.append((g, page))
            r.first_live[g] = max(r.first_live[g], keep_from)

    def close(self, req: Hashable) -> None:
        """Gives back every page and the slot of ``req``."""
        r = self._requests.pop(req, None)
        if r is None:
            raise CacheError(f"request {req!r} is not open (closed twice?)")
        for g, pool in enumerate(self._pools):
            for page in r.tables[g]:
                if page >= 0:
                    pool.give_back(page, req)
                    if self.freed_log is not None:
                        self.freed_log.append((g, page))
        self._free_slots.append(r.slot)

    # ------------------------------------------------------------------ accounting
    def check(self) -> None:
        """Raises if a page is lost, held twice or both free and held; same for slots."""
        for g, pool in enumerate(self._pools):
            held: Dict[int, Hashable] = {}
            for req, r in self._requests.items():
                for page in r.tables[g]:
                    if page < 0:
                        continue
                    if page in held:
                        raise CacheError(f"group {g}: page {page} held by {held[page]!r} and {req!r}")
                    held[page] = req
            free = set(pool.free)
            if len(free) != len(pool.free):
                raise CacheError(f"group {g}: a page is twice in the free list")
            if free & set(held):
                raise CacheError(f"group {g}: pages {sorted(free & set(held))} are both free and held")
            if len(free) + len(held) != pool.num_pages:
                lost = set(range(pool.num_pages)) - free - set(held)
                raise CacheError(f"group {g}: pages {sorted(lost)} are lost")
            for page, req in held.items():
                if pool.owner[page] != req:
                    raise CacheError(f"group {g}: page {page} owner record {pool.owner[page]!r} != {req!r}")
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a state slot is held twice or both free and held")
        if len(slots) + len(self._free_slots) != self.max_seqs:
            raise CacheError("a state slot is lost")
