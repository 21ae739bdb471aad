"""Host-side bookkeeping of the paged cache: which request holds which pages.

The reference keeps one pool whose page ids are valid in every layer
(tinyinfer/engine/block_manager.py:53-67) and gives pages back only when a request ends
(:174-177). Here the cache entries of a model are put into *groups* by what they need (number of
kv heads, head size, window); each group has a pool and each request one block table per group,
so that a group whose mixers read only a window of keys can give pages back as soon as the window
has passed them, while a group that reads all keys keeps them to the end. Beside the pages, a
request holds one *state slot* for per-request state of fixed size.

Nothing here touches device memory; ``CacheStorage`` owns the tensors these page ids index.
Free pages are reused oldest-first and a finished request returns its pages tail-first, as the
reference does (block_manager.py:139-150,174-177).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from ..parts.base import CacheNeed, StateNeed


class CacheExhausted(RuntimeError):
    pass


class PagePool:
    """Page ids 0..n-1 of one group."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        self._free = deque(range(num_pages))
        self._owner: List[Optional[Hashable]] = [None] * num_pages
        self.pages_taken = 0          # counters for stats(): how often pages changed hands
        self.pages_returned = 0

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, owner: Hashable) -> int:
        if not self._free:
            raise CacheExhausted("KV cache exhausted")
        page = self._free.popleft()
        if self._owner[page] is not None:
            raise RuntimeError(f"page {page} was free and owned at once")
        self._owner[page] = owner
        self.pages_taken += 1
        return page

    def give_back(self, page: int, owner: Hashable) -> None:
        if not 0 <= page < self.num_pages:
            raise RuntimeError(f"page {page} does not exist")
        if self._owner[page] is None:
            raise RuntimeError(f"page {page} freed twice")
        if self._owner[page] != owner:
            raise RuntimeError(f"page {page} belongs to {self._owner[page]!r}, not to {owner!r}")
        self._owner[page] = None
        self._free.append(page)
        self.pages_returned += 1

    def owner_of(self, page: int) -> Optional[Hashable]:
        return self._owner[page]

    def free_pages(self) -> List[int]:
        return list(self._free)


@dataclass
class CacheGroup:
    need: CacheNeed
    entries: List[int]                 # cache entries (of the model's run order) in this group
    pool: PagePool


@dataclass
class RequestCache:
    """What one live request holds."""
    request_id: Hashable
    state_slot: int
    length: int = 0                                          # tokens whose keys are stored
    tables: List[List[int]] = field(default_factory=list)    # per group: logical page -> id or -1


def group_cache_needs(needs: Sequence[Tuple[Optional[CacheNeed], Optional[StateNeed]]]):
    """Cache entries with equal page needs share a group. Returns the list of
    (CacheNeed, [entries]) in order of first appearance."""
    groups: List[Tuple[CacheNeed, List[int]]] = []
    for entry, (need, _state) in enumerate(needs):
        if need is None:
            continue
        for g_need, g_entries in groups:
            if g_need == need:
                g_entries.append(entry)
                break
        else:
            groups.append((need, [entry]))
    return groups


class CacheManager:
    def __init__(self, needs, page_size: int, num_pages: int, max_requests: int):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        if max_requests <= 0:
            raise ValueError("max_requests must be positive")
        self.page_size = page_size
        self.max_requests = max_requests
        self.groups = [CacheGroup(need, entries, PagePool(num_pages))
                       for need, entries in group_cache_needs(needs)]
        self.group_of_entry: Dict[int, int] = {e: g for g, grp in enumerate(self.groups)
                                               for e in grp.entries}
        self._free_slots = deque(range(max_requests))
        self._requests: Dict[Hashable, RequestCache] = {}

    # ------------------------------------------------------------------ requests
    def __contains__(self, request_id) -> bool:
        return request_id in self._requests

    def get(self, request_id) -> RequestCache:
        return self._requests[request_id]

    @property
    def live_requests(self) -> List[Hashable]:
        return list(self._requests)

    def can_admit(self) -> bool:
        return bool(self._free_slots)

    def admit(self, request_id) -> RequestCache:
        """Gives the request a state slot and empty block tables."""
        if request_id in self._requests:
            raise RuntimeError(f"request {request_id!r} is already live")
        if not self._free_slots:
            raise CacheExhausted("no free state slot: too many live requests")
        rc = RequestCache(request_id, self._free_slots.popleft(),
                          tables=[[] for _ in self.groups])
        self._requests[request_id] = rc
        return rc

    # ------------------------------------------------------------------ pages
    def _first_needed_page(self, group: CacheGroup, start: int) -> int:
        """Lowest logical page a query at position >= start can read in this group."""
        if group.need.window is None:
            return 0
        return max(0, start - group.need.window + 1) // self.page_size

    def _missing(self, rc: RequestCache, new_length: int) -> List[int]:
        """Per group, how many pages must be taken to hold positions < new_length."""
        want = (new_length + self.page_size - 1) // self.page_size
        return [max(0, want - len(table)) for table in rc.tables]

    def can_extend(self, request_id, new_length: int) -> bool:
        rc = self._requests[request_id]
        return all(m <= g.pool.num_free for m, g in zip(self._missing(rc, new_length), self.groups))

    def extend(self, request_id, new_length: int) -> None:
        """Makes room for positions < new_length in every group, or raises CacheExhausted and
        changes nothing (check, then commit, like block_manager.py:213-237 of the reference)."""
        rc = self._requests[request_id]
        if new_length < rc.length:
            raise ValueError("a request's cache cannot shrink")
        missing = self._missing(rc, new_length)
        for m, g in zip(missing, self.groups):
            if m > g.pool.num_free:
                raise CacheExhausted(f"KV cache exhausted: request {request_id!r} needs {m} more "
                                     f"pages, {g.pool.num_free} are free")
        for m, g, table in zip(missing, self.groups, rc.tables):
            for _ in range(m):
                table.append(g.pool.take(request_id))

    def commit(self, request_id, new_length: int) -> None:
        """Records that keys of positions < new_length are stored, and gives back every page a
        window has passed: no later query of this request can read it."""
        rc = self._requests[request_id]
        if new_length < rc.length:
            raise ValueError("a request's cache cannot shrink")
        for g, table in zip(self.groups, rc.tables):
            if len(table) * self.page_size < new_length:
                raise RuntimeError("commit beyond the pages held")
            if g.need.window is None:
                continue
            for logical in range(min(self._first_needed_page(g, new_length), len(table))):
                if table[logical] >= 0:
                    g.pool.give_back(table[logical], request_id)
                    table[logical] = -1
        rc.length = new_length

    def release(self, request_id) -> None:
        """The request is over: its pages go back tail-first, its state slot is free again."""
        rc = self._requests.pop(request_id)
        for g, table in zip(self.groups, rc.tables):
            for page in reversed(table):
                if page >= 0:
                    g.pool.give_back(page, request_id)
            table.clear()
        self._free_slots.append(rc.state_slot)

    def pages_for(self, length: int) -> int:
        return (length + self.page_size - 1) // self.page_size

    # ------------------------------------------------------------------ inspection
    def stats(self) -> dict:
        return {
            "live_requests": len(self._requests),
            "free_state_slots": len(self._free_slots),
            "groups": [{"window": g.need.window, "entries": len(g.entries),
                        "pages": g.pool.num_pages, "free_pages": g.pool.num_free,
                        "pages_taken": g.pool.pages_taken, "pages_returned": g.pool.pages_returned}
                       for g in self.groups],
        }

    def check_consistency(self) -> None:
        """No page lost, none held twice, none free and held at once; slots likewise."""
        for gi, g in enumerate(self.groups):
            free = g.pool.free_pages()
            if len(set(free)) != len(free):
                raise AssertionError(f"group {gi}: a page is on the free list twice")
            held: Dict[int, Hashable] = {}
            for rid, rc in self._requests.items():
                for page in rc.tables[gi]:
                    if page < 0:
                        continue
                    if page in held:
                        raise AssertionError(f"group {gi}: page {page} held by {held[page]!r} and {rid!r}")
                    held[page] = rid
                    if g.pool.owner_of(page) != rid:
                        raise AssertionError(f"group {gi}: page {page} owner record is wrong")
            if set(free) & set(held):
                raise AssertionError(f"group {gi}: a page is free and held at once")
            if len(free) + len(held) != g.pool.num_pages:
                raise AssertionError(f"group {gi}: {g.pool.num_pages - len(free) - len(held)} pages lost")
        slots = [rc.state_slot for rc in self._requests.values()] + list(self._free_slots)
        if sorted(slots) != list(range(self.max_requests)):
            raise AssertionError("state slots lost or held twice")
