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

Prefix cache (optional, block_manager.py:108-114,181-237,240-266): a page that is full of computed
keys is filed under a hash chained over all tokens up to its end. It keeps that entry after its
holders are gone, until the pool hands the page out again; a new request whose prompt starts with
the same tokens takes such pages over instead of computing them, and several requests may hold
one page at once. Only full pages are shared and at least one token of a prompt is always left to
run, so no shared page is ever written. It is offered only where every cache entry keeps all keys
and no mixer has state of its own: a window gives pages back early, and a state cannot be
recovered from pages.
"""
from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict, deque
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Set, Tuple

from ..parts.base import CacheNeed, StateNeed


class CacheExhausted(RuntimeError):
    pass


class PagePool:
    """Page ids 0..n-1 of one group. A page is free, or held by one request, or (prefix cache)
    by several; the free pages form a queue that is served from its head."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        self._free: "OrderedDict[int, None]" = OrderedDict((p, None) for p in range(num_pages))
        self._holders: List[Set[Hashable]] = [set() for _ in range(num_pages)]
        self.on_reuse: Optional[Callable[[int], None]] = None   # told when a free page is handed out
        self.pages_taken = 0          # counters for stats(): how often pages changed hands
        self.pages_returned = 0
        self.pages_shared = 0

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, owner: Hashable) -> int:
        """The free page that has waited longest; what it held is forgotten."""
        if not self._free:
            raise CacheExhausted("KV cache exhausted")
        page, _ = self._free.popitem(last=False)
        if self._holders[page]:
            raise RuntimeError(f"page {page} was free and owned at once")
        if self.on_reuse is not None:
            self.on_reuse(page)
        self._holders[page].add(owner)
        self.pages_taken += 1
        return page

    def share(self, page: int, owner: Hashable) -> None:
        """One more holder for a page whose content is kept: held by others, or free."""
        if not 0 <= page < self.num_pages:
            raise RuntimeError(f"page {page} does not exist")
        if owner in self._holders[page]:
            raise RuntimeError(f"page {page} is already held by {owner!r}")
        if not self._holders[page]:
            del self._free[page]
        self._holders[page].add(owner)
        self.pages_shared += 1

    def give_back(self, page: int, owner: Hashable) -> None:
        if not 0 <= page < self.num_pages:
            raise RuntimeError(f"page {page} does not exist")
        holders = self._holders[page]
        if not holders:
            raise RuntimeError(f"page {page} freed twice")
        if owner not in holders:
            raise RuntimeError(f"page {page} belongs to {sorted(map(repr, holders))}, not to {owner!r}")
        holders.remove(owner)
        if not holders:
            self._free[page] = None
        self.pages_returned += 1

    def holders_of(self, page: int) -> Set[Hashable]:
        return set(self._holders[page])

    def owner_of(self, page: int) -> Optional[Hashable]:
        """The holder of a page that has exactly one; None for a free page."""
        holders = self._holders[page]
        if len(holders) > 1:
            raise RuntimeError(f"page {page} has {len(holders)} holders")
        return next(iter(holders)) if holders else None

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
    page_hashes: List[int] = field(default_factory=list)     # prefix cache: chain over its full pages
    serial: int = 0                                          # which admission this is: ids may come back, serials never do


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


def prefix_caching_possible(needs) -> bool:
    """True if a prompt's first pages say all there is to say about its first tokens: one group
    of cache entries, every one keeping all keys, and no per-request state."""
    needs = list(needs)
    groups = group_cache_needs(needs)
    return (len(groups) == 1 and groups[0][0].window is None
            and all(state is None for _need, state in needs))


def hash_page(previous: int, token_ids: Sequence[int]) -> int:
    """64-bit hash of one full page, chained to the hash of the pages before it (0 for the first):
    equal hashes mean equal tokens from the start of the prompt (block_manager.py:108-114; the
    hash function itself is not the reference's, nothing depends on its values)."""
    h = hashlib.blake2b(digest_size=8)
    h.update(struct.pack("<Q", previous))
    h.update(struct.pack(f"<{len(token_ids)}i", *token_ids))
    return int.from_bytes(h.digest(), "little")


class CacheManager:
    def __init__(self, needs, page_size: int, num_pages: int, max_requests: int,
                 prefix_caching: bool = False):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        if max_requests <= 0:
            raise ValueError("max_requests must be positive")
        needs = list(needs)
        if prefix_caching and not prefix_caching_possible(needs):
            raise ValueError("a prefix cache needs a model whose cache entries all keep every key "
                             "and whose mixers have no state of their own")
        self.page_size = page_size
        self.max_requests = max_requests
        self.groups = [CacheGroup(need, entries, PagePool(num_pages))
                       for need, entries in group_cache_needs(needs)]
        self.group_of_entry: Dict[int, int] = {e: g for g, grp in enumerate(self.groups)
                                               for e in grp.entries}
        self._free_slots = deque(range(max_requests))
        self._fresh_slots: List[int] = []
        self._requests: Dict[Hashable, RequestCache] = {}
        self._admissions = 0
        self.prefix_caching = prefix_caching
        # prefix cache: page -> (hash, hash of the pages before, its tokens) and hash -> page
        self._page_key: Dict[int, Tuple[int, int, Tuple[int, ...]]] = {}
        self._page_of_hash: Dict[int, int] = {}
        self.prefix_queries = 0
        self.prefix_hit_tokens = 0
        if prefix_caching:
            self.groups[0].pool.on_reuse = self._forget_page

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

    def admit(self, request_id, token_ids: Optional[Sequence[int]] = None) -> RequestCache:
        """Gives the request a state slot and block tables: empty ones, or (prefix cache on and
        ``token_ids`` given) holding the kept pages that its tokens begin with; ``length`` of the
        result says how many tokens those cover. At least one token is left to run
        (block_manager.py:218)."""
        if request_id in self._requests:
            raise RuntimeError(f"request {request_id!r} is already live")
        if not self._free_slots:
            raise CacheExhausted("no free state slot: too many live requests")
        self._admissions += 1
        rc = RequestCache(request_id, self._free_slots.popleft(),
                          tables=[[] for _ in self.groups], serial=self._admissions)
        self._fresh_slots.append(rc.state_slot)
        self._requests[request_id] = rc
        if self.prefix_caching and token_ids is not None:
            pool, size = self.groups[0].pool, self.page_size
            previous = 0
            for i in range((len(token_ids) - 1) // size):
                tokens = tuple(int(t) for t in token_ids[i * size:(i + 1) * size])
                h = hash_page(previous, tokens)
                page = self._page_of_hash.get(h)
                if page is None or self._page_key[page] != (h, previous, tokens):
                    break
                pool.share(page, request_id)
                rc.tables[0].append(page)
                rc.page_hashes.append(h)
                previous = h
            rc.length = len(rc.page_hashes) * size
            self.prefix_queries += 1
            self.prefix_hit_tokens += rc.length
        return rc

    def take_fresh_slots(self) -> List[int]:
        """State slots handed out since the last call: whoever owns the state tensors clears
        them before the next step."""
        slots, self._fresh_slots = self._fresh_slots, []
        return slots

    def note_tokens(self, request_id, token_ids: Sequence[int]) -> None:
        """Prefix cache: files every page of the request that has become full of stored keys
        under its chained hash (block_manager.py:240-266). ``token_ids`` are the request's tokens
        from its start, at least as many as are stored."""
        if not self.prefix_caching:
            return
        rc = self._requests[request_id]
        size = self.page_size
        previous = rc.page_hashes[-1] if rc.page_hashes else 0
        for i in range(len(rc.page_hashes), rc.length // size):
            tokens = tuple(int(t) for t in token_ids[i * size:(i + 1) * size])
            if len(tokens) != size:
                raise ValueError("fewer tokens given than keys are stored")
            h = hash_page(previous, tokens)
            page = rc.tables[0][i]
            if h not in self._page_of_hash and page not in self._page_key:
                self._page_of_hash[h] = page
                self._page_key[page] = (h, previous, tokens)
            rc.page_hashes.append(h)
            previous = h

    def _forget_page(self, page: int) -> None:
        key = self._page_key.pop(page, None)
        if key is not None:
            del self._page_of_hash[key[0]]

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

    def extend_many(self, wanted: Sequence[Tuple[Hashable, int]]) -> None:
        """``extend`` for several requests at once, all or none: the pages that all of them lack
        are counted against the free ones first, and CacheExhausted leaves every table as it was."""
        lacking = [0] * len(self.groups)
        for request_id, new_length in wanted:
            rc = self._requests[request_id]
            if new_length < rc.length:
                raise ValueError("a request's cache cannot shrink")
            for gi, m in enumerate(self._missing(rc, new_length)):
                lacking[gi] += m
        for gi, (m, g) in enumerate(zip(lacking, self.groups)):
            if m > g.pool.num_free:
                raise CacheExhausted(f"KV cache exhausted: the step needs {m} more pages in group {gi}, "
                                     f"{g.pool.num_free} are free")
        for request_id, new_length in wanted:
            self.extend(request_id, new_length)

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
            "prefix_caching": self.prefix_caching,
            "prefix_queries": self.prefix_queries,
            "prefix_hit_tokens": self.prefix_hit_tokens,
            "kept_pages": len(self._page_key),
            "groups": [{"window": g.need.window, "entries": len(g.entries),
                        "pages": g.pool.num_pages, "free_pages": g.pool.num_free,
                        "pages_taken": g.pool.pages_taken, "pages_returned": g.pool.pages_returned}
                       for g in self.groups],
        }

    def check_consistency(self) -> None:
        """No page lost, none held twice (beyond the sharing the prefix cache does), none free
        and held at once, the prefix index and the pool agree; slots likewise."""
        for gi, g in enumerate(self.groups):
            free = g.pool.free_pages()
            if len(set(free)) != len(free):
                raise AssertionError(f"group {gi}: a page is on the free list twice")
            held: Dict[int, Set[Hashable]] = {}
            for rid, rc in self._requests.items():
                pages = [p for p in rc.tables[gi] if p >= 0]
                if len(set(pages)) != len(pages):
                    raise AssertionError(f"group {gi}: request {rid!r} holds a page twice")
                for page in pages:
                    if page in held and not self.prefix_caching:
                        raise AssertionError(f"group {gi}: page {page} held by "
                                             f"{sorted(map(repr, held[page]))} and {rid!r}")
                    held.setdefault(page, set()).add(rid)
            for page, holders in held.items():
                if g.pool.holders_of(page) != holders:
                    raise AssertionError(f"group {gi}: page {page} owner record is wrong")
            if set(free) & set(held):
                raise AssertionError(f"group {gi}: a page is free and held at once")
            if len(free) + len(held) != g.pool.num_pages:
                raise AssertionError(f"group {gi}: {g.pool.num_pages - len(free) - len(held)} pages lost")
        for page, (h, _previous, tokens) in self._page_key.items():
            if self._page_of_hash.get(h) != page or len(tokens) != self.page_size:
                raise AssertionError(f"prefix index: page {page} is filed wrongly")
        if len(self._page_of_hash) != len(self._page_key):
            raise AssertionError("prefix index: a hash without its page")
        for rid, rc in self._requests.items():
            if self.prefix_caching and len(rc.page_hashes) > rc.length // self.page_size:
                raise AssertionError(f"request {rid!r} has hashes for pages that are not full")
        slots = [rc.state_slot for rc in self._requests.values()] + list(self._free_slots)
        if sorted(slots) != list(range(self.max_requests)):
            raise AssertionError("state slots lost or held twice")
