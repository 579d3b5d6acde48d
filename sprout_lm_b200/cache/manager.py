"""Host-side cache manager: pages, block tables, prefix reuse, state slots.

The logical model is the reference's KVCache / PagedSequence
(src/kv-cache.ts:5-172): fixed pages of ``page_tokens`` positions, a block
table per request, a reference count per page (one per live request that holds
it, one for the prefix map), a free list that hands out the lowest page first
and reuses returned pages last-in first-out, a prefix map keyed by *all* tokens
from position 0 to the end of the page, and least-recently-used eviction of
prefix pages that no live request holds.

Beyond the reference, layers are put in *groups*.  Every group has pages of
its own (its own pool and its own block table in each request): a ``full``
group keeps every position, a ``window`` group gives a page back as soon as
every later query is further than ``window`` positions away from all of it.
Beside the pages there are slots for per-request state of fixed size, taken
when a request's cache is created and given back with it.

This module holds no device memory; it decides which page holds what.
"""
from __future__ import annotations

import heapq
from dataclasses import dataclass
from typing import Sequence


class CacheError(RuntimeError):
    pass


@dataclass(frozen=True)
class GroupSpec:
    """Layers (by cache slot) whose cache behaves alike.

    kind ``full`` keeps all positions; ``window`` keeps the last ``window``
    positions that a query can still see (a query at position q sees keys
    p with q - p < window).
    """
    name: str
    kind: str = "full"
    window: int | None = None
    slots: tuple[int, ...] = ()

    def __post_init__(self):
        if self.kind not in ("full", "window"):
            raise CacheError(f"unknown cache group kind {self.kind!r}")
        if (self.kind == "window") != (self.window is not None) or (self.window is not None and self.window <= 0):
            raise CacheError("a window group needs a positive window, a full group none")


class PagePool:
    """Reference counts and the free list of one group's pages (src/kv-cache.ts:94-95,125-145)."""

    def __init__(self, num_pages: int):
        if not isinstance(num_pages, int) or num_pages <= 0:
            raise CacheError("num_pages must be a positive integer.")
        self.num_pages = num_pages
        self.refs = [0] * num_pages
        self.free = list(range(num_pages - 1, -1, -1))

    def take(self) -> int | None:
        if not self.free:
            return None
        page = self.free.pop()
        self.refs[page] = 1
        return page

    def share(self, page: int) -> None:
        if self.refs[page] <= 0:
            raise CacheError("cannot share a free page.")
        self.refs[page] += 1

    def release(self, page: int) -> None:
        if self.refs[page] <= 0:
            raise CacheError("KV reference count underflow.")
        self.refs[page] -= 1
        if self.refs[page] == 0:
            self.free.append(page)


@dataclass
class _PrefixEntry:
    pages: tuple[int, ...]          # one page per group
    parent: int                     # id of the entry of the previous page, 0 at the start
    tokens: tuple[int, ...]         # this page's tokens
    last_used: int
    ident: int
    children: int = 0               # entries that continue this one (only an entry without any may be evicted)


class SequenceCache:
    """One request's block tables (one per group), its length and its state slot."""

    def __init__(self, manager: "CacheManager", state_slot: int):
        self._manager = manager
        self.tables: list[list[int]] = [[] for _ in manager.groups]
        self.length = 0
        self.state_slot = state_slot
        self.released = False
        self._prefix_tail = 0       # id of the prefix entry that covers the pages published or reused so far
        self._published_pages = 0

    @property
    def blocks(self) -> list[int]:
        """The first group's block table (the only one for a model with one group)."""
        return self.tables[0]

    def capacity(self, group: int = 0) -> int:
        return len(self.tables[group]) * self._manager.page_tokens

    def _assert_live(self):
        if self.released:
            raise CacheError("Sequence KV was released.")


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], num_pages, page_tokens: int,
                 state_slots: int = 0, prefix_caching: bool = True):
        if not groups:
            raise CacheError("at least one cache group is needed (it may have no layers).")
        if not isinstance(page_tokens, int) or page_tokens <= 0:
            raise CacheError("page_tokens must be a positive integer.")
        self.groups = tuple(groups)
        counts = [num_pages] * len(self.groups) if isinstance(num_pages, int) else list(num_pages)
        if len(counts) != len(self.groups):
            raise CacheError("one page count per group is needed.")
        self.pools = [PagePool(n) for n in counts]
        self.page_tokens = page_tokens
        # prefix reuse skips computing the reused positions: only sound when every group keeps
        # every position and no request carries state that those positions would have built
        self.prefix_caching = bool(prefix_caching) and all(g.kind == "full" for g in self.groups) \
            and state_slots == 0
        self._prefixes: dict[tuple[int, tuple[int, ...]], _PrefixEntry] = {}
        self._entry_by_id: dict[int, _PrefixEntry] = {}
        self._next_entry = 1
        self._clock = 0
        # For eviction without a walk over all entries: which entry a page belongs to (keyed by
        # (group, page): an entry holds one page of every group), a heap of (last_used, ident)
        # records pushed whenever an entry becomes evictable (stale records are skipped when
        # popped), and the number of entries whose pages only the map holds.
        self._entry_of_page: dict[tuple[int, int], _PrefixEntry] = {}
        self._evict_heap: list[tuple[int, int]] = []
        self._cached_only = 0
        self.evictions = 0
        self.state_slot_count = state_slots
        self._free_state = list(range(state_slots - 1, -1, -1))
        self._live: set[int] = set()

    # ------------------------------------------------------------------ sequences
    def create(self) -> SequenceCache:
        """An empty cache for a request; takes a state slot when the model has per-request state."""
        slot = -1
        if self.state_slot_count:
            if not self._free_state:
                raise CacheError("no free state slot.")
            slot = self._free_state.pop()
        seq = SequenceCache(self, slot)
        self._live.add(id(seq))
        return seq

    def can_create(self) -> bool:
        return not self.state_slot_count or bool(self._free_state)

    def reuse_prefix(self, tokens: Sequence[int]) -> SequenceCache:
        """A cache that already holds the longest published page-aligned prefix of ``tokens``,
        always leaving at least the last token to compute (src/kv-cache.ts:100-112)."""
        seq = self.create()
        if not self.prefix_caching:
            return seq
        parent = 0
        end = self.page_tokens
        while end < len(tokens):
            entry = self._prefixes.get((parent, tuple(tokens[end - self.page_tokens:end])))
            if entry is None:
                break
            if self._map_only(entry):
                self._cached_only -= 1                 # a request holds it again
            for group, page in enumerate(entry.pages):
                self.pools[group].share(page)
                seq.tables[group].append(page)
            self._clock += 1
            entry.last_used = self._clock
            seq.length = end
            parent = entry.ident
            end += self.page_tokens
        seq._prefix_tail = parent
        seq._published_pages = seq.length // self.page_tokens
        return seq

    def publish(self, tokens: Sequence[int], seq: SequenceCache) -> None:
        """Offer for reuse every page that ``seq`` has filled completely with ``tokens``.

        ``tokens`` are the tokens from position 0 on that may be shared (a request's prompt);
        pages beyond them, or not yet computed, are not offered.  The key of a page is the whole
        token sequence from position 0 to the page's end (src/kv-cache.ts:114-123), held as a
        chain: (entry of the previous page, this page's tokens)."""
        if not self.prefix_caching or seq.released:
            return
        pages_done = min(len(tokens), seq.length) // self.page_tokens
        while seq._published_pages < pages_done:
            index = seq._published_pages
            page_tokens = tuple(tokens[index * self.page_tokens:(index + 1) * self.page_tokens])
            key = (seq._prefix_tail, page_tokens)
            entry = self._prefixes.get(key)
            if entry is None:
                pages = tuple(table[index] for table in seq.tables)
                for group, page in enumerate(pages):
                    self.pools[group].share(page)      # the map's own reference
                self._clock += 1
                entry = _PrefixEntry(pages, seq._prefix_tail, page_tokens, self._clock, self._next_entry)
                self._next_entry += 1
                self._prefixes[key] = entry
                self._entry_by_id[entry.ident] = entry
                for group, page in enumerate(pages):
                    self._entry_of_page[(group, page)] = entry
                parent = self._entry_by_id.get(entry.parent)       # gone if the map was cleared meanwhile
                if parent is not None:
                    parent.children += 1
            seq._prefix_tail = entry.ident
            seq._published_pages += 1

    def reserve(self, seq: SequenceCache, tokens: int) -> bool:
        """Make room for positions up to ``tokens`` in every group, at most one new page per
        group and call.  False when a group has no page left even after evicting an unused
        prefix page (src/kv-cache.ts:13-20,125-139)."""
        seq._assert_live()
        for group, table in enumerate(seq.tables):
            if tokens <= len(table) * self.page_tokens:
                continue
            page = self._allocate(group)
            if page is None:
                return False
            table.append(page)
            if tokens > len(table) * self.page_tokens:
                raise CacheError("reserve() grows a request by at most one page per call.")
        return True

    def trim(self, seq: SequenceCache) -> int:
        """Give back the pages of window groups that no later query of ``seq`` can see.
        Their block-table entries become -1.  Returns how many pages were given back."""
        seq._assert_live()
        given_back = 0
        for group, spec in enumerate(self.groups):
            if spec.kind != "window":
                continue
            # the next query sits at position seq.length and sees keys p > seq.length - window
            first_needed = seq.length - spec.window + 1
            whole_pages_before = max(0, first_needed) // self.page_tokens
            table = seq.tables[group]
            for index in range(min(whole_pages_before, len(table))):
                if table[index] >= 0:
                    self.pools[group].release(table[index])
                    table[index] = -1
                    given_back += 1
        return given_back

    def release(self, seq: SequenceCache) -> None:
        """Drop the request's reference on each of its pages and give back its state slot."""
        if seq.released:
            return
        touched: dict[int, _PrefixEntry] = {}          # the prefix entries whose pages this request held
        for group, table in enumerate(seq.tables):
            for page in table:
                if page >= 0:
                    entry = self._entry_of_page.get((group, page))
                    if entry is not None:
                        touched[entry.ident] = entry
                    self.pools[group].release(page)
            table.clear()
        for entry in touched.values():                 # entries that only the prefix map holds now
            if self._map_only(entry):
                self._cached_only += 1
                self._consider(entry)
        if seq.state_slot >= 0:
            self._free_state.append(seq.state_slot)
            seq.state_slot = -1
        seq.released = True
        self._live.discard(id(seq))

    # ------------------------------------------------------------------ pages
    def _allocate(self, group: int) -> int | None:
        pool = self.pools[group]
        if not pool.free:
            self._evict_one()
        return pool.take()

    def _map_only(self, entry: _PrefixEntry) -> bool:
        """No live request holds any of the entry's pages (one per group): only the map does."""
        return all(self.pools[g].refs[p] == 1 for g, p in enumerate(entry.pages))

    def _consider(self, entry: _PrefixEntry) -> None:
        """Note ``entry`` as evictable if no live request holds its pages and no entry continues it."""
        if entry.children == 0 and self._map_only(entry):
            heapq.heappush(self._evict_heap, (entry.last_used, entry.ident))

    def _evict_one(self) -> bool:
        """Evict the least recently used prefix entry none of whose pages a live request holds
        and which no other entry continues (of two used at the same time, the older entry)."""
        while self._evict_heap:
            last_used, ident = heapq.heappop(self._evict_heap)
            candidate = self._entry_by_id.get(ident)
            if candidate is None or candidate.last_used != last_used or candidate.children:
                continue                               # a stale record
            if not self._map_only(candidate):
                continue
            del self._prefixes[(candidate.parent, candidate.tokens)]
            del self._entry_by_id[candidate.ident]
            for group, page in enumerate(candidate.pages):
                del self._entry_of_page[(group, page)]
            self._cached_only -= 1
            for group, page in enumerate(candidate.pages):
                self.pools[group].release(page)
            parent = self._entry_by_id.get(candidate.parent)
            if parent is not None:
                parent.children -= 1
                self._consider(parent)
            self.evictions += 1
            return True
        return False

    def clear_prefixes(self) -> None:
        for entry in self._prefixes.values():
            for group, page in enumerate(entry.pages):
                self.pools[group].release(page)
        self._prefixes.clear()
        self._entry_by_id.clear()
        self._entry_of_page.clear()
        self._evict_heap.clear()
        self._cached_only = 0

    # ------------------------------------------------------------------ reporting
    def free_pages(self, group: int = 0) -> int:
        return len(self.pools[group].free)

    def available_pages(self, group: int = 0) -> int:
        """Pages of ``group`` that a request could get now: the free ones and those that only the
        prefix map holds (an entry holds one page of every group; they are evicted on demand,
        leaves first)."""
        return len(self.pools[group].free) + self._cached_only

    def snapshot(self) -> dict:
        """Page accounting in the reference's form (src/kv-cache.ts:162-171); with more than one
        group the first group's figures are at the top level and all are under ``groups``."""
        groups = []
        for group, pool in enumerate(self.pools):
            cached = {e.pages[group] for e in self._prefixes.values()}
            groups.append({
                "name": self.groups[group].name, "totalPages": pool.num_pages, "freePages": len(pool.free),
                "cachedPages": len(cached), "evictions": self.evictions,
                "pages": [{"id": i, "refs": r, "cached": i in cached, "activeRefs": r - int(i in cached)}
                          for i, r in enumerate(pool.refs)]})
        top = dict(groups[0])
        top.pop("name")
        if len(groups) > 1:
            top["groups"] = groups
        if self.state_slot_count:
            top["stateSlots"] = {"total": self.state_slot_count, "free": len(self._free_state)}
        return top

    def check_invariants(self) -> None:
        """Every page is either free with no reference or held with at least one, and is on the
        free list at most once."""
        for pool in self.pools:
            if len(set(pool.free)) != len(pool.free):
                raise CacheError("a page is on the free list twice.")
            for page, refs in enumerate(pool.refs):
                if refs < 0:
                    raise CacheError("negative reference count.")
                if (refs == 0) != (page in set(pool.free)):
                    raise CacheError(f"page {page}: refs {refs} but free={page in pool.free}")
        if len(set(self._free_state)) != len(self._free_state):
            raise CacheError("a state slot is free twice.")
        # the eviction bookkeeping against a recount
        entries = list(self._entry_by_id.values())
        if self._cached_only != sum(1 for e in entries if self._map_only(e)):
            raise CacheError("the count of prefix entries that only the map holds is off.")
        children: dict[int, int] = {}
        for e in entries:
            children[e.parent] = children.get(e.parent, 0) + 1
        records = set(self._evict_heap)
        for e in entries:
            if e.children != children.get(e.ident, 0):
                raise CacheError(f"prefix entry {e.ident}: {e.children} children noted, {children.get(e.ident, 0)} found.")
            if any(self._entry_of_page.get((g, p)) is not e for g, p in enumerate(e.pages)):
                raise CacheError(f"prefix entry {e.ident} is not found by its pages.")
            evictable = e.children == 0 and self._map_only(e)
            if evictable and (e.last_used, e.ident) not in records:
                raise CacheError(f"prefix entry {e.ident} could be evicted but is not noted for it.")
