"""Host-side bookkeeping of the paged key/value cache and of per-request state slots.

What it owns: which physical page of which layer group belongs to which request, each
request's block table per group, how many tokens of a request are reserved and how many
are computed, and which fixed-size state slot a request has.  It owns no device memory
(``storage.py`` does) and launches nothing, so all of it is tested without a GPU.

In the reference the same duties are spread over ``base::BlockAllocator`` (one pool per
layer, FIFO free queue, refcounts, generations: infMain/source/base/block_allocator.cpp:
205-230, 264-282), ``base::SequenceKVManager`` (per-request page tables, transactional
append with rollback: infMain/source/base/sequence_kv_manager.cpp:204-299) and
``base::KVCacheManager`` (request handles made of slot and generation, stale handles
rejected: infMain/source/base/kv_cache_manager.cpp:44-59, 167-236, 756-784).  Differences
by design: a page id is valid for every layer of its group (the reference allocates all
layer pools in lock-step and then uses layer 0's table for all of them,
infMain/source/serving/mixed_batch_builder.cpp:150,190); layers with different needs
(all keys, or a window of keys) form groups with pools of their own; a windowed group
gives pages back as soon as the window has passed them.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

_SLOT_BITS = 20
_SLOT_MASK = (1 << _SLOT_BITS) - 1
NO_PAGE = -1


class CacheError(RuntimeError):
    """Misuse of the cache manager: a stale handle, a page freed twice, and the like."""


@dataclass(frozen=True)
class KVGroupSpec:
    """Layers whose keys and values have the same geometry and the same lifetime."""
    layers: Tuple[int, ...]          # cache layer indices of the model's run order
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None     # None: every key is kept; W: only the last W keys are read


class PagePool:
    """Physical page ids 0..n-1 of one group: a free queue, a reference count and a
    generation per page.  ``lifo`` takes the page given back last first (pages are then
    used again at once, which tests want); the default FIFO spreads reuse."""

    def __init__(self, num_pages: int, lifo: bool = False):
        if num_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = int(num_pages)
        self.lifo = lifo
        self._free = deque(range(self.num_pages))
        self._refs = [0] * self.num_pages
        self.generation = [0] * self.num_pages
        self.allocations = 0

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            return NO_PAGE
        page = self._free.pop() if self.lifo else self._free.popleft()
        if self._refs[page] != 0:
            raise CacheError(f"page {page} was in the free queue while held {self._refs[page]} times")
        self._refs[page] = 1
        self.generation[page] += 1
        self.allocations += 1
        return page

    def release(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise CacheError(f"page id {page} is outside the pool of {self.num_pages}")
        if self._refs[page] <= 0:
            raise CacheError(f"page {page} freed twice")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)

    def refcount(self, page: int) -> int:
        return self._refs[page]


@dataclass
class _Request:
    slot: int
    generation: int
    reserved: int = 0                 # tokens backed by pages (computed + in flight)
    computed: int = 0                 # tokens whose keys and values are written
    tables: List[List[int]] = field(default_factory=list)   # per group: page of logical block i
    first_live: List[int] = field(default_factory=list)     # per group: first block not yet given back
    user_id: object = None


class CacheManager:
    """Pages, block tables and state slots of all live requests.

    ``add_request`` gives a handle (slot and generation packed in one integer);
    ``reserve(handle, n)`` backs the next ``n`` tokens with pages in every group or
    changes nothing; ``commit(handle, n)`` marks them computed and gives back pages that
    a window has passed; ``free(handle)`` gives everything back.
    """

    def __init__(self, groups: Sequence[KVGroupSpec], page_tokens: int, num_pages,
                 max_requests: int = 256, state_bytes: int = 0, lifo: bool = False):
        if page_tokens <= 0:
            raise CacheError(f"page_tokens must be positive, got {page_tokens}")
        if max_requests <= 0 or max_requests > _SLOT_MASK:
            raise CacheError(f"max_requests must be in 1..{_SLOT_MASK}, got {max_requests}")
        self.groups = tuple(groups)
        self.page_tokens = int(page_tokens)
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(self.groups)
        if len(num_pages) != len(self.groups):
            raise CacheError("num_pages needs one entry per group")
        self.pools = [PagePool(n, lifo=lifo) for n in num_pages]
        self.max_requests = int(max_requests)
        self.state_bytes = int(state_bytes)
        self._slots: List[Optional[_Request]] = [None] * self.max_requests
        self._slot_generation = [0] * self.max_requests
        self._free_slots = deque(range(self.max_requests))
        self.state_slot_assignments = 0

    # ------------------------------------------------------------------ handles
    def _lookup(self, handle: int) -> _Request:
        if not isinstance(handle, int) or handle < 0:
            raise CacheError(f"malformed request handle {handle!r}")
        slot, gen = handle & _SLOT_MASK, handle >> _SLOT_BITS
        if slot >= self.max_requests:
            raise CacheError(f"request handle {handle} names slot {slot} of {self.max_requests}")
        req = self._slots[slot]
        if req is None or req.generation != gen:
            raise CacheError(f"stale request handle {handle} (slot {slot}, generation {gen})")
        return req

    def is_live(self, handle: int) -> bool:
        try:
            self._lookup(handle)
            return True
        except CacheError:
            return False

    @property
    def num_live_requests(self) -> int:
        return self.max_requests - len(self._free_slots)

    def add_request(self, user_id=None) -> Optional[int]:
        """A new request with no tokens; None when every request slot is taken."""
        if not self._free_slots:
            return None
        slot = self._free_slots.popleft()
        self._slot_generation[slot] += 1
        gen = self._slot_generation[slot]
        self._slots[slot] = _Request(slot=slot, generation=gen,
                                     tables=[[] for _ in self.groups],
                                     first_live=[0 for _ in self.groups], user_id=user_id)
        self.state_slot_assignments += 1
        return (gen << _SLOT_BITS) | slot

    def state_slot(self, handle: int) -> int:
        """Index of the request's fixed-size state (row of the state tensor)."""
        return self._lookup(handle).slot

    # ------------------------------------------------------------------ sizes
    def context_len(self, handle: int) -> int:
        return self._lookup(handle).computed

    def reserved_len(self, handle: int) -> int:
        return self._lookup(handle).reserved

    def num_free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def _blocks_for(self, tokens: int) -> int:
        return (tokens + self.page_tokens - 1) // self.page_tokens

    def pages_needed(self, handle: int, n_tokens: int) -> List[int]:
        """New pages per group that ``reserve(handle, n_tokens)`` would take."""
        req = self._lookup(handle)
        target = self._blocks_for(req.reserved + n_tokens)
        return [max(0, target - len(t)) for t in req.tables]

    def can_reserve(self, handle: int, n_tokens: int) -> bool:
        need = self.pages_needed(handle, n_tokens)
        return all(n <= p.num_free for n, p in zip(need, self.pools))

    def max_appendable_tokens(self, handle: int) -> int:
        """How many more tokens fit: room in the last page plus the free pages, the
        smallest over the groups (infMain/source/serving/scheduler.cpp:23-34)."""
        req = self._lookup(handle)
        best = None
        for table, pool in zip(req.tables, self.pools):
            room = len(table) * self.page_tokens - req.reserved + pool.num_free * self.page_tokens
            best = room if best is None else min(best, room)
        return max(0, best) if best is not None else (1 << 30)

    def capacity_tokens(self) -> int:
        """Tokens one request could hold with every page of the scarcest group."""
        if not self.pools:
            return 1 << 30
        return min(p.num_pages for p in self.pools) * self.page_tokens

    # ------------------------------------------------------------------ pages
    def reserve(self, handle: int, n_tokens: int) -> bool:
        """Back tokens [reserved, reserved + n) with pages in every group, or change nothing."""
        if n_tokens < 0:
            raise CacheError(f"cannot reserve {n_tokens} tokens")
        req = self._lookup(handle)
        # the usual decode step: the token still fits in the last page of every group
        room = req.reserved + n_tokens
        if all(room <= len(t) * self.page_tokens for t in req.tables):
            req.reserved = room
            return True
        need = self.pages_needed(handle, n_tokens)
        if any(n > p.num_free for n, p in zip(need, self.pools)):
            return False
        for g, n in enumerate(need):
            for _ in range(n):
                page = self.pools[g].allocate()
                if page == NO_PAGE:   # cannot happen after the check above
                    raise CacheError("page pool ran dry inside a checked reservation")
                req.tables[g].append(page)
        req.reserved += n_tokens
        return True

    def commit(self, handle: int, n_tokens: int) -> None:
        """Mark ``n_tokens`` more as computed and give back what a window has passed.

        A query at position p of a windowed group reads keys p-W+1..p, so once ``computed``
        tokens are written, the next query (position ``computed``) needs nothing below
        ``computed - W + 1``; pages that end at or before it go back to the pool and their
        block-table entries become NO_PAGE."""
        req = self._lookup(handle)
        if n_tokens < 0 or req.computed + n_tokens > req.reserved:
            raise CacheError(
                f"commit of {n_tokens} tokens exceeds the reservation ({req.computed}+{n_tokens} > {req.reserved})")
        req.computed += n_tokens
        for g, spec in enumerate(self.groups):
            if spec.window is None:
                continue
            first_needed = req.computed - spec.window + 1
            if first_needed <= 0:
                continue
            dead_blocks = min(first_needed // self.page_tokens, len(req.tables[g]))
            for b in range(req.first_live[g], dead_blocks):
                page = req.tables[g][b]
                if page != NO_PAGE:
                    self.pools[g].release(page)
                    req.tables[g][b] = NO_PAGE
            req.first_live[g] = max(req.first_live[g], dead_blocks)

    def truncate(self, handle: int, n_tokens: int) -> None:
        """Keep only the first ``n_tokens`` tokens (gives back tail pages).  Not allowed
        below what a window has already released."""
        req = self._lookup(handle)
        if n_tokens < 0 or n_tokens > req.reserved:
            raise CacheError(f"cannot truncate to {n_tokens} tokens (reserved {req.reserved})")
        keep = self._blocks_for(n_tokens)
        for g, table in enumerate(req.tables):
            if keep < req.first_live[g]:
                raise CacheError("cannot truncate below pages a window has already given back")
            while len(table) > keep:
                page = table.pop()
                if page != NO_PAGE:
                    self.pools[g].release(page)
        req.reserved = n_tokens
        req.computed = min(req.computed, n_tokens)

    def free(self, handle: int) -> None:
        req = self._lookup(handle)
        for g, table in enumerate(req.tables):
            for page in table:
                if page != NO_PAGE:
                    self.pools[g].release(page)
            table.clear()
        self._slots[req.slot] = None
        self._free_slots.append(req.slot)

    def reset(self) -> None:
        for slot, req in enumerate(self._slots):
            if req is not None:
                self.free((req.generation << _SLOT_BITS) | slot)

    # ------------------------------------------------------------------ views
    def block_table(self, handle: int, group: int = 0) -> List[int]:
        return self._lookup(handle).tables[group]

    def slot_of_token(self, handle: int, group: int, position: int) -> int:
        """page * page_tokens + offset of a token (infMain/source/base/sequence_kv_manager.cpp:41-52)."""
        table = self._lookup(handle).tables[group]
        page = table[position // self.page_tokens]
        if page == NO_PAGE:
            raise CacheError(f"position {position} lies in a page that was given back")
        return page * self.page_tokens + position % self.page_tokens

    def page_generation(self, group: int, page: int) -> int:
        return self.pools[group].generation[page]

    # ------------------------------------------------------------------ self check
    def check_invariants(self) -> None:
        """No page lost, held twice or both held and free; counts agree."""
        for g, pool in enumerate(self.pools):
            held: Dict[int, int] = {}
            for req in self._slots:
                if req is None:
                    continue
                for page in req.tables[g]:
                    if page == NO_PAGE:
                        continue
                    held[page] = held.get(page, 0) + 1
            free = list(pool._free)
            if len(set(free)) != len(free):
                raise CacheError(f"group {g}: a page is in the free queue twice")
            for page, n in held.items():
                if n != 1:
                    raise CacheError(f"group {g}: page {page} is held by {n} block tables")
                if pool.refcount(page) != 1:
                    raise CacheError(f"group {g}: page {page} is held but its count is {pool.refcount(page)}")
                if page in set(free):
                    raise CacheError(f"group {g}: page {page} is both held and free")
            if len(held) + len(free) != pool.num_pages:
                raise CacheError(
                    f"group {g}: {pool.num_pages - len(held) - len(free)} pages are lost "
                    f"({len(held)} held, {len(free)} free of {pool.num_pages})")
        for req in self._slots:
            if req is None:
                continue
            if not (0 <= req.computed <= req.reserved):
                raise CacheError("computed/reserved out of order")
            for table in req.tables:
                if len(table) != self._blocks_for(req.reserved):
                    raise CacheError("a block table does not cover the reservation")
