"""The cache manager: pages of keys and values with a block table per request, and slots for
per-request state of fixed size.  Pure host code; the device tensors live in ``storage.py``.

What is kept from the reference's ``BlockPool``/``KVCacheManager`` (src/kv_cache/block_pool.cpp:
13-103, src/kv_cache/manager.cpp:55-127,195-247): page 0 is a permanent null page that is never
handed out; free pages are reused in the order they were given back; a request's table grows
page by page as its tokens arrive; a prompt's pages are *reserved* at admission and drawn from the
reservation as the prompt is computed; pages are given back in reverse order when the request
ends.  What is new: caches are sorted into *groups* by what they need (all positions, or a window
of them); each group has its own pool and its own table per request, and a windowed group gives a
page back as soon as the window has passed it; and beside the pages there are state slots, one
per request, for mixers that keep a state of fixed size.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Hashable, Iterable

import numpy as np

from ..config.errors import InvalidArgumentError, OutOfPagesError

NULL_PAGE = 0


@dataclass(frozen=True)
class PagedCacheSpec:
    """A cache that grows with the context: per position and head a key of ``key_dim`` values and a
    value of ``value_dim`` values (the reference keeps the two widths apart per layer,
    src/include/kv_cache/cache_engine.hpp:18-22).  ``value_dim`` 0 means "as wide as the key"."""

    num_kv_heads: int
    key_dim: int
    value_dim: int = 0
    window: int = 0        # 0: every position is kept; n: only the last n positions are ever read

    def __post_init__(self) -> None:
        if self.value_dim == 0:
            object.__setattr__(self, "value_dim", self.key_dim)

    @property
    def head_dim(self) -> int:
        """The one width of keys and values, for the kernels that need them equal."""
        if self.key_dim != self.value_dim:
            raise InvalidArgumentError(
                f"this cache keeps keys of {self.key_dim} and values of {self.value_dim} values: it has no single head size")
        return self.key_dim

    @property
    def group_key(self) -> tuple:
        return ("paged", self.num_kv_heads, self.key_dim, self.value_dim, self.window)


@dataclass(frozen=True)
class StateCacheSpec:
    """A cache of fixed size per request (a recurrent state, a running sum, ...)."""

    shape: tuple[int, ...]
    dtype: str = "float32"     # a torch dtype name; state usually stays in 32 bits


class PagePool:
    """Physical pages 1..num_pages-1 of one group (page 0 is the null page)."""

    def __init__(self, num_pages: int):
        if num_pages < 2:
            raise InvalidArgumentError("a page pool needs the null page and at least one usable page")
        self.num_pages = num_pages
        self._free: deque[int] = deque(range(1, num_pages))
        self._in_use = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_usable(self) -> int:
        return self.num_pages - 1

    def allocate(self, count: int) -> list[int]:
        """``count`` pages or none at all."""
        if count < 0:
            raise InvalidArgumentError("cannot allocate a negative number of pages")
        if count > len(self._free):
            raise OutOfPagesError(f"{count} pages wanted, {len(self._free)} free")
        pages = [self._free.popleft() for _ in range(count)]
        for page in pages:
            self._in_use[page] = True
        return pages

    def free(self, pages: Iterable[int]) -> None:
        for page in pages:
            if page == NULL_PAGE:
                continue
            if not 0 < page < self.num_pages or not self._in_use[page]:
                raise InvalidArgumentError(f"page {page} is given back but is not in use")
            self._in_use[page] = False
            self._free.append(page)

    def in_use(self, page: int) -> bool:
        return self._in_use[page]


class StateSlots:
    """Slots 0..n-1 for per-request state of fixed size."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free: deque[int] = deque(range(num_slots))
        self._in_use = [False] * num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def acquire(self) -> int:
        if not self._free:
            raise OutOfPagesError("no state slot is free")
        slot = self._free.popleft()
        self._in_use[slot] = True
        return slot

    def release(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._in_use[slot]:
            raise InvalidArgumentError(f"state slot {slot} is released but is not in use")
        self._in_use[slot] = False
        self._free.append(slot)


@dataclass
class GroupState:
    key: tuple
    window: int
    cache_ids: list[int]
    pool: PagePool


@dataclass
class _Request:
    slot: int
    tables: list[list[int]]                 # one block table per group; NULL_PAGE where a page was given back
    released_blocks: list[int]              # per group: blocks [0, n) were given back (window passed them)
    reserved: list[int]                     # per group: pages promised at admission, not yet drawn
    reserve_tokens: int = 0                 # the positions the promise was made for (the prompt)
    step_tokens: int = 1                    # the most positions a step brings, as promised at admission
    length: int = 0                         # positions covered by the tables
    computed: int = 0                       # positions whose entries have been written
    arrays: list = field(default_factory=list)   # the tables again as int32 arrays, grown in step with them


class CacheManager:
    """Pages and slots for all live requests.

    ``cache_specs[c]`` is what cache id ``c`` of the model needs (``PagedCacheSpec``,
    ``StateCacheSpec`` or ``None``).  Paged caches with equal needs share a group."""

    def __init__(self, cache_specs: list[PagedCacheSpec | StateCacheSpec | None], page_size: int, num_pages: int,
                 max_requests: int):
        if page_size <= 0 or page_size & (page_size - 1):
            raise InvalidArgumentError("the page size must be a power of two")
        if max_requests <= 0:
            raise InvalidArgumentError("max_requests must be positive")
        self.page_size = page_size
        self.max_requests = max_requests
        self.cache_specs = list(cache_specs)
        self.groups: list[GroupState] = []
        self.group_of_cache: dict[int, int] = {}
        by_key: dict[tuple, int] = {}
        for cache_id, spec in enumerate(self.cache_specs):
            if isinstance(spec, PagedCacheSpec):
                if spec.window < 0:
                    raise InvalidArgumentError("a window cannot be negative")
                if spec.group_key not in by_key:
                    by_key[spec.group_key] = len(self.groups)
                    self.groups.append(GroupState(spec.group_key, spec.window, [], PagePool(num_pages)))
                index = by_key[spec.group_key]
                self.groups[index].cache_ids.append(cache_id)
                self.group_of_cache[cache_id] = index
        self.state_cache_ids = [c for c, s in enumerate(self.cache_specs) if isinstance(s, StateCacheSpec)]
        self.slots = StateSlots(max_requests)
        self._requests: dict[Hashable, _Request] = {}

    # ----------------------------------------------------------------- queries
    def __contains__(self, request_id: Hashable) -> bool:
        return request_id in self._requests

    @property
    def num_requests(self) -> int:
        return len(self._requests)

    def blocks_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def _live_blocks_needed(self, group: GroupState, length: int, step_tokens: int) -> int:
        """Pages a request of ``length`` positions holds at most at one time in ``group``, when no step
        brings more than ``step_tokens`` new positions."""
        full = self.blocks_for(length)
        if group.window == 0:
            return full
        return min(full, self.blocks_for(group.window + step_tokens) + 1)

    def num_free_pages(self, group: int = 0) -> int:
        return self.groups[group].pool.num_free

    def num_unreserved_pages(self, group: int = 0) -> int:
        reserved = sum(r.reserved[group] for r in self._requests.values())
        return self.groups[group].pool.num_free - reserved

    def block_table(self, request_id: Hashable, group: int = 0) -> list[int]:
        return self._requests[request_id].tables[group]

    def block_table_array(self, request_id: Hashable, group: int = 0) -> np.ndarray:
        """The same table as an int32 array (a view that the next change of the table may move):
        what a step copies into its description without walking a Python list."""
        request = self._requests[request_id]
        return request.arrays[group][:len(request.tables[group])]

    def state_slot(self, request_id: Hashable) -> int:
        return self._requests[request_id].slot

    def length(self, request_id: Hashable) -> int:
        return self._requests[request_id].length

    def computed(self, request_id: Hashable) -> int:
        return self._requests[request_id].computed

    def fits_at_all(self, length: int, step_tokens: int) -> bool:
        """Could a request of ``length`` positions be held if it had the pool to itself?"""
        return all(self._live_blocks_needed(g, length, step_tokens) <= g.pool.num_usable for g in self.groups)

    # --------------------------------------------------------------- lifecycle
    def add_request(self, request_id: Hashable, reserve_tokens: int = 0, step_tokens: int = 1) -> bool:
        """Admit a request: take a state slot and reserve the pages ``reserve_tokens`` positions need
        (the whole prompt, as the reference does at admission).  Returns False, changing nothing, if
        the slot or the pages are not to be had."""
        if request_id in self._requests:
            raise InvalidArgumentError(f"request {request_id!r} is already in the cache manager")
        if self.slots.num_free == 0:
            return False
        wanted = [self._live_blocks_needed(g, reserve_tokens, step_tokens) for g in self.groups]
        for index, count in enumerate(wanted):
            if count > self.num_unreserved_pages(index):
                return False
        self._requests[request_id] = _Request(
            slot=self.slots.acquire(), tables=[[] for _ in self.groups],
            released_blocks=[0 for _ in self.groups], reserved=wanted, reserve_tokens=reserve_tokens,
            step_tokens=step_tokens,
            arrays=[np.zeros(16, dtype=np.int32) for _ in self.groups])
        return True

    def ensure_capacity(self, request_id: Hashable, length: int) -> bool:
        """Make the request's tables cover positions [0, length).  All groups or none: returns False,
        changing nothing, when some group lacks the pages."""
        request = self._requests[request_id]
        if length <= request.length:
            return True
        needs = []
        for index, group in enumerate(self.groups):
            extra = self.blocks_for(length) - len(request.tables[index])
            # Pages promised to other requests are not this request's to take; its own promise is.
            others_reserved = sum(r.reserved[index] for r in self._requests.values()) - request.reserved[index]
            if extra > group.pool.num_free - others_reserved:
                return False
            needs.append((extra, min(extra, request.reserved[index])))
        for index, (extra, from_reservation) in enumerate(needs):
            if extra > 0:
                table = request.tables[index]
                have = len(table)
                table.extend(self.groups[index].pool.allocate(extra))
                if len(table) > request.arrays[index].size:
                    grown = np.zeros(max(len(table), 2 * request.arrays[index].size), dtype=np.int32)
                    grown[:have] = request.arrays[index][:have]
                    request.arrays[index] = grown
                request.arrays[index][have:len(table)] = table[have:]
                request.reserved[index] -= from_reservation
        request.length = length
        return True

    def commit(self, request_id: Hashable, computed: int) -> None:
        """Record that positions [0, computed) are written, and give back the pages of windowed
        groups that no later query can see: a query at position p >= computed reads keys
        > p - window, so block b is dead once (b + 1) * page_size <= computed - window + 1."""
        request = self._requests[request_id]
        if computed > request.length:
            raise InvalidArgumentError("cannot commit positions the tables do not cover")
        request.computed = max(request.computed, computed)
        for index, group in enumerate(self.groups):
            if group.window == 0:
                continue
            dead = max(0, (request.computed - group.window + 1) // self.page_size)
            dead = min(dead, len(request.tables[index]))
            if dead > request.released_blocks[index]:
                table = request.tables[index]
                group.pool.free(table[request.released_blocks[index]:dead])
                for block in range(request.released_blocks[index], dead):
                    table[block] = NULL_PAGE
                request.arrays[index][request.released_blocks[index]:dead] = NULL_PAGE
                given_back = dead - request.released_blocks[index]
                request.released_blocks[index] = dead
                # While its prompt is still being computed the request keeps its claim at what it will
                # hold at one time: the pages it has just given back stay promised to it, as far as it
                # still needs them, so that newcomers admitted meanwhile cannot starve it.
                if request.computed < request.reserve_tokens:
                    bound = self._live_blocks_needed(group, request.reserve_tokens, request.step_tokens)
                    to_come = self.blocks_for(request.reserve_tokens) - len(table)
                    wanted = min(to_come, max(0, bound - (len(table) - dead)))
                    if wanted > request.reserved[index]:
                        request.reserved[index] = min(wanted, request.reserved[index] + given_back)

    def free_request(self, request_id: Hashable) -> None:
        """Give back everything the request holds: pages last-to-first, reservation, state slot."""
        request = self._requests.pop(request_id)
        for index, group in enumerate(self.groups):
            group.pool.free(reversed(request.tables[index]))
        self.slots.release(request.slot)

    # -------------------------------------------------------------- invariants
    def check_invariants(self) -> None:
        """No page lost, none held twice, none both free and held.  Raises AssertionError."""
        for request in self._requests.values():
            for table, array in zip(request.tables, request.arrays):
                assert array[:len(table)].tolist() == table, "a table's array copy has drifted from the table"
        for index, group in enumerate(self.groups):
            held: dict[int, Hashable] = {}
            for request_id, request in self._requests.items():
                table = request.tables[index]
                assert len(table) == self.blocks_for(request.length), "table length does not match the positions"
                for block, page in enumerate(table):
                    if page == NULL_PAGE:
                        assert group.window > 0 and block < request.released_blocks[index], "hole in a table"
                        continue
                    assert 0 < page < group.pool.num_pages, f"page {page} out of range"
                    assert page not in held, f"page {page} held by {held[page]!r} and {request_id!r}"
                    assert group.pool.in_use(page), f"page {page} is in a table but marked free"
                    held[page] = request_id
                assert request.reserved[index] >= 0
            free = list(group.pool._free)
            assert len(set(free)) == len(free), "a page is in the free list twice"
            assert not set(free) & set(held), "a page is both free and held"
            assert len(free) + len(held) == group.pool.num_usable, "a page was lost"
        slots = [r.slot for r in self._requests.values()]
        assert len(set(slots)) == len(slots), "a state slot is held twice"
        assert len(slots) + self.slots.num_free == self.slots.num_slots, "a state slot was lost"
