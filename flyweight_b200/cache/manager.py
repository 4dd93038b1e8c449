"""The cache manager: pages of keys and values with a block table for each request,
and slots for per-request state of fixed size.

Layout (flyweight's own paged contract, native/src/paged_kv.h:48-83: 64-token pages,
page-major): every execution of a mixer that keeps keys and values owns two pools
``[num_pages][kv_heads][64][head_dim]``; one (page, KV head) tile is one contiguous
64 x head_dim block.

Executions are sorted into *groups* by what they need to keep: all keys (window 0) or
only the last ``window`` keys.  Each group has its own page pool and its own block
table per request; inside a group the same page id indexes every member's pools, since
members grow in step.  A request's pages go back to the pool when it ends, and in a
window group also as soon as the window has passed them.

Fixed-size state (the short convolution's rolling inputs here; any recurrent state in
general) lives in *slots*: every such execution owns one ``[num_slots][...]`` tensor in the
dtype its spec names (fp32 by default), and a request holds one slot id, zeroed when it is handed out, for as long as
it lives (flyweight zeroes the whole arena on reset, native/src/v2_runtime.cpp:20438-20440).

All bookkeeping is host-side and can be tested without a GPU (``device=None`` makes
no device tensors).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import FixedState, PagedKV

PAGE_SIZE = 64


class OutOfPages(RuntimeError):
    """A group's pool cannot give the pages a step needs."""


class OutOfSlots(RuntimeError):
    """Every state slot is held by a live request."""


class PagePool:
    """Page ids 0..n-1 with a LIFO free list (native/src/paged_kv.h:133-160); a page is
    never handed out twice and never taken back twice."""

    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise ValueError("num_pages must not be negative")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._held = [False] * num_pages
        self.high_water = 0

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_used(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        page = self._free.pop()
        assert not self._held[page], f"page {page} handed out twice"
        self._held[page] = True
        self.high_water = max(self.high_water, self.n_used)
        return page

    def release(self, page: int) -> None:
        if not 0 <= page < self.num_pages or not self._held[page]:
            raise RuntimeError(f"page {page} released but not held")
        self._held[page] = False
        self._free.append(page)

    def check(self) -> None:
        """Every page is either free or held, exactly once."""
        assert len(set(self._free)) == len(self._free), "a page is on the free list twice"
        for page in self._free:
            assert not self._held[page], f"page {page} is free and held"
        assert sum(self._held) + len(self._free) == self.num_pages, "a page was lost"


@dataclass
class LayerCache:
    """What one execution of a mixer gets from the manager."""
    group: Optional[int] = None              # index of its page group (block table to use)
    k_pool: Optional[torch.Tensor] = None
    v_pool: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None     # [num_slots][...] in the spec's dtype (fp32 by default)
    spec: object = None


@dataclass
class PageGroup:
    window: int                               # 0: keep every key
    pool: PagePool
    members: List[int] = field(default_factory=list)      # schedule positions
    tables: Dict[Hashable, List[int]] = field(default_factory=dict)   # logical page -> id or -1

    def first_needed_page(self, length: int) -> int:
        """Lowest logical page a query at position ``length`` (the next one) still reads."""
        if self.window <= 0:
            return 0
        first_key = max(0, length - self.window + 1)
        return first_key // PAGE_SIZE


class CacheManager:
    def __init__(self, state_specs: Sequence[object], num_pages: int, num_slots: int,
                 cache_dtype: torch.dtype = torch.float32, device=None):
        """``state_specs[i]`` is what schedule position i keeps: ``PagedKV``, ``FixedState``
        or ``None``.  ``num_pages`` pages per group, ``num_slots`` live requests at most."""
        self.num_pages = int(num_pages)
        self.num_slots = int(num_slots)
        self.device = device
        self.cache_dtype = cache_dtype
        self.groups: List[PageGroup] = []
        self.layer_caches: List[LayerCache] = []
        self._free_slots: List[int] = list(range(num_slots - 1, -1, -1))
        self._slot_of: Dict[Hashable, int] = {}
        self._length: Dict[Hashable, int] = {}
        self._fixed_positions: List[int] = []
        self._serial: Dict[Hashable, int] = {}
        self._admissions = 0
        self.slots_high_water = 0
        by_window: Dict[int, int] = {}
        for position, spec in enumerate(state_specs):
            cache = LayerCache(spec=spec)
            if isinstance(spec, PagedKV):
                if spec.window not in by_window:
                    by_window[spec.window] = len(self.groups)
                    self.groups.append(PageGroup(spec.window, PagePool(self.num_pages)))
                cache.group = by_window[spec.window]
                self.groups[cache.group].members.append(position)
                if device is not None:
                    shape = (self.num_pages, spec.n_kv_heads, PAGE_SIZE, spec.head_dim)
                    cache.k_pool = torch.zeros(shape, dtype=cache_dtype, device=device)
                    cache.v_pool = torch.zeros(shape, dtype=cache_dtype, device=device)
            elif isinstance(spec, FixedState):
                self._fixed_positions.append(position)
            elif spec is not None:
                raise TypeError(f"schedule position {position}: unknown state spec {spec!r}")
            self.layer_caches.append(cache)
        self._windowed = any(group.window for group in self.groups)
        self._rows: List[Dict[Hashable, tuple]] = [{} for _ in self.groups]   # block-table rows as arrays
        # All fixed-size states of one dtype lie side by side in one allocation, [num_slots][total],
        # and every execution sees its share as [num_slots][...]: admission clears one span per dtype.
        self._all_states: Dict[torch.dtype, torch.Tensor] = {}
        if device is not None and self._fixed_positions:
            by_dtype: Dict[torch.dtype, List[Tuple[int, int]]] = {}
            for position in self._fixed_positions:
                spec = self.layer_caches[position].spec
                count = 1
                for extent in spec.shape:
                    count *= int(extent)
                by_dtype.setdefault(spec.dtype, []).append((position, count))
            for dtype, members in by_dtype.items():
                pool = torch.zeros((self.num_slots, sum(count for _, count in members)), dtype=dtype,
                                   device=device)
                self._all_states[dtype] = pool
                offset = 0
                for position, count in members:
                    shape = tuple(self.layer_caches[position].spec.shape)
                    self.layer_caches[position].state = (
                        pool[:, offset:offset + count].unflatten(1, shape) if shape else pool[:, offset])
                    offset += count

    # ------------------------------------------------------------------ requests
    def live(self) -> Tuple[Hashable, ...]:
        return tuple(self._slot_of)

    def has(self, request: Hashable) -> bool:
        return request in self._slot_of

    def length(self, request: Hashable) -> int:
        return self._length[request]

    def slot(self, request: Hashable) -> int:
        return self._slot_of[request]

    def serial(self, request: Hashable) -> int:
        """A number that is new for every admission (a name may come back after a release)."""
        return self._serial[request]

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def admit(self, request: Hashable) -> int:
        """Give ``request`` a zeroed state slot and empty block tables."""
        if request in self._slot_of:
            raise RuntimeError(f"request {request!r} is already live")
        if not self._free_slots:
            raise OutOfSlots(f"all {self.num_slots} state slots are held")
        slot = self._free_slots.pop()
        self._slot_of[request] = slot
        self._length[request] = 0
        self._admissions += 1
        self._serial[request] = self._admissions
        self.slots_high_water = max(self.slots_high_water, len(self._slot_of))
        for group in self.groups:
            group.tables[request] = []
        for pool in self._all_states.values():
            pool[slot].zero_()
        return slot

    def release_passed(self, request: Hashable) -> int:
        """Give back the pages of ``request`` that a window has passed for good: no query
        at the request's next position or later reads them.  Returns how many."""
        count = 0
        for group in self.groups:
            table = group.tables[request]
            first = group.first_needed_page(self._length[request])
            for logical in range(min(first, len(table))):
                if table[logical] >= 0:
                    group.pool.release(table[logical])
                    table[logical] = -1
                    count += 1
        return count

    def pages_needed(self, request: Optional[Hashable], new_length: int) -> List[int]:
        """New pages per group to hold ``new_length`` tokens of ``request`` (None: a
        request that is not admitted yet)."""
        needs = []
        for group in self.groups:
            have = len(group.tables[request]) if request in self._slot_of else 0
            needs.append(max(0, -(-new_length // PAGE_SIZE) - have))
        return needs

    def pages_short(self, request: Hashable, new_length: int) -> int:
        """How many pages are lacking, over all groups, to hold ``new_length`` tokens of
        ``request`` (0: it fits)."""
        if request in self._slot_of:
            self.release_passed(request)
        return sum(max(0, need - group.pool.n_free)
                   for need, group in zip(self.pages_needed(request, new_length), self.groups))

    def extend(self, request: Hashable, new_length: int, checked: bool = False) -> None:
        """Map pages so positions < ``new_length`` of ``request`` have a home.  Raises
        ``OutOfPages`` and maps nothing if some group cannot.  ``checked``: the caller has
        already made sure that the pages are there (the step function checks a whole step)."""
        if new_length < self._length[request]:
            raise ValueError("a request's length never shrinks")
        if not checked:
            short = self.pages_short(request, new_length)
            if short:
                raise OutOfPages(f"request {request!r} needs {short} more pages than are free")
        for group in self.groups:
            table = group.tables[request]
            while len(table) * PAGE_SIZE < new_length:
                table.append(group.pool.allocate())
        self._length[request] = new_length

    def room_for_one_more(self, requests: Sequence[Hashable], width: int) -> bool:
        """Whether every one of these live requests can take one more token now: those at a page's
        edge find a free page in every group (all of them together), and no block table grows past
        ``width`` pages.  Nothing is changed."""
        at_edge = 0
        for request in requests:
            length = self._length[request]
            if length % PAGE_SIZE == 0:
                at_edge += 1
                if length // PAGE_SIZE + 1 > width:
                    return False
        # (pages that a window passes with this token are not counted as free: on the safe side)
        return not at_edge or all(group.pool.n_free >= at_edge for group in self.groups)

    def fits_last_page(self, request: Hashable) -> bool:
        """Whether one more token of a live ``request`` needs no new page in any group and gives
        none back: its next position lies inside its last mapped page, and no group has a window
        (the short way for the hundreds of one-token entries of a decode step)."""
        return not self._windowed and self._length[request] % PAGE_SIZE != 0

    def grow(self, request: Hashable, count: int) -> Tuple[int, int]:
        """``extend`` by ``count`` tokens for a caller that has checked the pages; returns the
        request's state slot and its length before."""
        length = self._length[request]
        new_length = length + count
        if count != 1 or length % PAGE_SIZE == 0:
            for group in self.groups:
                table = group.tables[request]
                while len(table) * PAGE_SIZE < new_length:
                    table.append(group.pool.allocate())
        self._length[request] = new_length
        return self._slot_of[request], length

    def advance_one(self, request: Hashable) -> bool:
        """One more token of a live ``request`` whose caller has asked ``room_for_one_more``: the
        pages a window has passed are given back, a request at a page's edge gets its next page in
        every group.  True if one of its block tables changed."""
        changed = self._windowed and self.release_passed(request) > 0
        length = self._length[request]
        if length % PAGE_SIZE == 0:
            for group in self.groups:
                group.tables[request].append(group.pool.allocate())
            changed = True
        self._length[request] = length + 1
        return changed

    def bump(self, request: Hashable) -> None:
        """One more token of ``request`` inside its last mapped page (the caller has checked)."""
        length = self._length[request]
        if length % PAGE_SIZE == 0:
            raise OutOfPages(f"request {request!r} needs a new page for position {length}")
        self._length[request] = length + 1

    def release(self, request: Hashable) -> None:
        """Give back everything ``request`` holds."""
        slot = self._slot_of.pop(request)
        del self._length[request]
        del self._serial[request]
        for index, group in enumerate(self.groups):
            for page in group.tables.pop(request):
                if page >= 0:
                    group.pool.release(page)
            self._rows[index].pop(request, None)
        self._free_slots.append(slot)

    def reset(self) -> None:
        for request in list(self._slot_of):
            self.release(request)

    # ------------------------------------------------------------------ views for a step
    def block_table(self, group_index: int, requests: Sequence[Hashable], width: int
                    ) -> List[List[int]]:
        """Rows of page ids (``-1`` where nothing is mapped), padded to ``width``."""
        group = self.groups[group_index]
        rows = []
        for request in requests:
            table = group.tables[request]
            if len(table) > width:
                raise ValueError("block table wider than the step's width")
            rows.append(table + [-1] * (width - len(table)))
        return rows

    def block_table_array(self, group_index: int, requests: Sequence[Hashable], width: int) -> np.ndarray:
        """The same rows as one int32 array [requests][width].  A request's row is kept as an
        array between steps and made again only when its table changed (a table grows by a page
        every 64 tokens), so a step with many decoding requests does not walk their lists."""
        group = self.groups[group_index]
        out = np.full((len(requests), width), -1, dtype=np.int32)
        kept = self._rows[group_index]
        for index, request in enumerate(requests):
            table = group.tables[request]
            stamp = (self._serial[request], len(table),
                     sum(1 for page in table if page < 0) if group.window else 0)
            entry = kept.get(request)
            if entry is None or entry[0] != stamp:
                entry = kept[request] = (stamp, np.asarray(table, dtype=np.int32))
            row = entry[1]
            if row.size > width:
                raise ValueError("block table wider than the step's width")
            out[index, :row.size] = row
        return out

    def max_table_len(self, requests: Sequence[Hashable]) -> int:
        width = 1
        for group in self.groups:
            for request in requests:
                width = max(width, len(group.tables[request]))
        return width

    # ------------------------------------------------------------------ accounting
    def stats(self) -> dict:
        return {
            "page_size": PAGE_SIZE,
            "groups": [{"window": g.window, "layers": len(g.members), "pages": g.pool.num_pages,
                        "pages_in_use": g.pool.n_used, "pages_high_water": g.pool.high_water}
                       for g in self.groups],
            "slots": self.num_slots, "slots_in_use": len(self._slot_of),
            "slots_high_water": self.slots_high_water,
        }

    def check(self) -> None:
        """Invariants: no page lost, held twice or freed twice; no slot shared."""
        for group in self.groups:
            group.pool.check()
            seen = set()
            for table in group.tables.values():
                for page in table:
                    if page >= 0:
                        assert page not in seen, f"page {page} is in two block tables"
                        seen.add(page)
            assert len(seen) == group.pool.n_used, "held pages and block tables disagree"
        slots = list(self._slot_of.values())
        assert len(set(slots)) == len(slots), "a slot is held twice"
        assert len(slots) + len(self._free_slots) == self.num_slots, "a slot was lost"
        assert not set(slots) & set(self._free_slots), "a slot is free and held"
