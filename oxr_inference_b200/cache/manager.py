"""The cache manager: pages of keys and values with a block table per request, and per-request state slots.

Host side (always): free lists, block tables, which pages a request needs for its next tokens, which pages a
window has passed. Device side (when given a device): one K pool and one V pool per group,
``[layers of the group, pages, page_size, KV, D]`` as in the reference (oxr_runtime/kv_cache.py:27-29) but with
the page size an argument, and one ``[slots, *shape]`` tensor per kind of per-request state.

A request's life: ``open`` (takes a state slot) -> any number of ``reserve(new_length)`` / step /
``advance(new_length)`` -> ``close`` (gives everything back). ``reserve`` is all-or-nothing over all groups.
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass, field

import numpy as np
import torch

from oxr_inference_b200.cache.pages import PagePool
from oxr_inference_b200.cache.plan import CachePlan
from oxr_inference_b200.parts.base import GroupView, LayerCache, StepContext

RELEASED = -1
"""Block-table entry of a page that a window has passed."""


@dataclass
class RequestCache:
    key: object
    state_slot: int
    length: int = 0
    """Tokens whose keys and values are in the cache."""
    tables: list[list[int]] = field(default_factory=list)
    """Per group: page id of each page-sized stretch of positions; RELEASED behind a window."""
    closed: bool = False
    version: int = 0
    """Changes whenever ``tables`` changes (pages added or released), so that a copy of a table row can be reused."""
    room: int = 0
    """Tokens that the pages held so far can take (the shortest table times the page size): lets the two calls that every
    request makes in every step, ``reserve`` and ``advance``, answer the common case with one comparison."""
    released: list[int] = field(default_factory=list)
    """Per group: how many pages at the front of the table a window has passed and given back."""
    serial: int = field(default_factory=itertools.count().__next__)
    """Unlike ``id()``, never given to a second request of this process: (serial, version) names one state of one
    request's tables for good."""


def pages_for(tokens: int, page_size: int) -> int:
    """Pages that hold ``tokens`` tokens (oxr_runtime/kv_cache.py:55-57)."""
    return (tokens + page_size - 1) // page_size


class CacheManager:
    def __init__(self, plan: CachePlan, *, page_size: int, num_pages: int, max_requests: int,
                 device: torch.device | None = None, dtype: torch.dtype | None = None, scratch: bool = True):
        if page_size <= 0 or num_pages <= 0 or max_requests <= 0:
            raise ValueError("page_size, num_pages and max_requests must be positive")
        self.plan, self.page_size, self.num_pages, self.max_requests = plan, page_size, num_pages, max_requests
        self.pools = [PagePool(num_pages) for _ in plan.groups]
        self.windows = [g.need.window for g in plan.groups]
        self._windowed = [g for g, w in enumerate(self.windows) if w > 0]
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self._open: dict[int, RequestCache] = {}
        self.scratch_slot = max_requests
        """State slot that rows added as padding use."""
        self.scratch_pages: list[int] = []
        """Per group, a page never given to a request: padding rows write and read there
        (oxr_runtime/decode_graph.py:44-48)."""
        if scratch:
            for pool in self.pools:
                got = pool.allocate(1)
                if got is None:
                    raise ValueError("the cache cannot spare one scratch page")
                self.scratch_pages.append(got[0])

        self.device, self.dtype = device, dtype
        self.k_pools: list[torch.Tensor] = []
        self.v_pools: list[torch.Tensor] = []
        self.states: list[torch.Tensor] = []
        if device is not None:
            for g in plan.groups:
                shape = (g.num_layers, num_pages, page_size, g.need.num_kv_heads, g.need.head_dim)
                self.k_pools.append(torch.zeros(shape, dtype=dtype, device=device))
                self.v_pools.append(torch.zeros(shape, dtype=dtype, device=device))
            for s in plan.states:
                self.states.append(torch.zeros((max_requests + 1, *s.shape), dtype=s.dtype, device=device))
        self.kv_maps: list = [None] * len(self.k_pools)
        if device is not None and torch.device(device).type == "cuda":
            from oxr_inference_b200 import ops

            self.kv_maps = [ops.make_kv_maps(k, v, page_size) for k, v in zip(self.k_pools, self.v_pools)]

    # ---- sizes
    @staticmethod
    def bytes_per_page(plan: CachePlan, page_size: int, dtype: torch.dtype) -> int:
        """Bytes of one page id over all groups and layers (oxr_runtime/kv_cache.py:34-37)."""
        element = torch.empty((), dtype=dtype).element_size()
        return sum(2 * g.num_layers * page_size * g.need.num_kv_heads * g.need.head_dim * element for g in plan.groups)

    @property
    def free_pages(self) -> int:
        """Pages free in the fullest group."""
        return min((p.free for p in self.pools), default=self.num_pages)

    @property
    def usable_pages(self) -> int:
        return self.num_pages - (1 if self.scratch_pages else 0)

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    # ---- requests
    def open(self, key: object = None) -> RequestCache | None:
        """Start a request: takes a state slot (zeroed on the device); None when all slots are taken."""
        if not self._free_slots:
            return None
        slot = self._free_slots.pop()
        rc = RequestCache(key=key, state_slot=slot, tables=[[] for _ in self.pools], released=[0] * len(self.pools))
        self._open[id(rc)] = rc
        for state in self.states:
            state[slot].zero_()
        return rc

    def _first_needed_page(self, group: int, start: int) -> int:
        """Index of the first page that a query at position ``start`` or later can still see."""
        w = self.windows[group]
        return 0 if w <= 0 else max(0, start - w + 1) // self.page_size

    def reserve(self, rc: RequestCache, new_length: int) -> bool:
        """Make room for the tokens at positions [rc.length, new_length). False, with nothing taken, if any
        group lacks the pages."""
        if rc.closed:
            raise ValueError("the request was closed")
        if new_length < rc.length:
            raise ValueError(f"a request cannot shrink ({rc.length} -> {new_length})")
        if new_length <= rc.room:
            return True   # the pages are there already (the common case while decoding)
        want = pages_for(new_length, self.page_size)
        needed = [max(0, want - len(table)) for table in rc.tables]
        if any(n > pool.free for n, pool in zip(needed, self.pools)):
            return False
        for table, pool, n in zip(rc.tables, self.pools, needed):
            table.extend(pool.allocate(n))
        rc.room = min(len(table) for table in rc.tables) * self.page_size
        rc.version += 1
        return True

    def advance(self, rc: RequestCache, new_length: int) -> None:
        """The step ran: the request now holds ``new_length`` tokens. Pages that every later query's window has
        passed are given back."""
        if new_length < rc.length or new_length > rc.room:
            raise ValueError("advance beyond what was reserved")
        rc.length = new_length
        for g in self._windowed:
            table, pool = rc.tables[g], self.pools[g]
            keep_from = min(self._first_needed_page(g, new_length), len(table))  # the next query sits at position new_length
            done = rc.released[g]
            if keep_from > done:   # the pages given back are a prefix of the table: only what is new is touched
                pool.release(table[done:keep_from])
                table[done:keep_from] = [RELEASED] * (keep_from - done)
                rc.released[g] = keep_from
                rc.version += 1

    def close(self, rc: RequestCache) -> None:
        """Give back every page and the state slot (finish, cancel, preemption, error:
        oxr_runtime/engine.py:747-749,472-475,623-625,459-461)."""
        if rc.closed:
            raise ValueError("the request is closed twice")
        for table, pool in zip(rc.tables, self.pools):
            pool.release([p for p in table if p != RELEASED])
            table.clear()
        self._free_slots.append(rc.state_slot)
        rc.closed = True
        rc.version += 1
        rc.length = 0
        rc.room = 0
        rc.released = [0] * len(self.pools)
        del self._open[id(rc)]

    def open_requests(self) -> list[RequestCache]:
        return list(self._open.values())

    def check(self) -> None:
        """Every page is free, scratch, or held by exactly one open request; likewise every slot."""
        for g, pool in enumerate(self.pools):
            owners: dict[int, int] = {}
            if self.scratch_pages:
                owners[self.scratch_pages[g]] = 1
            for rc in self._open.values():
                for p in rc.tables[g]:
                    if p != RELEASED:
                        owners[p] = owners.get(p, 0) + 1
            twice = [p for p, c in owners.items() if c > 1]
            if twice:
                raise AssertionError(f"group {g}: pages {twice} are held twice")
            held = set(pool.held())
            if held != set(owners):
                raise AssertionError(f"group {g}: pool says {sorted(held)} are held, tables say {sorted(owners)}")
            if len(held) + pool.free != pool.num_pages:
                raise AssertionError(f"group {g}: {len(held)} held + {pool.free} free != {pool.num_pages}")
        for rc in self._open.values():
            if rc.room != min(len(t) for t in rc.tables) * self.page_size:
                raise AssertionError(f"request {rc.key!r}: room {rc.room} does not match its tables")
            for g, table in enumerate(rc.tables):
                k = rc.released[g]
                if any(p != RELEASED for p in table[:k]) or any(p == RELEASED for p in table[k:]):
                    raise AssertionError(f"request {rc.key!r}, group {g}: the released pages are not the first {k}")
        slots = [rc.state_slot for rc in self._open.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise AssertionError("a state slot is held twice or is both held and free")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise AssertionError("a state slot was lost")

    # ---- what a step needs
    def slots(self, rc: RequestCache, group: int, start: int, end: int) -> np.ndarray:
        """Cache slot (page * page_size + offset) of each position in [start, end)
        (oxr_runtime/language.py:320-322)."""
        pos = np.arange(start, end, dtype=np.int64)
        table = np.asarray(rc.tables[group], dtype=np.int64)
        pages = table[pos // self.page_size]
        if (pages < 0).any():
            raise ValueError("a position to be written lies on a released page")
        return (pages * self.page_size + pos % self.page_size).astype(np.int32)

    def slot(self, rc: RequestCache, group: int, position: int) -> int:
        """Cache slot of one position (the single-token case of :meth:`slots`, without numpy)."""
        page = rc.tables[group][position // self.page_size]
        if page < 0:
            raise ValueError("a position to be written lies on a released page")
        return page * self.page_size + position % self.page_size

    def table_width(self, rcs: list[RequestCache], group: int) -> int:
        return max([len(rc.tables[group]) for rc in rcs] + [1])

    def layer_cache(self, schedule_pos: int, ctx: StepContext) -> LayerCache:
        e = self.plan.entries[schedule_pos]
        return LayerCache(
            group=ctx.groups[e.group] if e.group is not None else None,
            layer_in_group=e.layer_in_group,
            store=e.store,
            state=self.states[e.state] if e.state is not None else None,
        )

    def group_view(self, group: int, block_table: torch.Tensor, slots: torch.Tensor) -> GroupView:
        return GroupView(self.page_size, self.k_pools[group] if self.k_pools else None,
                         self.v_pools[group] if self.v_pools else None, block_table, slots,
                         self.kv_maps[group] if self.k_pools else None)
