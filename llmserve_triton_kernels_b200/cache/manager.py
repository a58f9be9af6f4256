"""The cache manager: pages of keys and values with a table per request, and slots of state.

Parity: src/llmserve/kvcache/paged.py:113-218 (a pool of pages shared by all layers of a kind, a
table of page ids and a length per sequence, atomic reservation before a forward pass, pages
given back when the sequence ends) with two additions the reference has no use for:

* groups: the entries of the model's order are grouped by what they keep (``PagedKVSpec``:
  key/value heads, head size, window).  Each group has its own pool, allocator and tables;
  a group with a window gives a page back as soon as every key in it is older than the window
  of the next query.
* state slots: every request holds one slot id; an entry whose mixer keeps a ``StateSpec``
  has a tensor ``[slots, *shape]`` indexed by it, zeroed when the request starts.

Reservation and commit are separate: ``reserve`` finds pages for the new tokens of a whole
step or raises ``OutOfPages`` with nothing changed; ``commit`` advances the lengths once the
step has run and releases what the windows have passed.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..parts.base import PagedKVSpec, StateSpec
from .allocator import IdAllocator, OutOfPages

RELEASED = -1  # table entry of a page that a window has passed


@dataclass
class PagedKVView:
    """What an attention layer sees of its cache in one step."""

    pool: torch.Tensor  # [pages, 2, kv_heads, page_size, head_dim]: this entry's plane
    page_table: torch.Tensor  # [requests, width] int32, physical page of each logical page
    slot_map: torch.Tensor  # [tokens] int32: page * page_size + offset of each new token
    page_size: int
    spec: PagedKVSpec


@dataclass
class StateView:
    """What a mixer with fixed-size state sees: ``states[slots[r]]`` belongs to request r."""

    states: torch.Tensor  # [slots, *shape]
    slots: torch.Tensor  # [requests] int32 (device)
    host_slots: list[int]


class PageGroup:
    def __init__(self, spec: PagedKVSpec, entries: list[int], num_pages: int, page_size: int, dtype, device):
        self.spec = spec
        self.entries = entries  # positions in the model's order that own a plane here
        self.num_pages = int(num_pages)
        self.page_size = int(page_size)
        self.pool = torch.zeros(
            (len(entries), self.num_pages, 2, spec.kv_heads, self.page_size, spec.head_dim),
            dtype=dtype,
            device=device,
        )
        self.allocator = IdAllocator(self.num_pages, "page")
        self.tables: dict[object, list[int]] = {}
        # the same tables as int32 arrays with room to grow (released pages as 0), so that a step's table is put
        # together from slices, not from Python lists
        self._rows: dict[object, np.ndarray] = {}

    def new_table(self, req) -> None:
        self.tables[req] = []
        self._rows[req] = np.zeros(16, dtype=np.int32)

    def drop_table(self, req) -> list[int]:
        del self._rows[req]
        return self.tables.pop(req)

    def append_page(self, req, page: int) -> None:
        table = self.tables[req]
        row = self._rows[req]
        if len(table) == row.shape[0]:
            row = self._rows[req] = np.concatenate((row, np.zeros_like(row)))
        row[len(table)] = page
        table.append(page)

    def release_page(self, req, index: int) -> None:
        self.tables[req][index] = RELEASED
        self._rows[req][index] = 0

    def row(self, req) -> np.ndarray:
        """The request's table as int32 (released pages read 0); a view, not to be written."""
        return self._rows[req][: len(self.tables[req])]

    def first_needed_page(self, length: int) -> int:
        """Logical index of the first page that a query at position ``length`` or later reads."""
        if self.spec.window is None:
            return 0
        return max(0, length - self.spec.window + 1) // self.page_size

    def extra_pages(self, req, length: int, new_tokens: int) -> int:
        table = self.tables[req]
        last = (length + new_tokens - 1) // self.page_size
        return max(0, last + 1 - len(table))

    def bytes_per_page(self) -> int:
        return len(self.entries) * 2 * self.spec.kv_heads * self.page_size * self.spec.head_dim * self.pool.element_size()


class CacheManager:
    def __init__(
        self,
        cache_specs: list,
        schedule,
        *,
        page_size: int,
        num_pages: int,
        max_requests: int,
        dtype: torch.dtype,
        device: torch.device | str,
    ):
        if page_size < 1:
            raise ValueError(f"page_size must be positive, got {page_size}")
        self.page_size = int(page_size)
        self.num_pages = int(num_pages)
        self.max_requests = int(max_requests)
        self.device = torch.device(device)
        self.dtype = dtype
        self.schedule = list(schedule)
        self.groups: list[PageGroup] = []
        self._entry_group: dict[int, tuple[int, int]] = {}  # order entry -> (group, plane)
        by_spec: dict[PagedKVSpec, list[int]] = {}
        self._state_entries: dict[int, torch.Tensor] = {}
        for i, spec in enumerate(cache_specs):
            if isinstance(spec, PagedKVSpec):
                by_spec.setdefault(spec, []).append(i)
            elif isinstance(spec, StateSpec):
                self._state_entries[i] = torch.zeros(
                    (self.max_requests, *spec.shape), dtype=spec.dtype, device=self.device
                )
            elif spec is not None:
                raise TypeError(f"entry {i} of the order has an unknown cache spec {spec!r}")
        for g, (spec, entries) in enumerate(by_spec.items()):
            self.groups.append(PageGroup(spec, entries, self.num_pages, self.page_size, dtype, self.device))
            for plane, i in enumerate(entries):
                self._entry_group[i] = (g, plane)
        self.slots = IdAllocator(self.max_requests, "state slot")
        self.lengths: dict[object, int] = {}
        self.slot_of: dict[object, int] = {}

    # ------------------------------------------------------------------ sizes
    def pages_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def peak_pages_for(self, tokens: int, chunk: int) -> int:
        """The most pages of one group that a request of ``tokens`` tokens ever holds when it
        is fed in portions of at most ``chunk`` tokens."""
        need = 0
        for g in self.groups:
            if g.spec.window is None:
                need = max(need, self.pages_for(tokens))
            else:
                need = max(need, min(self.pages_for(tokens), self.pages_for(g.spec.window + chunk) + 1))
        return need

    @property
    def num_free_pages(self) -> int:
        """Free pages of the tightest group (what admission looks at)."""
        return min((g.allocator.num_free for g in self.groups), default=self.num_pages)

    def utilization(self) -> float:
        if not self.groups or not self.num_pages:
            return 0.0
        return max(g.allocator.num_used for g in self.groups) / self.num_pages

    def internal_fragmentation(self) -> float:
        """Share of held token places that hold no token (tails of last pages), over groups that keep all keys."""
        held = sum(g.allocator.num_used for g in self.groups if g.spec.window is None) * self.page_size
        if held == 0:
            return 0.0
        used = sum(self.lengths.values()) * sum(1 for g in self.groups if g.spec.window is None)
        return 1.0 - used / held

    def nbytes(self) -> int:
        total = sum(g.pool.numel() * g.pool.element_size() for g in self.groups)
        return total + sum(t.numel() * t.element_size() for t in self._state_entries.values())

    # ------------------------------------------------------------------ lifecycle
    def has_request(self, req) -> bool:
        return req in self.lengths

    def add_request(self, req) -> None:
        if req in self.lengths:
            raise ValueError(f"request {req!r} already exists")
        slot = self.slots.allocate()
        self.lengths[req] = 0
        self.slot_of[req] = slot
        for g in self.groups:
            g.new_table(req)
        for states in self._state_entries.values():
            states[slot].zero_()

    def free_request(self, req) -> None:
        if req not in self.lengths:
            raise KeyError(f"request {req!r} is not held")
        for g in self.groups:
            g.allocator.free([p for p in g.drop_table(req) if p != RELEASED])
        self.slots.free([self.slot_of.pop(req)])
        del self.lengths[req]

    def extra_pages_needed(self, req, new_tokens: int) -> int:
        """Pages the tightest group must still find to take ``new_tokens`` more tokens of ``req``."""
        length = self.lengths[req]
        return max((g.extra_pages(req, length, new_tokens) for g in self.groups), default=0)

    def reserve(self, entries: list[tuple[object, int]]) -> None:
        """Find pages for ``new_tokens`` more tokens of each ``(request, new_tokens)``.
        Atomic: raises ``OutOfPages`` before any state changes."""
        seen = set()
        for req, n in entries:
            if req not in self.lengths:
                raise KeyError(f"request {req!r} is not held")
            if req in seen:
                raise ValueError(f"request {req!r} appears twice in one step")
            if n < 1:
                raise ValueError(f"request {req!r} brings {n} tokens")
            seen.add(req)
        for g in self.groups:
            need = sum(g.extra_pages(req, self.lengths[req], n) for req, n in entries)
            if need > g.allocator.num_free:
                raise OutOfPages(f"step needs {need} pages, {g.allocator.num_free} free of {g.num_pages}")
        for g in self.groups:
            for req, n in entries:
                for _ in range(g.extra_pages(req, self.lengths[req], n)):
                    g.append_page(req, g.allocator.allocate())

    def commit(self, entries: list[tuple[object, int]]) -> None:
        """The step ran: advance lengths and give back the pages that windows have passed."""
        for req, n in entries:
            self.lengths[req] += n
            length = self.lengths[req]
            for g in self.groups:
                if g.spec.window is None:
                    continue
                table = g.tables[req]
                stale = [i for i in range(min(g.first_needed_page(length), len(table))) if table[i] != RELEASED]
                g.allocator.free([table[i] for i in stale])
                for i in stale:
                    g.release_page(req, i)

    def reset(self) -> None:
        for req in list(self.lengths):
            self.free_request(req)

    def check(self) -> None:
        """Invariants: no page lost, held twice or freed twice; every held page is in exactly one table."""
        for g in self.groups:
            g.allocator.check()
            held = [p for t in g.tables.values() for p in t if p != RELEASED]
            assert len(held) == len(set(held)), "a page is in two tables"
            assert set(held) == g.allocator._used, "tables and allocator disagree"
            assert g.tables.keys() == g._rows.keys()
            for req, t in g.tables.items():
                assert g.row(req).tolist() == [max(p, 0) for p in t], "a table and its array disagree"
        self.slots.check()
        assert set(self.slot_of.values()) == self.slots._used

    # ------------------------------------------------------------------ views of a step
    def step_tables(self, entries: list[tuple[object, int]]):
        """Host arrays for a reserved step: per group a page table ``[R, width]`` and the slot of
        every new token; and the state slot of every request."""
        out = []
        starts = np.asarray([self.lengths[req] for req, _ in entries], dtype=np.int64)
        counts = np.asarray([n for _, n in entries], dtype=np.int64)
        # position of every new token, request by request, and the row of `table` it belongs to
        owner = np.repeat(np.arange(len(entries)), counts)
        first = np.cumsum(counts) - counts
        pos = np.arange(int(counts.sum())) - np.repeat(first, counts) + np.repeat(starts, counts)
        for g in self.groups:
            rows = [g.row(req) for req, _ in entries]
            width = max(1, max(r.shape[0] for r in rows))
            table = np.zeros((len(entries), width), dtype=np.int32)
            for r, row in enumerate(rows):
                table[r, : row.shape[0]] = row
            slots = table[owner, pos // g.page_size].astype(np.int64) * g.page_size + pos % g.page_size
            out.append((table, slots.astype(np.int32)))
        state_slots = np.asarray([self.slot_of[req] for req, _ in entries], dtype=np.int32)
        return out, state_slots

    def views(self, group_tensors, state_slots: torch.Tensor, host_slots: list[int]) -> list:
        """One view per entry of the order, from the device copies of ``step_tables``'s arrays."""
        views: list = []
        for i, run in enumerate(self.schedule):
            src = i if run.cache_of is None else run.cache_of
            if src in self._entry_group:
                g, plane = self._entry_group[src]
                group = self.groups[g]
                table, slot_map = group_tensors[g]
                views.append(PagedKVView(group.pool[plane], table, slot_map, group.page_size, group.spec))
            elif src in self._state_entries:
                views.append(StateView(self._state_entries[src], state_slots, host_slots))
            else:
                views.append(None)
        return views
